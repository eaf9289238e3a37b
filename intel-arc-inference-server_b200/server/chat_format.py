"""How the server reads a model's chat requests and outputs: the per-model choice behind one ``Server``.

The serve CLI picks it from ``config.json``'s ``model_type``; the request path asks the format, never the model
name.  The role of the reference's ``server::ChatFormat`` (src/server/chat_format.h:32-65).

  qwen      (anything not listed) the template reads ``enable_thinking`` only; the output opens with reasoning
            when the prompt ends in ``<think>``; tool calls are Qwen XML.
  kolibri   (``model_type`` kolibri1) ChatML; the template also reads the request's ``chat_template_kwargs``
            (``reasoning_effort`` of seven levels, ``enable_thinking``, ``preserve_thinking``) and the OpenAI
            top-level ``reasoning_effort``; the MODEL opens its reasoning with ``<think>`` (the prompt never ends in
            it), so reasoning is keyed on the output; tool calls are hermes JSON in ``<tool_call>``; a message whose
            content is a list of text parts reaches the template as one string joined with newlines.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

EFFORTS = ("none", "minimal", "low", "medium", "high", "xhigh", "max")
THINK_OPEN = "<think>"


@dataclass(frozen=True)
class ChatFormat:
    kind: str = "qwen"

    @staticmethod
    def for_model_type(model_type: Optional[str]) -> "ChatFormat":
        return ChatFormat("kolibri") if model_type == "kolibri1" else ChatFormat("qwen")

    # ---- what the format switches
    @property
    def tool_format(self) -> str:
        return "hermes" if self.kind == "kolibri" else "qwen_xml"

    @property
    def template_kwargs(self) -> bool:
        """The request's chat_template_kwargs reach the template beside enable_thinking."""
        return self.kind == "kolibri"

    @property
    def string_content(self) -> bool:
        return self.kind == "kolibri"

    @property
    def reasoning_in_output(self) -> bool:
        """The model itself opens its reasoning with <think>: the output parser looks at the output, not the prompt."""
        return self.kind == "kolibri"

    # ---- requests
    def template_messages(self, messages: List[dict]) -> List[dict]:
        """The messages as this format's template reads them: with ``string_content`` a content that is a list of text
        parts becomes their texts joined with newlines; otherwise unchanged."""
        if not self.string_content:
            return messages
        out = []
        for m in messages:
            c = m.get("content") if isinstance(m, dict) else None
            if isinstance(c, list):
                texts = [p.get("text", "") for p in c if isinstance(p, dict) and p.get("type", "text") == "text"]
                m = dict(m, content="\n".join(texts))
            out.append(m)
        return out

    def check_template_kwargs(self, kwargs: Optional[dict]):
        """A bad value is the client's error (a 400): raises ``ValueError`` naming the field."""
        if not kwargs or not self.template_kwargs:
            return
        eff = kwargs.get("reasoning_effort")
        if eff is not None and eff not in EFFORTS:
            raise ValueError(f"chat_template_kwargs.reasoning_effort must be one of {', '.join(EFFORTS)} or null")
        for name in ("preserve_thinking", "enable_thinking"):
            if name in kwargs and not isinstance(kwargs[name], bool):
                raise ValueError(f"chat_template_kwargs.{name} must be a boolean")

    def request_template_kwargs(self, kwargs: Optional[dict]) -> dict:
        """The kwargs this format's template gets (the request's chat_template_kwargs with the OpenAI top-level
        ``reasoning_effort`` already folded in by the request parser).  Formats without template kwargs keep
        ``enable_thinking`` alone, as their templates read nothing else."""
        kwargs = dict(kwargs or {})
        if self.template_kwargs:
            return kwargs
        return {k: v for k, v in kwargs.items() if k == "enable_thinking"}


class OutputOpening:
    """Decides, for a format whose model opens its own reasoning, whether the output starts with ``<think>``: holds
    back the first characters until they can no longer be a prefix of the tag, then hands everything to the parser
    it creates (in the reasoning state when the tag was there, the tag itself dropped)."""

    def __init__(self, make_parser):
        self._make, self._held, self._parser = make_parser, "", None

    def push(self, text: str):
        if self._parser is not None:
            return self._parser.push(text)
        self._held += text
        probe = self._held.lstrip()
        if len(probe) < len(THINK_OPEN) and THINK_OPEN.startswith(probe):
            return []                                   # may still become the tag
        if probe.startswith(THINK_OPEN):
            self._parser = self._make(True)
            return self._parser.push(probe[len(THINK_OPEN):])
        self._parser = self._make(False)
        return self._parser.push(self._held)

    def finish(self):
        if self._parser is None:                        # the output ended inside a possible tag: it was plain text
            self._parser = self._make(False)
            out = self._parser.push(self._held)
            return list(out) + list(self._parser.finish())
        return self._parser.finish()
