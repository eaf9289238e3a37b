"""Chat template rendering.

A checkpoint's own ``chat_template`` (``tokenizer_config.json`` or ``chat_template.jinja``) is
rendered with jinja2 the way ``transformers`` does (ordered ``tojson``, ``raise_exception``,
``strftime_now``, keyword arguments from ``chat_template_kwargs``) -- the role of the
reference's minja wrapper (src/tokenizer/chat_template.h:12-47).  Without a template the
built-in ChatML format is used: ``<|im_start|>role\\ncontent<|im_end|>`` turns, a ``# Tools``
section with one JSON schema per line and the Qwen XML call syntax, ``<tool_response>`` blocks
for tool results, and a ``<think>`` opener (or an empty think block when thinking is off).
"""
from __future__ import annotations

import datetime
import json
import os
from typing import Any, Dict, List, Optional


def _tojson(value, ensure_ascii=False, indent=None, separators=None, sort_keys=False):
    return json.dumps(value, ensure_ascii=ensure_ascii, indent=indent, separators=separators, sort_keys=sort_keys)


class ChatTemplate:
    def __init__(self, source: Optional[str] = None, bos_token: str = "", eos_token: str = "<|im_end|>"):
        self.source = source
        self.bos_token, self.eos_token = bos_token, eos_token
        self._compiled = None
        if source:
            import jinja2
            from jinja2.sandbox import ImmutableSandboxedEnvironment

            def raise_exception(msg):
                raise jinja2.exceptions.TemplateError(msg)

            env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True,
                                                extensions=["jinja2.ext.loopcontrols"])
            env.filters["tojson"] = _tojson
            env.globals["raise_exception"] = raise_exception
            env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
            self._compiled = env.from_string(source)

    @staticmethod
    def from_snapshot(path: str) -> "ChatTemplate":
        src, bos, eos = None, "", "<|im_end|>"
        cfg_path = os.path.join(path, "tokenizer_config.json")
        if os.path.exists(cfg_path):
            with open(cfg_path) as f:
                cfg = json.load(f)
            src = cfg.get("chat_template")
            if isinstance(src, list):      # named templates: take "default"
                src = next((t["template"] for t in src if t.get("name") == "default"), src[0]["template"])

            def tok(v, d):
                return v.get("content", d) if isinstance(v, dict) else (v or d)
            bos, eos = tok(cfg.get("bos_token"), ""), tok(cfg.get("eos_token"), eos)
        jpath = os.path.join(path, "chat_template.jinja")
        if src is None and os.path.exists(jpath):
            with open(jpath) as f:
                src = f.read()
        return ChatTemplate(src, bos, eos)

    def thinking_opened(self, prompt: str) -> bool:
        """True when the rendered prompt ends inside an open ``<think>`` block."""
        tail = prompt.rstrip()
        return tail.endswith("<think>")

    def render(self, messages: List[Dict[str, Any]], tools: Optional[list] = None,
               add_generation_prompt: bool = True, **kwargs) -> str:
        if self._compiled is not None:
            return self._compiled.render(messages=messages, tools=tools, add_generation_prompt=add_generation_prompt,
                                         bos_token=self.bos_token, eos_token=self.eos_token, **kwargs)
        return self._builtin(messages, tools, add_generation_prompt, **kwargs)

    # ------------------------------------------------------------------ built-in ChatML
    @staticmethod
    def _content(m) -> str:
        c = m.get("content")
        if c is None:
            return ""
        if isinstance(c, list):    # OpenAI content parts: text parts only
            return "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type", "text") == "text")
        return str(c)

    def _builtin(self, messages, tools, add_generation_prompt, enable_thinking: bool = True, **_):
        out = []
        msgs = list(messages)
        system = ""
        if msgs and msgs[0].get("role") == "system":
            system = self._content(msgs.pop(0))
        if tools:
            parts = ["# Tools\n\nYou have access to the following functions:\n\n<tools>"]
            parts += [_tojson(t, sort_keys=True) for t in tools]
            parts.append("</tools>\n\nIf you choose to call a function ONLY reply in the following format with NO suffix:"
                         "\n\n<tool_call>\n<function=example_function_name>\n<parameter=example_parameter_1>\nvalue_1\n"
                         "</parameter>\n</function>\n</tool_call>")
            block = "\n".join(parts)
            system = block + ("\n\n" + system if system else "")
        if system:
            out.append(f"<|im_start|>system\n{system}<|im_end|>\n")
        i = 0
        while i < len(msgs):
            m = msgs[i]
            role = m.get("role")
            if role == "tool":
                body = []
                while i < len(msgs) and msgs[i].get("role") == "tool":
                    body.append(f"<tool_response>\n{self._content(msgs[i])}\n</tool_response>")
                    i += 1
                out.append("<|im_start|>user\n" + "\n".join(body) + "<|im_end|>\n")
                continue
            if role == "assistant":
                text = ""
                rc = m.get("reasoning_content")
                text += f"<think>\n{rc.strip()}\n</think>\n\n" if rc else "<think>\n\n</think>\n\n"
                text += self._content(m)
                for tc in m.get("tool_calls") or []:
                    fn = tc.get("function", tc)
                    args = fn.get("arguments", {})
                    if isinstance(args, str):
                        try:
                            args = json.loads(args)
                        except json.JSONDecodeError:
                            args = {}
                    if text and not text.endswith("\n\n"):
                        text += "\n\n"
                    text += f"<tool_call>\n<function={fn.get('name')}>\n"
                    for k, v in args.items():
                        val = v if isinstance(v, str) else _tojson(v)
                        text += f"<parameter={k}>\n{val}\n</parameter>\n"
                    text += "</function>\n</tool_call>"
                out.append(f"<|im_start|>assistant\n{text}<|im_end|>\n")
            else:
                out.append(f"<|im_start|>{role}\n{self._content(m)}<|im_end|>\n")
            i += 1
        if add_generation_prompt:
            out.append("<|im_start|>assistant\n" + ("<think>\n" if enable_thinking else "<think>\n\n</think>\n\n"))
        return "".join(out)
