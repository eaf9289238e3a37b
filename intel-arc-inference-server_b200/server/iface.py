"""Interfaces between the server and what it serves with.

The server is written against three small interfaces -- tokenizer, chat template, engine -- so it
can be exercised with mocks on a machine without a GPU, exactly the reference's arrangement
(src/server/deps.h:18-236 ``TokIface / TemplateIface / EngineIface``; tests/server/mock.h).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np


class EngineIface:
    """What the server needs from an engine.  Slots are independent sequences."""
    vocab_size: int = 0
    max_len: int = 0
    max_seqs: int = 1
    eos_ids: Sequence[int] = ()

    def reset(self, slot: int) -> None: ...
    def length(self, slot: int) -> int: ...
    def truncate(self, slot: int, length: int) -> None: ...
    def prefill(self, slot: int, ids: Sequence[int]) -> int:
        """Ingest ``ids`` after the slot's current length; returns the greedy next token."""
    def step(self, rows: Dict[int, List[int]]) -> Dict[int, List[int]]:
        """For every slot, run its row tokens at consecutive positions (the first is the pending token,
        the rest are drafts); returns the arg-max after each row."""
    def logits(self, slot: int, row: int = 0) -> np.ndarray:
        """fp32 logits of ``row`` of ``slot`` from the last prefill / step (for host sampling)."""
    def kv_form(self) -> str:
        return "bf16"


class MockEngine(EngineIface):
    """Deterministic stand-in: the next token is a hash of the sequence so far.  ``script`` overrides the
    continuation of a given prompt (to produce tool calls, stop strings, EOS)."""

    def __init__(self, vocab_size=1000, max_len=4096, max_seqs=4, eos_ids=(2,), script=None, step_delay=0.0):
        self.vocab_size, self.max_len, self.max_seqs, self.eos_ids = vocab_size, max_len, max_seqs, tuple(eos_ids)
        self.seqs: List[List[int]] = [[] for _ in range(max_seqs)]
        self.script = script or {}
        self._logits: Dict[int, List[np.ndarray]] = {}
        self.prefilled_tokens = 0
        self.steps = 0
        self.step_delay = step_delay
        self.fail_slots = set()

    def reset(self, slot):
        self.seqs[slot] = []

    def length(self, slot):
        return len(self.seqs[slot])

    def truncate(self, slot, length):
        del self.seqs[slot][length:]

    def _next(self, seq: List[int]) -> int:
        for prompt, cont in self.script.items():
            n = len(prompt)
            if tuple(seq[:n]) == prompt and len(seq) - n < len(cont):
                return cont[len(seq) - n]
        h = 1469598103934665603
        for t in seq[-8:]:
            h = ((h ^ (t + 1)) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
        return 3 + h % (self.vocab_size - 3)

    def _row(self, tok: int) -> np.ndarray:
        v = np.full(self.vocab_size, -5.0, dtype=np.float32)
        v[tok] = 5.0
        v[(tok + 1) % self.vocab_size] = 4.0
        return v

    def prefill(self, slot, ids):
        if len(self.seqs[slot]) + len(ids) > self.max_len:
            raise ValueError("prompt exceeds max_len")
        self.seqs[slot].extend(ids)
        self.prefilled_tokens += len(ids)
        t = self._next(self.seqs[slot])
        self._logits[slot] = [self._row(t)]
        return t

    def step(self, rows):
        import time
        if self.step_delay:
            time.sleep(self.step_delay)
        self.steps += 1
        out = {}
        for slot, toks in rows.items():
            if slot in self.fail_slots:
                raise RuntimeError(f"slot {slot} failed")
            res, lg = [], []
            for t in toks:
                self.seqs[slot].append(t)
                n = self._next(self.seqs[slot])
                res.append(n)
                lg.append(self._row(n))
            out[slot] = res
            self._logits[slot] = lg
        return out

    def logits(self, slot, row=0):
        return self._logits[slot][row]


class TokIface:
    def encode(self, text: str) -> List[int]: ...
    def decode(self, ids: Sequence[int]) -> str: ...
    def streamer(self): ...


class ByteTok(TokIface):
    """Mock tokenizer: one id per UTF-8 byte (+3), ids 0..2 are specials (pad, bos, eos).  A model whose
    vocabulary is larger than 259 (every preset with random weights) emits ids that are no byte: they fold onto
    the byte range (``(id - 3) % 256``) so that serving a preset streams something instead of failing."""

    def encode(self, text):
        return [b + 3 for b in text.encode("utf-8")]

    def decode(self, ids):
        return bytes((i - 3) % 256 for i in ids if i >= 3).decode("utf-8", "replace")

    def streamer(self):
        tok = self

        class _S:
            def __init__(self):
                self.buf = b""

            def push(self, i):
                if i < 3:
                    return b""
                self.buf += bytes([(i - 3) % 256])
                # hold an unfinished UTF-8 character
                for back in range(1, min(4, len(self.buf)) + 1):
                    c = self.buf[-back]
                    if c & 0xC0 == 0x80:
                        continue
                    need = 1 if c < 0x80 else 2 if c & 0xE0 == 0xC0 else 3 if c & 0xF0 == 0xE0 else 4
                    cut = len(self.buf) - back if need > back else len(self.buf)
                    out, self.buf = self.buf[:cut], self.buf[cut:]
                    return out
                return b""

            def finish(self):
                out, self.buf = self.buf, b""
                return out
        return _S()


class NativeTok(TokIface):
    """The native byte-level BPE tokenizer behind the interface."""

    def __init__(self, path: str):
        from ..native import host as H
        self.H = H
        self.tok = H.Tokenizer.from_file(path)

    def encode(self, text):
        return list(self.tok.encode(text))

    def decode(self, ids):
        return self.tok.decode(list(ids), True).decode("utf-8", "replace")

    def streamer(self):
        return self.H.Streamer(self.tok, True)

    def token_to_id(self, s):
        return self.tok.token_to_id(s)
