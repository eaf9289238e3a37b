"""EngineIface over the single-GPU engine: host-driven rows, logits read-back for host sampling.

The role of the reference's ``EngineAdapter`` / ``SlotsEngine`` (src/cli/serve_adapters.h:153-470,
src/cli/slots_engine.h:1-60): a lone greedy row replays the captured decode graph; several rows
(several slots, or a pending token plus draft rows) run as one multi-row step.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np
import torch

from ..runtime.engine import Engine, Row
from .iface import EngineIface


class EngineAdapter(EngineIface):
    def __init__(self, engine: Engine, eos_ids: Sequence[int] = ()):
        self.e = engine
        self.vocab_size = engine.cfg.vocab
        self.max_len = engine.max_len
        self.max_seqs = engine.max_seqs
        self.eos_ids = tuple(eos_ids)
        self._rows_of: Dict[int, range] = {}
        self._logits_host = None

    def reset(self, slot):
        self.e.reset(slot)

    def length(self, slot):
        return self.e.seq_len[slot]

    def truncate(self, slot, length):
        self.e.truncate(slot, length)

    def kv_form(self):
        return self.e.kv_dtype

    def prefill(self, slot, ids):
        tok = self.e.prefill(slot, list(ids))
        r = self.e.last_prefill_row
        self._rows_of = {slot: range(r, r + 1)}
        self._logits_host = None
        return tok

    def step(self, rows: Dict[int, List[int]]):
        flat, spans = [], {}
        for slot, toks in rows.items():
            base = self.e.seq_len[slot]
            spans[slot] = range(len(flat), len(flat) + len(toks))
            flat += [Row(slot, base + i, int(t)) for i, t in enumerate(toks)]
        out = self.e.forward_rows(flat, advance=False, read=True)
        self._rows_of = spans
        self._logits_host = None
        return {slot: [out[i] for i in span] for slot, span in spans.items()}

    def logits(self, slot, row=0):
        if self._logits_host is None:
            n = max(r.stop for r in self._rows_of.values())
            self._logits_host = self.e.logits(n).float().cpu().numpy()
        return self._logits_host[self._rows_of[slot][row]]
