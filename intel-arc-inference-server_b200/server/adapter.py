"""EngineIface over the single-GPU engine: host-driven rows, sampling on the device (``sample``) with the logits
read-back for the host sampler as the fallback.

The role of the reference's ``EngineAdapter`` / ``SlotsEngine`` (src/cli/serve_adapters.h:153-470,
src/cli/slots_engine.h:1-60): a lone greedy row replays the captured decode graph; several rows
(several slots, or a pending token plus draft rows) run as one multi-row step.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..ops import lib as K
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
        self._samp = None       # (pinned host words, device words, device out) of the device sampler

    def reset(self, slot):
        self.e.reset(slot)

    def length(self, slot):
        return self.e.seq_len[slot]

    def truncate(self, slot, length):
        self.e.truncate(slot, length)

    def kv_form(self):
        return self.e.kv_dtype

    def reset_failure(self):
        """After a step failed on a bounded wait: clear the device status and release the engine's latch."""
        self.e.reset_failure()

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

    def logits_shard(self, slot, row=0):
        """(first vocabulary id, fp32 values) of the part of the row's logits that this rank holds: the whole row
        on one GPU, this rank's slice of the vocabulary under tensor parallelism, nothing on a pipeline stage that
        does not run the head."""
        m = self.e.model
        if not getattr(self.e, "last", True):      # a pipeline stage before the last one: the head did not run here
            return 0, np.zeros(0, dtype=np.float32)
        off = m.vocab_offset if self.e.tp is not None else (getattr(m, "vocab_offset_nccl", 0) if m.nccl is not None else 0)
        part = np.asarray(self.logits(slot, row))
        return int(off), part[: max(0, min(len(part), self.vocab_size - off))]

    # ------------------------------------------------------------------ sampling on the device
    _SAMP_HEAD = 8      # parameter words before the history ids

    def sample(self, slot, row, temperature, top_k, top_p, seed, penalty=1.0, history=()) -> Optional[int]:
        """Draws the row's token with the device sampler (ops/csrc/sampler.cu: the host sampler's rule and random
        number, so the token is the one ``native.sample`` would return) and reads back 8 bytes instead of the
        row's logits.  ``None``: the caller samples on the host (sharded logits, or a filtered set the kernel
        does not decide)."""
        if self.e.tp is not None or self.e.model.nccl is not None:
            return None
        cap = self.e.max_len + 64
        if self._samp is None:
            host = torch.zeros(self._SAMP_HEAD + cap, dtype=torch.int32).pin_memory()
            dev = torch.zeros(self._SAMP_HEAD + cap, dtype=torch.int32, device=self.e.device)
            out = torch.zeros(2, dtype=torch.int32, device=self.e.device)
            self._samp = (host, dev, out)
        host, dev, out = self._samp
        hist = list(history)[-cap:] if penalty != 1.0 else []
        hf = host[:4].view(torch.float32)
        hf[0], hf[2], hf[3] = float(temperature), float(top_p), float(penalty)
        host[1] = int(top_k)
        host[4:6].view(torch.int64)[0] = int(seed) - (1 << 64) if int(seed) >= (1 << 63) else int(seed)
        host[6] = len(hist)
        if hist:
            host[self._SAMP_HEAD: self._SAMP_HEAD + len(hist)] = torch.tensor(hist, dtype=torch.int32)
        n = self._SAMP_HEAD + len(hist)
        dev[:n].copy_(host[:n], non_blocking=True)
        lg = self.e.logits(max(r.stop for r in self._rows_of.values()))[self._rows_of[slot][row]: self._rows_of[slot][row] + 1]
        df = dev[:4].view(torch.float32)
        K.sample_rows(lg, 1, self.vocab_size, df[0:1], dev[1:2], df[2:3], dev[4:6], out[0:1], out[1:2],
                      penalty=df[3:4] if hist else None, hist=dev[self._SAMP_HEAD:].view(1, -1) if hist else None,
                      hist_len=dev[6:7] if hist else None)
        tok, status = out.tolist()
        return None if status != 0 else int(tok)
