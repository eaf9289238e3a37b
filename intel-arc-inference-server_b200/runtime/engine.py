"""Single-GPU engine: sequence slots, paged KV, control block, CUDA-graph replay.

The role of the reference's ``runtime::Engine`` (src/runtime/engine.h:52-690):
ingest a prompt, replay decode steps, verify draft rows, keep per-sequence
state in slots.  Here a "captured command list" is a ``torch.cuda.CUDAGraph``
per (row count, advance) pair; the device control block carries positions and
tokens from one replay to the next, so plain decode needs no host write between
steps.  Host-side bookkeeping (sequence lengths, page tables) is deterministic
from the number of steps, so the host never reads the device to know where a
sequence is.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..models.config import ModelConfig
from ..models.decoder import DecoderModel, KVCache, attn_splits
from ..models.weights import ModelWeights
from ..ops import lib as K
from ..utils.staging import Staged
from .kv_pool import KvPool

PAGE = 16


@dataclass
class Row:
    slot: int
    pos: int
    token: int
    block: int = 0      # 1: a block drafter's row, which attends to all positions of its request's rows in the step


class Engine:
    def __init__(self, weights: ModelWeights, max_seqs: int = 1, max_len: int = 4096, kv_dtype: str = "bf16",
                 max_rows: int = 64, use_graphs: bool = True, int8_head: bool = False, num_pages: Optional[int] = None,
                 nsplit_attn: int = 0, prefill_backend: str = "auto", tp=None, nccl=None,
                 extra_kv_layers: int = 0):
        """``tp``: wires of a tensor-parallel group; every rank builds the same Engine over its weight shard and
        is driven with the same calls (same rows, same order) -- the step's kernels do the crossings."""
        self.cfg = cfg = weights.cfg
        self.tp = tp if tp is not None and tp.world > 1 else None
        self.device = weights.embed.device
        self.max_seqs, self.max_len, self.max_rows = max_seqs, max_len, max_rows
        self.max_blocks = (max_len + PAGE - 1) // PAGE
        if num_pages is None:
            num_pages = max_seqs * self.max_blocks + 1
        if not nsplit_attn:     # sized for contexts near the longest one the engine holds
            nsplit_attn = attn_splits(cfg.n_kv_heads, max_len)
        self.model = DecoderModel(weights, max_rows=max_rows, max_pos=max_len, nsplit_attn=nsplit_attn,
                                  int8_head=int8_head, tp=self.tp, nccl=nccl)
        self.kv = KVCache(cfg, cfg.n_layers + extra_kv_layers, num_pages, self.device, kv_dtype,   # + draft-head layers
                          n_slots=max_seqs)
        self.kv_dtype = kv_dtype
        self.pool = KvPool(num_pages, max_seqs, self.max_blocks)
        self.ctrl = torch.zeros(K.CTRL_WORDS, dtype=torch.int32, device=self.device)
        # pinned staging rings: a queued non-blocking copy may run long after the host moved on (see utils/staging.py)
        self.ctrl_stage = Staged((K.CTRL_WORDS,), torch.int32)
        self.table_stage = Staged((self.max_blocks,), torch.int32, depth=4)
        self.out_host = torch.zeros(K.CTRL_WORDS, dtype=torch.int32).pin_memory()
        self.block_table = torch.zeros(max_seqs, self.max_blocks, dtype=torch.int32, device=self.device)
        self.seq_len = [0] * max_seqs
        self._gdn_snap = None       # (rows, {slot: state before them}) of the last forward_rows step of a hybrid model
        self.use_graphs = use_graphs
        self.graphs: Dict[Tuple[int, bool, bool], torch.cuda.CUDAGraph] = {}
        self._one_request = False   # the rows last written are consecutive positions of one request
        self.prefill_backend = prefill_backend
        self._prefill = None
        self.steps_replayed = 0
        self.last_prefill_row = 0
        # failure latch (the reference's TpEngine keeps `broken_` until reset(): src/runtime/tp_engine.cc:203-256,418-424)
        self.broken: Optional[str] = None
        if self.device.type == "cuda":
            K.arm_failure_word()
        import os
        if os.environ.get("B200SERVE_AUDIT", "0") == "1":     # every buffer has a planner entry (see buffer_registry.py)
            from .buffer_registry import audit
            audit(self.model.buf, self.kv, cfg, kv_dtype, max_seqs)
        self.launches_per_step: Dict[Tuple[int, bool, bool], int] = {}

    def close(self):
        """Releases the cross-GPU buffers of a tensor-parallel engine (mapped peer memory)."""
        torch.cuda.synchronize(self.device)
        self.graphs.clear()
        if self._prefill is not None and hasattr(self._prefill, "close"):
            self._prefill.close()
        self._prefill = None
        if self.tp is not None:
            self.tp.close()
            self.tp = self.model.tp = None

    # ------------------------------------------------------------------ slots and pages
    def reset(self, slot: Optional[int] = None):
        slots = range(self.max_seqs) if slot is None else [slot]
        for s in slots:
            self.pool.release(s)
            self.seq_len[s] = 0
            self.kv.reset_slot(s)       # recurrent state of gated delta-net layers

    def truncate(self, slot: int, length: int):
        """Drop everything after ``length`` positions (rejected draft rows)."""
        assert length <= self.seq_len[slot]
        replay = None
        if length < self.seq_len[slot] and self.cfg.n_gdn_layers:
            # A recurrent state cannot be rewound.  The last multi-row step left a copy of the slot's state from
            # before its rows (the reference snapshots its GDN state the same way around verify rows): put it
            # back and run the rows that stay once more.
            snap = self._gdn_snap
            rows = [] if snap is None else [r for r in snap[0] if r.slot == slot]
            if not rows or slot not in snap[1] or length < rows[0].pos or self.seq_len[slot] != rows[-1].pos + 1:
                raise NotImplementedError("a gated delta-net layer's recurrent state can only be rewound to a position "
                                          "inside the last multi-row step (prefix reuse is not available for the "
                                          "hybrid family)")
            conv, state = snap[1][slot]
            self.kv.gdn_conv[:, slot].copy_(conv)
            self.kv.gdn_state[:, slot].copy_(state)
            replay = [r for r in rows if r.pos < length]
            self.seq_len[slot] = rows[0].pos
            self._gdn_snap = None
        self.seq_len[slot] = min(self.seq_len[slot], length)
        self.pool.truncate(slot, (length + PAGE - 1) // PAGE)
        if replay:
            self.forward_rows(replay, advance=False, read=False)
            self._gdn_snap = None       # one rewind per step

    def _ensure_pages(self, slot: int, upto_len: int):
        if upto_len > self.max_len:
            raise ValueError(f"sequence of {upto_len} positions exceeds max_len {self.max_len}")
        want = (upto_len + PAGE - 1) // PAGE
        try:
            changed = self.pool.ensure(slot, want)
        except MemoryError:
            # the pool is short of pages: whoever keeps finished sessions and cached blocks on the device (the prefix
            # store) gives some back -- cached blocks go to the host tier, idle sessions leave, least recently used
            # first -- and the request goes on; only when that does not cover it does the request fail
            hook = getattr(self, "on_pool_pressure", None)
            need = want - len(self.pool.table(slot))
            if hook is None or not hook(slot, need):
                raise
            changed = self.pool.ensure(slot, want)
        if changed:
            row = self.pool.table(slot)
            host = self.table_stage.begin()
            host[: len(row)] = torch.from_numpy(np.asarray(row, dtype=np.int32))
            self.table_stage.push(self.block_table[slot, : len(row)], host[: len(row)])

    def _write_rows(self, rows: Sequence[Row]):
        m = len(rows)
        c = self.ctrl_stage.begin()
        c[K.CTRL_N_ROWS] = m
        for i, r in enumerate(rows):
            c[K.CTRL_ROW_REQ + i] = r.slot
            c[K.CTRL_ROW_POS + i] = r.pos
            c[K.CTRL_CUR_TOKEN + i] = r.token
            c[K.CTRL_ROW_BLOCK + i] = r.block
        self._one_request = all(r.slot == rows[0].slot and r.pos == rows[0].pos + i for i, r in enumerate(rows))
        self.ctrl_stage.push(self.ctrl)

    # ------------------------------------------------------------------ session snapshots
    def save_kv(self, slot: int, begin: int, end: int) -> dict:
        """The KV of positions ``[begin, end)`` of ``slot`` (whole pages: both multiples of 16, or ``end`` the
        sequence length) as pinned host tensors in page order -- the reference's ``save_kv`` (src/runtime/engine.h:170-209);
        the layout is ``[layer][page][kv head][16][head dim]`` per tensor and does not depend on the parallel mode."""
        if begin % PAGE or (end % PAGE and end != self.seq_len[slot]) or not 0 <= begin <= end <= self.seq_len[slot]:
            raise ValueError("save_kv takes whole pages inside the sequence")
        if self.kv.gdn_state is not None and end != self.seq_len[slot]:
            raise ValueError("save_kv: a hybrid model's snapshot ends at the sequence end (the recurrent state of its "
                             "gated delta-net layers is the one after the last position)")
        pages = list(self.pool.table(slot))[begin // PAGE: (end + PAGE - 1) // PAGE]
        idx = torch.as_tensor(pages, device=self.device, dtype=torch.int64)
        tensors = {"k": self.kv.k, "v": self.kv.v}
        if self.kv.kv_int8:
            tensors.update({"k_scale": self.kv.k_scale, "v_scale": self.kv.v_scale})
        out = {"begin": begin, "end": end, "kv_dtype": self.kv_dtype}
        if self.kv.gdn_state is not None:      # the recurrent state and the convolution window after position end - 1
            for name, t in (("gdn_conv", self.kv.gdn_conv), ("gdn_state", self.kv.gdn_state)):
                host = torch.empty((t.shape[0],) + tuple(t.shape[2:]), dtype=t.dtype).pin_memory()
                host.copy_(t[:, slot], non_blocking=True)
                out[name] = host
        for name, t in tensors.items():
            host = torch.empty((t.shape[0], len(pages)) + tuple(t.shape[2:]), dtype=t.dtype).pin_memory()
            host.copy_(t.index_select(1, idx), non_blocking=True)
            out[name] = host
        torch.cuda.current_stream().synchronize()
        return out

    def load_kv(self, slot: int, blob: dict):
        """Puts a ``save_kv`` blob back at its positions; the slot must hold exactly ``blob["begin"]`` positions."""
        begin, end = blob["begin"], blob["end"]
        if blob["kv_dtype"] != self.kv_dtype or self.seq_len[slot] != begin:
            raise ValueError("load_kv: the slot must end where the blob begins and use the same KV form")
        self._ensure_pages(slot, end)
        pages = list(self.pool.table(slot))[begin // PAGE: (end + PAGE - 1) // PAGE]
        idx = torch.as_tensor(pages, device=self.device, dtype=torch.int64)
        tensors = {"k": self.kv.k, "v": self.kv.v}
        if self.kv.kv_int8:
            tensors.update({"k_scale": self.kv.k_scale, "v_scale": self.kv.v_scale})
        for name, t in tensors.items():
            t.index_copy_(1, idx, blob[name].to(self.device, non_blocking=True))
        if self.kv.gdn_state is not None:
            if "gdn_state" not in blob:
                raise ValueError("load_kv: the blob holds no recurrent state for this hybrid model")
            self.kv.gdn_conv[:, slot].copy_(blob["gdn_conv"].to(self.device, non_blocking=True))
            self.kv.gdn_state[:, slot].copy_(blob["gdn_state"].to(self.device, non_blocking=True))
            self._gdn_snap = None
        self.seq_len[slot] = end

    # ------------------------------------------------------------------ running a step
    def _enqueue(self, m: int, advance: bool):
        self.model.step_rows(m, self.ctrl, self.block_table, self.max_blocks, self.kv, advance,
                             one_request=self._one_request)

    def _run(self, m: int, advance: bool):
        if not self.use_graphs:
            self._enqueue(m, advance)
            return
        key = (m, advance, self._one_request)
        g = self.graphs.get(key)
        if g is None:
            # warm-up outside capture (sets function attributes, allocates split-K scratch), then
            # restore the control block the warm-up advanced
            saved = self.ctrl.clone()
            # KV appends repeat harmlessly; a gated delta-net layer's recurrent update does not: its state is put back
            saved_gdn = None if self.kv.gdn_state is None else (self.kv.gdn_conv.clone(), self.kv.gdn_state.clone())
            n0 = K.launch_count
            self._enqueue(m, advance)
            self.launches_per_step[key] = K.launch_count - n0
            torch.cuda.current_stream().synchronize()
            self.ctrl.copy_(saved)
            if saved_gdn is not None:
                self.kv.gdn_conv.copy_(saved_gdn[0])
                self.kv.gdn_state.copy_(saved_gdn[1])
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._enqueue(m, advance)
            self.ctrl.copy_(saved)
            self.graphs[key] = g
        g.replay()
        self.steps_replayed += 1

    def launches(self, m: int, advance: bool = True) -> int:
        """Kernel launches of one captured step of ``m`` rows (0 before the first such step)."""
        return max((v for (mm, adv, _), v in self.launches_per_step.items() if mm == m and adv == advance), default=0)

    # ------------------------------------------------------------------ failure latch
    def require_ok(self):
        if self.broken is not None:
            raise K.KernelError(f"engine is latched after a failed step ({self.broken}); call reset_failure()")

    def check_failed(self, what: str = "step"):
        """After a synchronize: if any kernel's bounded wait ran out during the work just finished, latch the engine and
        raise an error that names the unit, the code and where it gave up (rank, tile).  The step's outputs are garbage."""
        if not K.failed_fast():
            return
        st = K.status()
        rank = self.tp.rank if self.tp is not None else (self.model.nccl[0] if self.model.nccl is not None else 0)
        self.broken = f"{what} on rank {rank}: " + ", ".join(
            f"{u}: code {v['code']} detail {v['detail']:#x} ({v['count']} waits)" for u, v in st.items())
        raise K.KernelError(f"device kernels gave up on a bounded wait during {self.broken}")

    def reset_failure(self):
        """Clears the status words, the whole-step kernel's barrier words and the wires' flags and call counters, and
        releases the latch.  Under tensor parallelism every rank must call it before the next step."""
        torch.cuda.synchronize(self.device)
        K.status_clear()
        self.model.mega_reset()
        if self.tp is not None:
            self.tp.reset()
        torch.cuda.synchronize(self.device)
        self.broken = None

    def _read_out(self, m: int) -> List[int]:
        self.out_host.copy_(self.ctrl, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.check_failed()
        return self.out_host[K.CTRL_OUT_TOKEN: K.CTRL_OUT_TOKEN + m].tolist()

    # ------------------------------------------------------------------ public API
    def forward_rows(self, rows: Sequence[Row], advance: bool = False, read: bool = True):
        """Run arbitrary rows (verify, batched decode, chunked ingest). KV of each row is appended."""
        self.require_ok()
        for r in rows:
            self._ensure_pages(r.slot, r.pos + 1)
        self._gdn_snap = None
        if self.kv.gdn_state is not None:
            slots = sorted({r.slot for r in rows})
            self._gdn_snap = (list(rows), {s: (self.kv.gdn_conv[:, s].clone(), self.kv.gdn_state[:, s].clone())
                                           for s in slots})
        self._write_rows(rows)
        self._run(len(rows), advance)
        for r in rows:
            self.seq_len[r.slot] = max(self.seq_len[r.slot], r.pos + 1)
        return self._read_out(len(rows)) if read else None

    def logits(self, m: int) -> torch.Tensor:
        """fp32 logits of the last step's rows (device tensor view)."""
        return self.model.buf.logits[:m]

    def prefill(self, slot: int, ids: Sequence[int], chunk: Optional[int] = None) -> int:
        """Ingest ``ids`` after the slot's current length; returns the greedy next token."""
        self.require_ok()
        ids = list(ids)
        if self._use_tc_prefill(len(ids)):
            if self._prefill is None:
                if self.tp is not None:
                    from ..parallel.tp_prefill import TpPrefillRunner
                    self._prefill = TpPrefillRunner(self)
                elif self.model.nccl is not None:
                    from ..parallel.tp_prefill import NcclPrefillRunner
                    self._prefill = NcclPrefillRunner(self, self.model.nccl[2])
                else:
                    from .prefill import PrefillRunner
                    self._prefill = PrefillRunner(self)
            self.last_prefill_row = 0      # row of model.buf.logits that holds the prompt's last position
            tok = self._prefill.run(slot, ids, chunk)
            self.check_failed("prompt pass")
            return tok
        start = self.seq_len[slot]
        out = None
        for c0 in range(0, len(ids), self.max_rows):
            part = ids[c0: c0 + self.max_rows]
            rows = [Row(slot, start + c0 + i, t) for i, t in enumerate(part)]
            last = c0 + self.max_rows >= len(ids)
            out = self.forward_rows(rows, advance=False, read=last)
            hook = getattr(self, "on_chunk_hidden", None)
            if hook is not None:
                hook(None, slot, part, start + c0, self.model.buf.resid[: len(part)])
        self.last_prefill_row = len(out) - 1
        return out[-1]

    def _use_tc_prefill(self, n: int) -> bool:
        """Prompt chunks longer than the row kernels take go through the tcgen05 path when the shape
        has one (head size 128, bf16 KV, dense FFN or MoE with a grouped path)."""
        if self.prefill_backend == "rows" or n <= self.max_rows:
            return False
        if self.cfg.n_gdn_layers and (self.kv.kv_int8 or self.tp is not None or self.model.nccl is not None):
            return False        # hybrid models: the layer-major int8-KV pass and the parallel runners know no GDN layers
        # an int8 KV cache: the one-GPU runner's layer-major pass, or the tensor-parallel runner's bf16 scratch of
        # the request; the NCCL comparison build has neither
        ok = self.cfg.head_dim == 128 and (not self.kv.kv_int8 or self.model.nccl is None)
        if not ok and self.prefill_backend != "auto":
            raise ValueError(f"prefill backend {self.prefill_backend!r} needs head_dim 128 (and a bf16 KV cache under "
                             "tensor parallelism)")
        return ok

    def decode_begin(self, slots: Sequence[int], tokens: Sequence[int]):
        """Arm plain decode: one row per slot, starting with ``tokens`` at each slot's current length."""
        rows = [Row(s, self.seq_len[s], t) for s, t in zip(slots, tokens)]
        self._write_rows(rows)
        self._decode_slots = list(slots)

    def decode_step(self, read: bool = True):
        """One replay of the armed decode rows; the device advances tokens and positions itself."""
        self.require_ok()
        slots = self._decode_slots
        for s in slots:
            self._ensure_pages(s, self.seq_len[s] + 1)
        self._run(len(slots), True)
        for s in slots:
            self.seq_len[s] += 1
        return self._read_out(len(slots)) if read else None

    def generate(self, ids: Sequence[int], n_new: int, slot: int = 0) -> List[int]:
        """Greedy: prefill ``ids`` then ``n_new`` tokens; returns the new tokens."""
        self.reset(slot)
        first = self.prefill(slot, ids)
        out = [first]
        if n_new > 1:
            self.decode_begin([slot], [first])
            for _ in range(n_new - 1):
                out.append(self.decode_step()[0])
        return out
