"""Tensor-parallel prompt pass: sequence-parallel residual stream, fused collectives.

Every rank keeps the residual rows of ITS tokens of the chunk (contiguous blocks of ``rows_cap``
tokens).  Per layer:

  all-gather -> GEMM   qkv and gate‖up read the gathered, normalised activations from this GPU's own
                       memory (ordinary TMA); their producer waits tile by tile on arrival counters
                       that the row owners bump after pushing the rows over NVLink;
  GEMM -> reduce-scatter   o and down store their bf16 output tiles straight into the landing buffer
                       of the rank that owns the rows (coalesced peer stores from the tcgen05
                       epilogue) and count arrivals there;
  fold                 the owner adds the partial sums in rank order to its residual rows, applies
                       the next RMSNorm and pushes the normalised rows to every rank -- which is the
                       all-gather feeding the next GEMM.

No NCCL call and no library GEMM on this path.  ``NcclPrefillRunner`` is the comparison: cuBLAS
GEMMs (``torch.matmul``) with NCCL all-reduces after the row-parallel linears, residual stream
replicated.  The reference's two-card prompt pass crosses with copy-engine copies between chunk
pairs instead (src/runtime/prefill/tp_prefill.cc:5-46).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..ops import gemm as G
from ..ops import lib as K
from ..runtime.prefill import PrefillRunner
from .symm import Wire


class TpPrefillRunner(PrefillRunner):
    def __init__(self, engine, group=None, max_chunk: int = 4096):
        import torch.distributed as dist
        super().__init__(engine, max_chunk)
        self.group = group
        if self.backend not in ("bf16", "bf16-resident"):
            raise ValueError("the tensor-parallel prompt pass runs the bf16 GEMMs")
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        cfg, w = self.cfg, self.world
        h = cfg.hidden
        tiles = (max_chunk + 127) // 128
        self.tpr = (tiles + w - 1) // w              # m-tiles per owner
        self.rows_cap = self.tpr * 128
        nbytes = w * self.rows_cap * h * 2
        self.rs = Wire(nbytes, w * self.tpr, 0, group, self.dev)      # landing [src][rows_cap][h] bf16 + counters
        self.xw = Wire(nbytes, w * self.tpr, 0, group, self.dev)      # gathered activations + tile counters
        self.x_full = self.xw.buf.view(torch.bfloat16, 0, w * self.rows_cap * h).view(w * self.rows_cap, h)
        self.own = torch.zeros(self.rows_cap, h, dtype=torch.bfloat16, device=self.dev)   # this rank's residual rows
        self.done = torch.zeros(self.tpr, dtype=torch.int32, device=self.dev)
        self.ag_epoch = 0
        self._kv16 = None     # int8 KV cache: bf16 K / V of the request being ingested, all local layers (see run)

    def _fold(self, nsrc: int, arrivals: int, norm_w, c: int):
        K.rs_fold(self.rs, arrivals, nsrc, self.done, self.own, norm_w, self.cfg.rms_eps, self.xw, self.cfg.hidden,
                  self.tpr, c)
        self.ag_epoch += 1

    def chunk(self, slot: int, ids: List[int], pos0: int):
        eng, cfg, m = self.eng, self.cfg, self.eng.model
        c, h, w = len(ids), cfg.hidden, self.world
        eng._ensure_pages(slot, pos0 + c)
        ids_host = self.ids_stage.begin()
        ids_host[:c] = torch.as_tensor(ids, dtype=torch.int64)
        self.ids_stage.push(self.ids_dev[:c], ids_host[:c])
        lo = self.rank * self.rows_cap
        hi = min(c, lo + self.rows_cap)
        if hi > lo:
            torch.index_select(m.w.embed, 0, self.ids_dev[lo:hi], out=self.own[: hi - lo])
        layers = m.w.layers
        self._fold(0, 0, layers[0].input_norm, c)
        bt_row = eng.block_table[slot]
        xg = self.x_full[:c]
        for li, lw in enumerate(layers):
            qkv = self.qkv[:c]
            G.gemm_tp(xg, self._w_bf16(lw.qkv), qkv, G.EPI_F32, ag_cnt=self.xw.flags, ag_expect=128 * self.ag_epoch)
            if self._kv16 is None:
                kc, vc, ks, vs = eng.kv.layer(li)
                K.rope_append(qkv, 0, 1, c, None, eng.block_table, eng.max_blocks, m.cos_t, m.sin_t, cfg.n_q_heads,
                              cfg.n_kv_heads, cfg.head_dim, self.q, kc, vc, ks, vs, False, req=slot, pos0=pos0)
                K.attn_prefill(self.q, kc, vc, bt_row, self.attn, c, pos0, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim,
                               eng.kv.num_pages, eng.max_blocks, m.scale, window=m._window(li))
            else:       # the bf16 scratch of this request: identity page table, request 0
                k16, v16, tab16 = self._kv16
                K.rope_append(qkv, 0, 1, c, None, tab16, tab16.shape[1], m.cos_t, m.sin_t, cfg.n_q_heads,
                              cfg.n_kv_heads, cfg.head_dim, self.q, k16[li], v16[li], None, None, False, req=0, pos0=pos0)
                K.attn_prefill(self.q, k16[li], v16[li], tab16[0], self.attn, c, pos0, cfg.n_q_heads, cfg.n_kv_heads,
                               cfg.head_dim, k16.shape[1], tab16.shape[1], m.scale, window=m._window(li))
            arr = G.gemm_tp(self.attn[:c], self._w_bf16(lw.o), None, G.EPI_RS_PUSH, rs=self.rs, rs_tpr=self.tpr)
            self._fold(w, arr, lw.post_norm, c)
            act = self.act[:c, : cfg.ffn]
            G.gemm_tp(xg, self._w_bf16(lw.gate_up), act, G.EPI_SILU_MUL, ag_cnt=self.xw.flags,
                      ag_expect=128 * self.ag_epoch)
            arr = G.gemm_tp(act, self._w_bf16(lw.down), None, G.EPI_RS_PUSH, rs=self.rs, rs_tpr=self.tpr)
            nxt = layers[li + 1].input_norm if li + 1 < len(layers) else m.w.final_norm
            self._fold(w, arr, nxt, c)
        hook = getattr(eng, "on_chunk_hidden", None)
        if hook is not None:
            # a draft head ingests the prompt from the trunk's hidden rows: every rank holds the rows it owns, so the
            # ranks exchange them (one all-gather per chunk) and each runs the head over the whole chunk, in row steps
            hook(None, slot, ids, pos0, self._gather_resid(c))
        eng.seq_len[slot] = max(eng.seq_len[slot], pos0 + c)
        return c

    def _gather_resid(self, c: int) -> torch.Tensor:
        import torch.distributed as dist
        if self.world == 1:
            return self.own[:c]
        if getattr(self, "_resid_all", None) is None:
            self._resid_all = torch.empty(self.world * self.rows_cap, self.cfg.hidden, dtype=torch.bfloat16, device=self.dev)
        dist.all_gather_into_tensor(self._resid_all, self.own, group=self.group)
        return self._resid_all[:c]

    def run(self, slot: int, ids: List[int], chunk: Optional[int] = None) -> int:
        eng, cfg, m = self.eng, self.cfg, self.eng.model
        chunk = min(chunk or self.max_chunk, self.max_chunk)
        start = eng.seq_len[slot]
        n = len(ids)
        if eng.kv.kv_int8:
            self._int8_begin(slot, start, n)
        for c0 in range(0, n, chunk):
            self.chunk(slot, ids[c0: c0 + chunk], start + c0)
        if eng.kv.kv_int8:
            self._int8_end(slot, start, n)
        last = (n - 1) % chunk
        # the last fold pushed final_norm(residual) of every token: wait for the last token's tile, then the head
        K.wire_wait(self.xw.flags[last // 128:], 128 * self.ag_epoch)
        b = m.buf
        x = self.x_full[last: last + 1]
        nv = m.head_rows
        K.head_gemv(m.w.lm_head, x, b.logits, 1, nv, cfg.hidden, b.cand_val, b.cand_idx)
        if m.tp is not None:
            K.argmax_finish_tp(b.cand_val, b.cand_idx, b.ncand, 1, m.vocab_offset, eng.ctrl, False, m.tp.head, m.tp.mcap)
        else:
            K.argmax_finish(b.cand_val, b.cand_idx, b.ncand, 1, eng.ctrl, False)
        eng.last_prefill_row = 0
        return eng._read_out(1)[0]

    # ------------------------------------------------------------------ int8 KV cache
    # The prompt attention kernel reads bf16 pages.  With an int8 cache the request's K / V of ALL local layers are
    # kept in a bf16 scratch while it is ingested (a rank holds n_kv_heads / world heads: 4 GB for 32,768 positions of
    # the 27B shape at two ranks) and quantised into the cache afterwards; positions the slot already holds are
    # dequantised into the scratch first.  The chunk walk stays chunk-major, so the fused collectives are unchanged.
    def _int8_begin(self, slot: int, start: int, n: int):
        eng, cfg = self.eng, self.cfg
        total = start + n
        eng._ensure_pages(slot, total)
        blocks = (total + 15) // 16
        sc = self._kv16
        if sc is None or sc[0].shape[1] < blocks + 1:
            cap = max(blocks, eng.max_blocks) + 1
            shape = (len(eng.model.w.layers), cap, cfg.n_kv_heads, cfg.page_size, cfg.head_dim)
            self._kv16 = None
            sc = (torch.zeros(shape, dtype=torch.bfloat16, device=self.dev),
                  torch.zeros(shape, dtype=torch.bfloat16, device=self.dev),
                  torch.arange(1, cap + 1, dtype=torch.int32, device=self.dev).clamp_(max=cap - 1).view(1, cap))
        self._kv16 = sc
        if start > 0:
            k16, v16, tab16 = sc
            tab8 = eng.block_table[slot]
            for li in range(k16.shape[0]):
                k8, v8, ks, vs = eng.kv.layer(li)
                K.kv_convert(k16[li], v16[li], tab16[0], k8, v8, ks, vs, tab8, 0, start, cfg.n_kv_heads, cfg.head_dim, False)

    def _int8_end(self, slot: int, start: int, n: int):
        eng, cfg = self.eng, self.cfg
        k16, v16, tab16 = self._kv16
        tab8 = eng.block_table[slot]
        for li in range(k16.shape[0]):
            k8, v8, ks, vs = eng.kv.layer(li)
            K.kv_convert(k16[li], v16[li], tab16[0], k8, v8, ks, vs, tab8, start, n, cfg.n_kv_heads, cfg.head_dim, True)

    def close(self):
        self.x_full = None
        self._kv16 = None
        self.rs.close()
        self.xw.close()


class NcclPrefillRunner(PrefillRunner):
    """Comparison path: replicated residual stream, cuBLAS GEMMs, NCCL all-reduce after o and down."""

    def __init__(self, engine, group=None, max_chunk: int = 4096):
        import torch.distributed as dist
        super().__init__(engine, max_chunk)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        cfg = self.cfg
        self.part = torch.empty(max_chunk, cfg.hidden, dtype=torch.bfloat16, device=self.dev)
        self.qkv16 = torch.empty(max_chunk, cfg.qkv_dim, dtype=torch.bfloat16, device=self.dev)
        self.gu = torch.empty(max_chunk, 2 * cfg.ffn, dtype=torch.bfloat16, device=self.dev)

    def chunk(self, slot: int, ids: List[int], pos0: int):
        import torch.distributed as dist
        eng, cfg, m = self.eng, self.cfg, self.eng.model
        c, h = len(ids), cfg.hidden
        eng._ensure_pages(slot, pos0 + c)
        ids_host = self.ids_stage.begin()
        ids_host[:c] = torch.as_tensor(ids, dtype=torch.int64)
        self.ids_stage.push(self.ids_dev[:c], ids_host[:c])
        resid, x = self.resid[:c], self.x[:c]
        torch.index_select(m.w.embed, 0, self.ids_dev[:c], out=resid)
        bt_row = eng.block_table[slot]
        for li, lw in enumerate(m.w.layers):
            kc, vc, ks, vs = eng.kv.layer(li)
            K.resid_norm(1, c, h, lw.input_norm, cfg.rms_eps, resid, x, resid_in=resid, splits=0)
            torch.matmul(x, self._w_bf16(lw.qkv).t(), out=self.qkv16[:c])
            qkv = self.qkv[:c]
            qkv.copy_(self.qkv16[:c])
            K.rope_append(qkv, 0, 1, c, None, eng.block_table, eng.max_blocks, m.cos_t, m.sin_t, cfg.n_q_heads,
                          cfg.n_kv_heads, cfg.head_dim, self.q, kc, vc, ks, vs, eng.kv.kv_int8, req=slot, pos0=pos0)
            K.attn_prefill(self.q, kc, vc, bt_row, self.attn, c, pos0, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim,
                           eng.kv.num_pages, eng.max_blocks, m.scale, window=m._window(li))
            part = self.part[:c]
            torch.matmul(self.attn[:c], self._w_bf16(lw.o).t(), out=part)
            if self.world > 1:
                dist.all_reduce(part, group=self.group)
            resid.add_(part)
            K.resid_norm(1, c, h, lw.post_norm, cfg.rms_eps, resid, x, resid_in=resid, splits=0)
            gu = self.gu[:c]
            torch.matmul(x, self._w_bf16(lw.gate_up).t(), out=gu)
            g4 = gu.view(c, cfg.ffn // 16, 2, 16)
            act = self.act[:c, : cfg.ffn]
            act.copy_((torch.nn.functional.silu(g4[:, :, 0, :].float()) * g4[:, :, 1, :].float()).reshape(c, cfg.ffn))
            torch.matmul(act, self._w_bf16(lw.down).t(), out=part)
            if self.world > 1:
                dist.all_reduce(part, group=self.group)
            resid.add_(part)
        eng.seq_len[slot] = max(eng.seq_len[slot], pos0 + c)
        return resid

    def run(self, slot: int, ids: List[int], chunk: Optional[int] = None) -> int:
        eng, cfg, m = self.eng, self.cfg, self.eng.model
        chunk = min(chunk or self.max_chunk, self.max_chunk)
        start = eng.seq_len[slot]
        resid = None
        n = len(ids)
        for c0 in range(0, n, chunk):
            resid = self.chunk(slot, ids[c0: c0 + chunk], start + c0)
        last = (n - 1) % chunk
        b = m.buf
        b.resid[0].copy_(resid[last])
        K.resid_norm(1, 1, cfg.hidden, m.w.final_norm, cfg.rms_eps, b.resid, b.x, resid_in=b.resid, splits=0)
        K.head_gemv(m.w.lm_head, b.x, b.logits, 1, m.head_rows, cfg.hidden, b.cand_val, b.cand_idx)
        if m.nccl is not None:
            m._head_nccl(1, eng.ctrl, False)
        elif m.tp is not None:
            K.argmax_finish_tp(b.cand_val, b.cand_idx, b.ncand, 1, m.vocab_offset, eng.ctrl, False, m.tp.head, m.tp.mcap)
        else:
            K.argmax_finish(b.cand_val, b.cand_idx, b.ncand, 1, eng.ctrl, False)
        eng.last_prefill_row = 0
        return eng._read_out(1)[0]
