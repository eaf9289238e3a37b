"""Chunked prompt pass on the tensor cores.

The role of the reference's prefill walk (src/runtime/prefill/step.cc:102-319,
engine_prefill.cc:159-322): the prompt is cut in chunks, each chunk walks the
layers once with GEMM-shaped kernels, nothing waits on the host inside a chunk.
Per layer: RMSNorm rows -> qkv GEMM (fp32 out) -> RoPE + paged KV append ->
causal flash attention over the page pool -> o GEMM with the residual add in its
epilogue -> RMSNorm -> gate‖up GEMM with SiLU*up in its epilogue -> down GEMM
with the residual add.  Only the last row of the last chunk goes through the head.

Weight forms for the GEMMs:
  ``bf16``      W4B is dequantised to a bf16 slab right before each GEMM (two-pass, as the
                reference's pf_dequant_slab + pf_gemm) -- no second resident copy of the model;
  ``bf16-resident``  the dequantised matrices stay in HBM (a 27B model is 42 GB of the 180 GB);
  ``int8``      per-token int8 activations x per-row int8 weights on kind::i8, scales in the epilogue
                (the reference's ``--prefill-backend l0-int8``, docs/16-int8-prefill.md).
"""
from __future__ import annotations

import os

from typing import List, Optional

import torch

from ..utils.staging import Staged

from ..models.weights import QLinear
from ..ops import gemm as G
from ..ops import lib as K


class PhaseProfile:
    """Per-phase device times of the prompt pass (CUDA events around each phase), switched on with the environment
    variable ``B200SERVE_PREFILL_PROFILE=1`` and printed per prompt on stderr -- the reference's
    ``B70_PREFILL_PROFILE`` (src/runtime/prefill/profile.h:20-91).  Events are only recorded, never waited on,
    until the prompt is done."""

    def __init__(self):
        self.spans = []      # (phase, start event, end event)
        self._open = None

    def begin(self, phase: str):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._open = (phase, ev)

    def end(self):
        if self._open is None:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.spans.append((self._open[0], self._open[1], ev))
        self._open = None

    def report(self, out, tokens: int):
        torch.cuda.synchronize()
        tot = {}
        for name, a, b in self.spans:
            tot[name] = tot.get(name, 0.0) + a.elapsed_time(b)
        allms = sum(tot.values()) or 1.0
        parts = ", ".join(f"{k} {v:.2f} ms ({100 * v / allms:.0f} %)" for k, v in sorted(tot.items(), key=lambda kv: -kv[1]))
        out.write(f"prefill profile: {tokens} tokens, {allms:.2f} ms in phases: {parts}\n")
        self.spans = []


class PrefillRunner:
    def __init__(self, engine, max_chunk: int = 4096):
        import os
        self.profile = PhaseProfile() if os.environ.get("B200SERVE_PREFILL_PROFILE", "0") not in ("", "0") else None
        self.eng = engine
        self.cfg = cfg = engine.cfg
        self.dev = engine.device
        self.max_chunk = max_chunk
        self.backend = engine.prefill_backend
        if self.backend == "auto":
            # keep dequantised bf16 copies of the linears when they take at most 45 % of the GPU's memory (a 27B
            # model is 54 GB, a 35B-A3B one 70 GB of a B200's 180 GB): the prompt pass then reads them in place
            # instead of dequantising a slab before every GEMM
            total = torch.cuda.get_device_properties(self.dev).total_memory if self.dev.type == "cuda" else 0
            self.backend = "bf16-resident" if 2 * cfg.param_count() <= 0.45 * total else "bf16"
        if self.backend in ("int4", "w4a16"):
            self.backend = "w4"
        if self.backend == "l0":
            self.backend = "bf16"
        if self.backend == "l0-int8":
            self.backend = "int8"
        bf, f32 = torch.bfloat16, torch.float32
        c, h = max_chunk, cfg.hidden
        self.resid = torch.empty(c, h, dtype=bf, device=self.dev)
        self.x = torch.empty(c, h, dtype=bf, device=self.dev)
        self.qkv = torch.empty(c, cfg.qkv_dim, dtype=f32, device=self.dev)
        self.q = torch.empty(c, cfg.q_dim, dtype=bf, device=self.dev)
        self.attn = torch.empty(c, cfg.q_dim, dtype=bf, device=self.dev)
        ffn = cfg.ffn if not cfg.is_moe else max(cfg.expert_ffn, cfg.shared_ffn)
        self.act = torch.empty(c, max(ffn, 1), dtype=bf, device=self.dev)
        if cfg.n_gdn_layers:     # gated delta-net layers: projection, convolved activations, read-out
            self.gdn_proj = torch.empty(c, cfg.gdn_proj_dim, dtype=f32, device=self.dev)
            self.gdn_act = torch.empty(c, cfg.gdn_proj_dim, dtype=f32, device=self.dev)
            self.gdn_out = torch.empty(c, cfg.gdn_value_dim, dtype=bf, device=self.dev)
            # the chunked scan's operand images, one block per (64-row chunk, value head); B2_GDN_WY=0: sequential scan
            self.gdn_ws = None
            if os.environ.get("B2_GDN_WY", "1") == "1" and cfg.gdn_head_dim == 128:
                self.gdn_ws = torch.empty(((c + 63) // 64) * cfg.gdn_v_heads * K.gdn_wy_block_bytes(), dtype=torch.uint8,
                                          device=self.dev)
        self.ids_stage = Staged((max_chunk,), torch.int64)   # ring of pinned buffers: the host runs a chunk ahead of the copies
        self.ids_dev = torch.empty(max_chunk, dtype=torch.int64, device=self.dev)
        self._slab: Optional[torch.Tensor] = None
        if self.backend == "int8":
            kmax = max(h, cfg.q_dim, ffn)
            self.a8 = torch.empty(c, kmax, dtype=torch.int8, device=self.dev)
            self.a_scale = torch.empty(c, dtype=f32, device=self.dev)

    # ------------------------------------------------------------------ weights
    def _w_bf16(self, ql: QLinear) -> torch.Tensor:
        if ql._w_bf16 is not None:
            return ql._w_bf16
        if self.backend == "bf16-resident":
            ql._w_bf16 = G.dequant_w4b(ql.w4b, ql.n, ql.k)
            return ql._w_bf16
        need = ql.n * ql.k
        if self._slab is None or self._slab.numel() < need:
            self._slab = torch.empty(need, dtype=torch.bfloat16, device=self.dev)
        out = self._slab[:need].view(ql.n, ql.k)
        return G.dequant_w4b(ql.w4b, ql.n, ql.k, out)

    def _w_i8(self, ql: QLinear):
        if ql._w_i8 is None:
            w = G.dequant_w4b(ql.w4b, ql.n, ql.k).float()
            sc = w.abs().amax(dim=1).clamp_min(1e-12) / 127.0
            ql._w_i8 = (torch.round(w / sc[:, None]).clamp_(-127, 127).to(torch.int8).contiguous(), sc.contiguous())
            del w
        return ql._w_i8

    def linear(self, ql: QLinear, a: torch.Tensor, out: torch.Tensor, epi: int, resid=None):
        """``out = epilogue(a @ W^T)`` for ``a`` ``[rows][k]`` bf16."""
        if self.backend == "int8":
            rows = a.shape[0]
            a8 = self.a8[:rows, : ql.k] if self.a8.shape[1] == ql.k else self.a8.view(-1)[: rows * ql.k].view(rows, ql.k)
            G.quant_rows_i8(a, a8, self.a_scale[:rows])
            w8, ws = self._w_i8(ql)
            G.gemm_i8(a8, w8, self.a_scale[:rows], ws, out, epi=epi, resid=resid)
        elif self.backend == "w4":      # the GEMM reads the int4 blocks itself: nothing but the W4B weights is resident
            G.gemm_w4(a, ql.w4b, ql.n, ql.k, out, epi=epi, resid=resid)
        else:
            G.gemm_bf16(a, self._w_bf16(ql), out, epi=epi, resid=resid)

    # ------------------------------------------------------------------ one layer over a chunk
    def layer(self, lw, kv_index: int, slot: int, c: int, pos0: int, resid, x):
        """``resid[:c]`` through one decoder layer whose KV lives at ``kv_index`` of the cache."""
        eng, cfg, m = self.eng, self.cfg, self.eng.model
        h = cfg.hidden
        bt_row = eng.block_table[slot]
        pr = self.profile

        def phase(name):
            if pr is not None:
                pr.end()
                pr.begin(name)
        phase("norm")
        K.resid_norm(1, c, h, lw.input_norm, cfg.rms_eps, resid, x, resid_in=resid, splits=0)
        if lw.gdn is not None:
            # gated delta-net layer: the projections run as GEMMs over the chunk; the recurrence walks the chunk's
            # rows in order inside one CTA per value head (a sequential scan, not the chunked WY form)
            g, gi, n = lw.gdn, cfg.gdn_index(kv_index), cfg.gdn_proj_dim
            phase("gdn_in")
            self.linear(g.in_proj, x, self.gdn_proj[:c], G.EPI_F32)
            phase("gdn_scan")
            K.gdn_conv(self.gdn_proj, 1, c, n, cfg.gdn_conv_channels, None, g.conv_w, eng.kv.gdn_conv[gi],
                       self.gdn_act, slot=slot)
            if self.gdn_ws is not None and c >= 64:
                K.gdn_chunk_wy(self.gdn_act, c, n, cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim, slot, g.a_log,
                               g.dt_bias, g.norm_w, cfg.rms_eps, eng.kv.gdn_state[gi], self.gdn_out, self.gdn_ws)
            else:
                K.gdn_chunk(self.gdn_act, c, n, cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim, slot, g.a_log,
                            g.dt_bias, g.norm_w, cfg.rms_eps, eng.kv.gdn_state[gi], self.gdn_out)
            phase("gdn_out")
            self.linear(g.out_proj, self.gdn_out[:c], resid, G.EPI_RESID_ADD, resid=resid)
        else:
            kc, vc, ks, vs = eng.kv.layer(kv_index)
            qkv = self.qkv[:c]
            phase("qkv")
            self.linear(lw.qkv, x, qkv, G.EPI_F32)
            phase("rope+append")
            K.rope_append(qkv, 0, 1, c, None, eng.block_table, eng.max_blocks, m.cos_t, m.sin_t, cfg.n_q_heads,
                          cfg.n_kv_heads, cfg.head_dim, self.q, kc, vc, ks, vs, eng.kv.kv_int8, req=slot, pos0=pos0)
            phase("attention")
            K.attn_prefill(self.q, kc, vc, bt_row, self.attn, c, pos0, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim,
                           eng.kv.num_pages, eng.max_blocks, m.scale, window=m._window(kv_index))
            phase("o")
            self.linear(lw.o, self.attn[:c], resid, G.EPI_RESID_ADD, resid=resid)
        phase("norm")
        K.resid_norm(1, c, h, lw.post_norm, cfg.rms_eps, resid, x, resid_in=resid, splits=0)
        if lw.gate_up is not None:
            act = self.act[:c, : cfg.ffn]
            phase("gate_up")
            self.linear(lw.gate_up, x, act, G.EPI_SILU_MUL)
            phase("down")
            self.linear(lw.down, act, resid, G.EPI_RESID_ADD, resid=resid)
        else:
            from ..models import moe as _moe
            phase("moe")
            _moe.moe_block_prefill(self, lw, c)
        if pr is not None:
            pr.end()

    # ------------------------------------------------------------------ one chunk
    def chunk(self, slot: int, ids: List[int], pos0: int):
        eng, cfg, m = self.eng, self.cfg, self.eng.model
        c, h = len(ids), cfg.hidden
        eng._ensure_pages(slot, pos0 + c)
        eng._gdn_snap = None      # (a hybrid model's recurrent state moves on: nothing to rewind to)
        ids_host = self.ids_stage.begin()
        ids_host[:c] = torch.as_tensor(ids, dtype=torch.int64)
        self.ids_stage.push(self.ids_dev[:c], ids_host[:c])
        resid, x = self.resid[:c], self.x[:c]
        torch.index_select(m.w.embed, 0, self.ids_dev[:c], out=resid)
        bt_row = eng.block_table[slot]
        for li, lw in enumerate(m.w.layers):
            self.layer(lw, li, slot, c, pos0, resid, x)
        hook = getattr(eng, "on_chunk_hidden", None)
        if hook is not None:      # draft heads ingest the prompt from the trunk's hidden states
            hook(self, slot, ids, pos0, resid)
        eng.seq_len[slot] = max(eng.seq_len[slot], pos0 + c)
        return resid

    # ------------------------------------------------------------------ int8 KV cache: layer-major pass
    def _run_int8_kv(self, slot: int, ids: List[int], chunk: int):
        """Prompt pass into an int8 KV cache.  The attention kernel reads bf16 pages, so the walk is LAYER-major:
        all chunks go through layer l against a one-layer bf16 scratch (identity page table, positions of the
        whole sequence), then the layer's new rows are quantised into the int8 cache and the scratch is reused
        by layer l + 1.  Earlier positions of the sequence (a cached prefix, earlier turns) are dequantised
        into the scratch first.  Costs one residual row per prompt token (kept across the layer loop) instead
        of a bf16 cache of all layers."""
        eng, cfg, m = self.eng, self.cfg, self.eng.model
        n, start = len(ids), eng.seq_len[slot]
        total = start + n
        eng._ensure_pages(slot, total)
        blocks = (total + 15) // 16
        sc = getattr(self, "_kv16", None)
        if sc is None or sc[0].shape[1] < blocks + 1:
            cap = max(blocks, eng.max_blocks) + 1
            shape = (1, cap, cfg.n_kv_heads, cfg.page_size, cfg.head_dim)
            sc = self._kv16 = (torch.zeros(shape, dtype=torch.bfloat16, device=self.dev),
                               torch.zeros(shape, dtype=torch.bfloat16, device=self.dev),
                               torch.arange(1, cap + 1, dtype=torch.int32, device=self.dev).clamp_(max=cap - 1).view(1, cap))
        k16, v16, tab16 = sc
        if getattr(self, "_resid_all", None) is None or self._resid_all.shape[0] < n:
            self._resid_all = torch.empty(max(n, self.max_chunk), cfg.hidden, dtype=torch.bfloat16, device=self.dev)
        resid_all = self._resid_all[:n]
        ids_dev = torch.as_tensor(ids, dtype=torch.int64).pin_memory().to(self.dev, non_blocking=True)
        torch.index_select(m.w.embed, 0, ids_dev, out=resid_all)
        tab8 = eng.block_table[slot]
        h = cfg.hidden
        for li, lw in enumerate(m.w.layers):
            k8, v8, ks, vs = eng.kv.layer(li)
            if start > 0:
                K.kv_convert(k16[0], v16[0], tab16[0], k8, v8, ks, vs, tab8, 0, start, cfg.n_kv_heads, cfg.head_dim, False)
            for c0 in range(0, n, chunk):
                c = min(chunk, n - c0)
                resid, x = resid_all[c0: c0 + c], self.x[:c]
                pos0 = start + c0
                K.resid_norm(1, c, h, lw.input_norm, cfg.rms_eps, resid, x, resid_in=resid, splits=0)
                qkv = self.qkv[:c]
                self.linear(lw.qkv, x, qkv, G.EPI_F32)
                K.rope_append(qkv, 0, 1, c, None, tab16, tab16.shape[1], m.cos_t, m.sin_t, cfg.n_q_heads, cfg.n_kv_heads,
                              cfg.head_dim, self.q, k16[0], v16[0], None, None, False, req=0, pos0=pos0)
                K.attn_prefill(self.q, k16[0], v16[0], tab16[0], self.attn, c, pos0, cfg.n_q_heads, cfg.n_kv_heads,
                               cfg.head_dim, k16.shape[1], tab16.shape[1], m.scale, window=m._window(li))
                self.linear(lw.o, self.attn[:c], resid, G.EPI_RESID_ADD, resid=resid)
                K.resid_norm(1, c, h, lw.post_norm, cfg.rms_eps, resid, x, resid_in=resid, splits=0)
                if lw.gate_up is not None:
                    act = self.act[:c, : cfg.ffn]
                    self.linear(lw.gate_up, x, act, G.EPI_SILU_MUL)
                    self.linear(lw.down, act, resid, G.EPI_RESID_ADD, resid=resid)
                else:
                    self.resid, keep = resid, self.resid      # the MoE block works on self.resid / self.x
                    try:
                        from ..models import moe as _moe
                        _moe.moe_block_prefill(self, lw, c)
                    finally:
                        self.resid = keep
            K.kv_convert(k16[0], v16[0], tab16[0], k8, v8, ks, vs, tab8, start, n, cfg.n_kv_heads, cfg.head_dim, True)
        eng.seq_len[slot] = total
        return resid_all[n - 1: n]

    def run(self, slot: int, ids: List[int], chunk: Optional[int] = None) -> int:
        eng, cfg, m = self.eng, self.cfg, self.eng.model
        chunk = min(chunk or self.max_chunk, self.max_chunk)
        if eng.kv.kv_int8:
            last_row = self._run_int8_kv(slot, ids, chunk)
            b = m.buf
            b.resid[0].copy_(last_row[0])
            return self._head_of_row0()
        start = eng.seq_len[slot]
        resid = None
        n = len(ids)
        for c0 in range(0, n, chunk):
            resid = self.chunk(slot, ids[c0: c0 + chunk], start + c0)
        last = (n - 1) % chunk
        m.buf.resid[0].copy_(resid[last])
        tok = self._head_of_row0()
        if self.profile is not None:
            import sys
            self.profile.report(sys.stderr, n)
        return tok

    def _head_of_row0(self) -> int:
        """Final norm, lm_head and arg-max of the residual row in ``buf.resid[0]``."""
        eng, cfg, m = self.eng, self.cfg, self.eng.model
        b = m.buf
        K.resid_norm(1, 1, cfg.hidden, m.w.final_norm, cfg.rms_eps, b.resid, b.x, resid_in=b.resid, splits=0)
        if m.int8_head:
            w8, sc = m.w.lm_head_i8
            K.head_gemv(w8, b.x, b.logits, 1, cfg.vocab, cfg.hidden, b.cand_val, b.cand_idx, wscale=sc)
        else:
            K.head_gemv(m.w.lm_head, b.x, b.logits, 1, cfg.vocab, cfg.hidden, b.cand_val, b.cand_idx)
        K.argmax_finish(b.cand_val, b.cand_idx, b.ncand, 1, eng.ctrl, False)
        return eng._read_out(1)[0]
