"""Mixture-of-experts FFN on the GPU: the row path (decode / verify) and the prompt path.

Row path (M <= 64 rows): router GEMV -> route kernel -> one batched W4A16 GEMV launch for all
(row, slot) pairs' gate‖up, one for their down projections (SiLU*up folded into its activation
load), the shared expert through the ordinary row GEMV, and a combine that folds split-K slices
and weights in slot order -- the role of the reference's moe_route / moe_gate_up / moe_down
(src/kernels/moe.cl:1-70).  Prompt path: router GEMM -> route -> device-side sort into
expert-major 128-row blocks -> gather -> grouped tcgen05 GEMM (gate‖up with SiLU*up epilogue,
then down) -> combine with the shared expert and the residual -- the role of pf_moe_sort_mw.cl,
pf_moe.cl and pf_moe_gemm.cl.  The host never reads a count.
"""
from __future__ import annotations

import torch

from ..ops import gemm as G
from ..ops import lib as K
from ..ops import moe as M
from ..utils import quant as Q
from .weights import LayerWeights


def router_cat(lw: LayerWeights, cfg) -> torch.Tensor:
    """Router rows, then the shared expert's gate row, zero-padded to a multiple of 8 rows."""
    t = getattr(lw, "_router_cat", None)
    if t is None:
        rows = [lw.router]
        if lw.shared_gate is not None:
            rows.append(lw.shared_gate)
        cat = torch.cat(rows, dim=0)
        pad = (-cat.shape[0]) % 8
        if pad:
            cat = torch.cat([cat, torch.zeros(pad, cat.shape[1], dtype=cat.dtype, device=cat.device)])
        t = lw._router_cat = cat.contiguous()
    return t


class _RowScratch:
    def __init__(self, model):
        cfg, dev, mr = model.cfg, model.device, model.max_rows
        e, k, h, i = cfg.n_experts, cfg.top_k, cfg.hidden, cfg.expert_ffn
        self.ld = (e + (1 if cfg.shared_ffn else 0) + 7) // 8 * 8
        self.logits = torch.zeros(mr, self.ld, dtype=torch.float32, device=dev)
        self.topk_idx = torch.zeros(mr * (k + 1), dtype=torch.int32, device=dev)      # + the shared expert's slot
        self.topk_w = torch.zeros(mr * (k + 1), dtype=torch.float32, device=dev)
        self.s_gu = K.gemv_splits(2 * i, h)
        self.s_dn = K.gemv_splits(h, i)
        self.part_gu = torch.zeros(mr * (k + 1) * self.s_gu * 2 * i, dtype=torch.float32, device=dev)
        self.part_dn = torch.zeros(mr * (k + 1) * self.s_dn * h, dtype=torch.float32, device=dev)
        self.out = torch.zeros(mr * h, dtype=torch.float32, device=dev)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=dev)


def moe_block_rows(model, lw: LayerWeights, m: int, fold: bool = False):
    """Returns (partials, splits) of the MoE branch for the next residual fold.  ``fold``: the weighted sum is added
    to ``buf.resid`` in place and ``buf.ssq`` gets the rows' sums of squares (returns ``(None, 0)``)."""
    cfg, b = model.cfg, model.buf
    sc = getattr(model, "_moe_rows", None)
    if sc is None:
        sc = model._moe_rows = _RowScratch(model)
    e, k, h, i = cfg.n_experts, cfg.top_k, cfg.hidden, cfg.expert_ffn
    rc = router_cat(lw, cfg)
    gu_bytes = lw.experts_gate_up_w4b[0].numel()
    dn_bytes = lw.experts_down_w4b[0].numel()
    if lw.shared is None or (cfg.shared_ffn == i and lw.shared.gate_up.w4b.numel() == gu_bytes):
        # Four launches: router logits + routing (one kernel, the shared expert becomes slot k of every row with
        # weight sigmoid(gate)), the two batched int4 GEMVs over k (+ 1) slots per row -- the shared expert's weights
        # ride along as an alternative tensor for its slot id -- and the weighted sum.
        ks = k + (1 if lw.shared is not None else 0)
        M.router_rows(rc, b.x, sc.logits, m, e + (1 if lw.shared_gate is not None else 0), h, sc.ld, e, k,
                      lw.shared is not None, lw.shared_gate is not None, sc.topk_idx, sc.topk_w, sc.ticket)
        alt_gu = lw.shared.gate_up.w4b if lw.shared is not None else None
        alt_dn = lw.shared.down.w4b if lw.shared is not None else None
        M.gemv_experts(lw.experts_gate_up_w4b, gu_bytes, sc.topk_idx, m * ks, b.x, ks, h * 2, sc.part_gu, 2 * i, h, sc.s_gu, h,
                       alt_w=alt_gu, alt_id=e)
        M.gemv_experts(lw.experts_down_w4b, dn_bytes, sc.topk_idx, m * ks, sc.part_gu, 1, sc.s_gu * 2 * i * 4, sc.part_dn,
                       h, i, sc.s_dn, 2 * i, x_mode=1, s_in=sc.s_gu, x_slice=2 * i, alt_w=alt_dn, alt_id=e)
        if fold:
            M.combine_rows(sc.part_dn, sc.s_dn, m, ks, h, sc.topk_w, None, 0, None, sc.ld, sc.out, fold_resid=b.resid,
                           fold_ssq=b.ssq)
            return None, 0
        M.combine_rows(sc.part_dn, sc.s_dn, m, ks, h, sc.topk_w, None, 0, None, sc.ld, sc.out)
        return sc.out, 1
    if fold:
        raise NotImplementedError("the folding combine covers a shared expert of the routed experts' shape")
    K.head_gemv(rc, b.x, sc.logits, m, rc.shape[0], h)
    M.route(sc.logits, sc.ld, m, e, k, sc.topk_idx, sc.topk_w)
    M.gemv_experts(lw.experts_gate_up_w4b, gu_bytes, sc.topk_idx, m * k, b.x, k, h * 2, sc.part_gu, 2 * i, h, sc.s_gu, h)
    M.gemv_experts(lw.experts_down_w4b, dn_bytes, sc.topk_idx, m * k, sc.part_gu, 1, sc.s_gu * 2 * i * 4, sc.part_dn,
                   h, i, sc.s_dn, 2 * i, x_mode=1, s_in=sc.s_gu, x_slice=2 * i)
    sh_part, s_sh, gate = None, 0, None
    if lw.shared is not None:
        gu, s_gu = model._gemv("sh_gate_up", lw.shared.gate_up, b.x, m)
        sh_part, s_sh = model._gemv("sh_down", lw.shared.down, gu, m, x_mode=1, s_in=s_gu,
                                    x_slice=m * 2 * cfg.shared_ffn)
        gate = sc.logits[:, e:]
    M.combine_rows(sc.part_dn, sc.s_dn, m, k, h, sc.topk_w, sh_part, s_sh, gate, sc.ld, sc.out)
    return sc.out, 1


class _PrefillScratch:
    def __init__(self, runner):
        cfg, dev, c = runner.cfg, runner.dev, runner.max_chunk
        e, k, h, i = cfg.n_experts, cfg.top_k, cfg.hidden, cfg.expert_ffn
        i32, f32, bf = torch.int32, torch.float32, torch.bfloat16
        self.ld = (e + (1 if cfg.shared_ffn else 0) + 7) // 8 * 8
        self.logits = torch.empty(c, self.ld, dtype=f32, device=dev)
        self.topk_idx = torch.empty(c * k, dtype=i32, device=dev)
        self.topk_w = torch.empty(c * k, dtype=f32, device=dev)
        self.max_blk = (c * k + 127) // 128 + e
        rows = self.max_blk * 128
        self.counts = torch.zeros(e, dtype=i32, device=dev)
        self.rank = torch.empty(c * k, dtype=i32, device=dev)
        self.expert_base = torch.empty(e, dtype=i32, device=dev)
        self.blk_expert = torch.zeros(self.max_blk, dtype=i32, device=dev)
        self.blk_row0 = torch.zeros(self.max_blk, dtype=i32, device=dev)
        self.blk_rows = torch.zeros(self.max_blk, dtype=i32, device=dev)
        self.n_blk = torch.zeros(1, dtype=i32, device=dev)
        self.total_rows = torch.zeros(1, dtype=i32, device=dev)
        self.row_of = torch.empty(c * k, dtype=i32, device=dev)
        self.xs = torch.zeros(rows, h, dtype=bf, device=dev)
        self.act = torch.zeros(rows, i, dtype=bf, device=dev)
        self.y = torch.zeros(rows, h, dtype=bf, device=dev)
        self.shared_y = torch.empty(c, h, dtype=bf, device=dev) if cfg.shared_ffn else None
        self.slab_gu = self.slab_dn = None


def _expert_bf16(runner, lw: LayerWeights, sc: _PrefillScratch):
    """bf16 ``[E][N][K]`` forms of the stacked experts: resident when asked for, else dequantised into
    slabs that the next layer overwrites."""
    cfg = runner.cfg
    e, h, i = cfg.n_experts, cfg.hidden, cfg.expert_ffn
    cached = getattr(lw, "_experts_bf16", None)
    if cached is not None:
        return cached
    if runner.backend == "bf16-resident":
        gu = G.dequant_w4b(lw.experts_gate_up_w4b.view(-1, h // 64, Q.BLOCK_BYTES), e * 2 * i, h).view(e, 2 * i, h)
        dn = G.dequant_w4b(lw.experts_down_w4b.view(-1, i // 64, Q.BLOCK_BYTES), e * h, i).view(e, h, i)
        lw._experts_bf16 = (gu, dn)
        return lw._experts_bf16
    if sc.slab_gu is None:
        sc.slab_gu = torch.empty(e, 2 * i, h, dtype=torch.bfloat16, device=runner.dev)
        sc.slab_dn = torch.empty(e, h, i, dtype=torch.bfloat16, device=runner.dev)
    G.dequant_w4b(lw.experts_gate_up_w4b, e * 2 * i, h, sc.slab_gu)
    G.dequant_w4b(lw.experts_down_w4b, e * h, i, sc.slab_dn)
    return sc.slab_gu, sc.slab_dn


def moe_block_prefill(runner, lw: LayerWeights, c: int):
    """``runner.resid[:c] += MoE(runner.x[:c])`` for a prompt chunk."""
    cfg = runner.cfg
    ep = getattr(runner, "ep", None)
    if ep is not None:      # experts spread over the ranks of a group (parallel/ep.py)
        return ep.block_prefill(runner, lw, c)
    sc = getattr(runner, "_moe_pf", None)
    if sc is None:
        sc = runner._moe_pf = _PrefillScratch(runner)
    e, k, h, i = cfg.n_experts, cfg.top_k, cfg.hidden, cfg.expert_ffn
    x, resid = runner.x[:c], runner.resid[:c]
    rc = router_cat(lw, cfg)
    logits = sc.logits[:c]
    G.gemm_bf16(x, rc, logits, epi=G.EPI_F32)
    M.route(logits, sc.ld, c, e, k, sc.topk_idx, sc.topk_w)
    sc.counts.zero_()
    M.sort(sc.topk_idx, c, k, e, sc.max_blk, sc.counts, sc.rank, sc.expert_base, sc.blk_expert, sc.blk_row0,
           sc.blk_rows, sc.n_blk, sc.total_rows)
    M.scatter(sc.topk_idx, sc.rank, sc.expert_base, c, k, x, h, sc.row_of, sc.xs)
    blocks = (sc.blk_expert, sc.blk_row0, sc.blk_rows, sc.n_blk, sc.max_blk)
    if runner.backend == "w4":      # grouped GEMMs over the experts' int4 blocks (a quarter of the bf16 bytes from HBM)
        G.gemm_w4(sc.xs, lw.experts_gate_up_w4b, 2 * i, h, sc.act, epi=G.EPI_SILU_MUL, blocks=blocks, n_experts=e)
        G.gemm_w4(sc.act, lw.experts_down_w4b, h, i, sc.y, epi=G.EPI_BF16, blocks=blocks, n_experts=e)
    else:
        gu, dn = _expert_bf16(runner, lw, sc)
        G.gemm_grouped_bf16(sc.xs, gu, sc.act, blocks, epi=G.EPI_SILU_MUL)
        G.gemm_grouped_bf16(sc.act, dn, sc.y, blocks, epi=G.EPI_BF16)
    shared_y, gate = None, None
    if lw.shared is not None:
        act = runner.act[:c, : cfg.shared_ffn]
        runner.linear(lw.shared.gate_up, x, act, G.EPI_SILU_MUL)
        shared_y = sc.shared_y[:c]
        runner.linear(lw.shared.down, act, shared_y, G.EPI_BF16)
        gate = logits[:, e:]
    M.combine(sc.y, sc.row_of, sc.topk_w, c, k, h, shared_y, gate, sc.ld, resid, resid)
