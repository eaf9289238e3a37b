"""Bindings of the mixture-of-experts kernels (``csrc/moe.cu``) and the batched expert GEMV."""
from __future__ import annotations

import ctypes

import torch

from . import lib as K


def route(logits: torch.Tensor, ld: int, t: int, e: int, k: int, topk_idx: torch.Tensor, topk_w: torch.Tensor):
    """softmax over the first ``e`` columns -> top-k (ties to the lower id) -> renormalise."""
    K._check(K.lib().b2_moe_route(K._p(logits), ld, t, e, k, K._p(topk_idx), K._p(topk_w), K._stream()), "moe_route")


def sort(topk_idx, t, k, e, max_blk, counts, rank, expert_base, blk_expert, blk_row0, blk_rows, n_blk, total_rows):
    """Histogram + ranks, then the padded expert-major plan (block table for the grouped GEMM)."""
    rc = K.lib().b2_moe_sort(K._p(topk_idx), t, k, e, max_blk, K._p(counts), K._p(rank), K._p(expert_base),
                             K._p(blk_expert), K._p(blk_row0), K._p(blk_rows), K._p(n_blk), K._p(total_rows),
                             K._stream())
    K.launch_count += 1
    K._check(rc, "moe_sort")


def count(topk_idx, n, counts, rank):
    """Per-expert histogram (``counts`` zeroed by the caller) and every entry's rank inside its expert."""
    K._check(K.lib().b2_moe_count(K._p(topk_idx), n, K._p(counts), K._p(rank), K._stream()), "moe_count")


def scatter(topk_idx, rank, expert_base, t, k, x, h, row_of, xs):
    K._check(K.lib().b2_moe_scatter(K._p(topk_idx), K._p(rank), K._p(expert_base), t, k, K._p(x), h, K._p(row_of),
                                    K._p(xs), K._stream()), "moe_scatter")


def combine(y, row_of, topk_w, t, k, h, shared_y, gate_logit, gate_ld, resid, out):
    K._check(K.lib().b2_moe_combine(K._p(y), K._p(row_of), K._p(topk_w), t, k, h, K._p(shared_y), K._p(gate_logit),
                                    gate_ld, K._p(resid), K._p(out), K._stream()), "moe_combine")


def combine_rows(part, s, m, k, h, topk_w, shared_part, s_sh, gate_logit, gate_ld, out, fold_resid=None, fold_ssq=None):
    """Weighted sum of a row's slots (split-K slices folded).  ``fold_resid`` / ``fold_ssq``: add the sum to the bf16
    residual rows in place and leave the per-128-column sums of squares for the next fused RMSNorm, instead of
    writing ``out``."""
    K._check(K.lib().b2_moe_combine_rows(K._p(part), s, m, k, h, K._p(topk_w), K._p(shared_part), s_sh,
                                         K._p(gate_logit), gate_ld, K._p(out), K._p(fold_resid), K._p(fold_ssq),
                                         K._stream()), "moe_combine_rows")


def router_rows(w, x, logits, m, r, h, ld, e, k, shared_slot, has_gate, topk_idx, topk_w, ticket):
    """Decode rows: router logits (``r`` rows of ``w``: the experts, then the shared expert's gate row) and the
    routing of every row in one launch.  ``shared_slot``: each row gets slot k = (expert id ``e``, sigmoid(gate logit)
    or 1), so ``topk_idx`` / ``topk_w`` hold k + 1 entries per row.  ``ticket``: one zeroed int32 word."""
    K._check(K.lib().b2_moe_router_rows(K._p(w), K._p(x), K._p(logits), m, r, h, ld, e, k, int(shared_slot), int(has_gate),
                                        K._p(topk_idx), K._p(topk_w), K._p(ticket), K._stream()), "moe_router_rows")


def gemv_experts(w4b_stack, expert_bytes, expert_ids, batches, x, x_div, x_batch_bytes, out, n, k, splits, ldx,
                 x_mode=0, s_in=1, x_slice=0, sparse=False, alt_w=None, alt_id=-1):
    """One row per batch against the W4B weights of expert ``expert_ids[b]``; ``out`` is ``[b][splits][n]``.
    ``sparse``: batches whose id is negative are skipped (their output rows are left as they are).  ``alt_w``: batches
    whose id is ``alt_id`` read this tensor instead of the stack (the shared expert as one more slot of a row)."""
    if alt_w is not None:
        rc = K.lib().b2_gemv_w4_experts_alt(K._p(w4b_stack), ctypes.c_longlong(expert_bytes), K._p(expert_ids), batches,
                                            K._p(x), x_div, ctypes.c_longlong(x_batch_bytes), K._p(out), n, k, splits, ldx,
                                            x_mode, s_in, ctypes.c_longlong(x_slice), K._p(alt_w), alt_id, K._stream())
        K._check(rc, "gemv_w4_experts_alt")
        return
    fn = K.lib().b2_gemv_w4_experts_sparse if sparse else K.lib().b2_gemv_w4_experts
    rc = fn(K._p(w4b_stack), ctypes.c_longlong(expert_bytes), K._p(expert_ids), batches,
                                    K._p(x), x_div, ctypes.c_longlong(x_batch_bytes), K._p(out), n, k, splits, ldx,
                                    x_mode, s_in, ctypes.c_longlong(x_slice), K._stream())
    K._check(rc, "gemv_w4_experts")
