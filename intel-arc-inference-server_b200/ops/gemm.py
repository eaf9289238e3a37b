"""Bindings of the tcgen05 prefill GEMMs (``csrc/gemm_tc.cu``)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import lib as K

EPI_BF16, EPI_F32, EPI_SILU_MUL, EPI_RESID_ADD, EPI_RS_PUSH, EPI_EP_RETURN = 0, 1, 2, 3, 4, 5


def _launch(a, b, c, m, n, k, ldc, i8, epi, resid=None, a_scale=None, b_scale=None, blocks=None, n_experts=0, bn=0):
    be = br0 = brn = nb = None
    max_blk = 0
    if blocks is not None:
        be, br0, brn, nb, max_blk = blocks
    rc = K.lib().b2_gemm_tc(K._p(a), K._p(b), K._p(c), m, n, k, ldc, int(i8), epi, K._p(resid), K._p(a_scale),
                            K._p(b_scale), K._p(be), K._p(br0), K._p(brn), K._p(nb), max_blk, n_experts, bn,
                            K._stream())
    K._check(rc, "gemm_tc")


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, epi: int = EPI_BF16,
              resid: Optional[torch.Tensor] = None, bn: int = 0):
    """``c = a @ b.T`` with ``a`` ``[M][K]``, ``b`` ``[N][K]`` bf16.  ``epi``: bf16 / fp32 store,
    SiLU(gate)*up over interleave16 columns (``c`` is ``[M][N/2]``), or ``resid + a b^T`` in bf16."""
    m, k = a.shape
    n = b.shape[0]
    _launch(a, b, c, m, n, k, c.stride(0), False, epi, resid=resid, bn=bn)


def gemm_i8(a8, b8, a_scale, b_scale, c, epi: int = EPI_BF16, resid=None, bn: int = 0):
    """int8 x int8 -> int32 on kind::i8, ``c = (a8 @ b8.T) * a_scale[:, None] * b_scale[None, :]``."""
    m, k = a8.shape
    n = b8.shape[0]
    _launch(a8, b8, c, m, n, k, c.stride(0), True, epi, resid=resid, a_scale=a_scale, b_scale=b_scale, bn=bn)


def gemm_w4(a: torch.Tensor, w4b: torch.Tensor, n: int, k: int, c: torch.Tensor, epi: int = EPI_BF16,
            resid: Optional[torch.Tensor] = None, blocks=None, n_experts: int = 1, bn: int = 0):
    """``c = epilogue(a @ W.T)`` with ``W`` read as int4: ``w4b`` holds the W4B blocks of an ``[n][k]`` weight (or of
    ``n_experts`` stacked ones with ``blocks`` = the grouped form's tables).  The blocks are expanded to bf16 inside
    the kernel's shared-memory tiles (``bf16_rne((q - 8) * scale)``, the bits ``dequant_w4b`` produces); no bf16
    copy of the weight exists in global memory."""
    be = br0 = brn = nb = None
    max_blk = 0
    if blocks is not None:
        be, br0, brn, nb, max_blk = blocks
    rc = K.lib().b2_gemm_w4(K._p(a), K._p(w4b), K._p(c), a.shape[0], n, k, c.stride(0), epi, K._p(resid), K._p(be),
                            K._p(br0), K._p(brn), K._p(nb), max_blk, n_experts, bn, K._stream())
    K._check(rc, "gemm_w4")


def gemm_tp(a, b, c, epi: int, *, rs=None, rs_tpr: int = 1, ag_cnt=None, ag_expect: int = 0, bn: int = 0,
            a_scale=None, b_scale=None):
    """The tensor-parallel forms of the GEMM (bf16, or int8 when scales are given).

    ``epi=EPI_RS_PUSH`` with ``rs`` (a wire of ``parallel.symm``): row-parallel GEMM -> reduce-scatter -- the
    bf16 tiles are stored into the row owners' landing buffers over NVLink and counted there; ``c`` is unused.
    ``ag_cnt``: all-gather -> GEMM -- ``a`` is this GPU's copy of the gathered activations, whose rows arrive
    from their owners; m-tile ``i`` is loaded once ``ag_cnt[i] >= ag_expect``.  Returns arrivals per (source,
    m-tile) that complete a push."""
    m, k = a.shape
    n = b.shape[0]
    if bn == 0:
        bn = 256 if n % 256 == 0 else 128
    i8 = a_scale is not None
    rc = K.lib().b2_gemm_tc_tp(K._p(a), K._p(b), K._p(c), m, n, k, c.stride(0) if c is not None else n, int(i8), epi,
                               None, K._p(a_scale), K._p(b_scale), bn, K._p(rs.table) if rs is not None else None,
                               rs.rank if rs is not None else 0, rs.world if rs is not None else 1, rs_tpr,
                               K._p(ag_cnt), ag_expect, K._stream())
    K._check(rc, "gemm_tc_tp")
    return 4 * ((n + bn - 1) // bn)


def gemm_grouped_bf16(a, b, c, blocks, epi: int = EPI_BF16, bn: int = 0):
    """Grouped (MoE) GEMM: ``a`` ``[rows][K]`` expert-sorted rows, ``b`` ``[E][N][K]``; ``blocks`` is
    ``(blk_expert, blk_row0, blk_rows, n_blk, max_blk)`` device tables of 128-row blocks."""
    e, n, k = b.shape
    _launch(a, b, c, a.shape[0], n, k, c.stride(0), False, epi, blocks=blocks, n_experts=e, bn=bn)


def gemm_grouped_ep(a, b, c, blocks, epi: int, *, blk_wait=None, row_src=None, ret_table=None, bn: int = 0):
    """Expert-parallel forms of the grouped GEMM.  ``blk_wait``: block ``i`` of ``a`` (rows stored by the source
    ranks' dispatch kernels) is loaded once ``blk_wait[i] >= blk_rows[i]``.  ``epi=EPI_EP_RETURN``: every result
    row goes to the return buffer of the rank it came from (``row_src`` per row, ``ret_table`` of buffers)."""
    e, n, k = b.shape
    be, br0, brn, nb, max_blk = blocks
    rc = K.lib().b2_gemm_tc_ep(K._p(a), K._p(b), K._p(c), a.shape[0], n, k, c.stride(0) if c is not None else n, epi,
                               K._p(be), K._p(br0), K._p(brn), K._p(nb), max_blk, e, bn, K._p(blk_wait), K._p(row_src),
                               K._p(ret_table), K._stream())
    K._check(rc, "gemm_tc_ep")


def dequant_w4b(w4b: torch.Tensor, n: int, k: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """W4B -> bf16 ``[n][k]`` with ``bf16_rne((q - 8) * scale)``."""
    if out is None:
        out = torch.empty(n, k, dtype=torch.bfloat16, device=w4b.device)
    rc = K.lib().b2_dequant_w4b(K._p(w4b), K._p(out), n, k, K._stream())
    K._check(rc, "dequant_w4b")
    return out


def quant_rows_i8(x: torch.Tensor, q: Optional[torch.Tensor] = None, scale: Optional[torch.Tensor] = None):
    """Per-token symmetric int8: ``scale[m] = max|x[m]| / 127``."""
    m, k = x.shape
    if q is None:
        q = torch.empty(m, k, dtype=torch.int8, device=x.device)
    if scale is None:
        scale = torch.empty(m, dtype=torch.float32, device=x.device)
    rc = K.lib().b2_quant_rows_i8(K._p(x), K._p(q), K._p(scale), m, k, K._stream())
    K._check(rc, "quant_rows_i8")
    return q, scale
