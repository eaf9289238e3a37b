"""Bindings of the block drafter's candidate kernels (``csrc/dflash.cu``): top-K of a head's logits, exact rerank of
candidates against the target's lm_head rows, and the per-row pick (arg-max or keyed Gumbel-arg-max)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import lib as K

NO_IDX = 0x7FFFFFFF
DRAFT_SALT = 1 << 30


def topk(logits: torch.Tensor, rows: int, n: int, used: int, k: int, cand: torch.Tensor, value: torch.Tensor,
         id_table: Optional[torch.Tensor] = None, out_mult: float = 1.0, softcap: float = 0.0):
    """The ``k`` (<= 16) best of ``logits[r][:min(n, used)]`` per row, best first; ties go to the lower index, NaN never
    wins.  ``id_table`` maps indices to real token ids (a draft vocabulary); values are scaled by ``out_mult`` and then
    soft-capped (``softcap * tanh(v / softcap)``) when ``softcap`` > 0."""
    rc = K.lib().b2_df_topk(K._p(logits), rows, logits.stride(0), n, used, k, K._p(id_table), ctypes.c_float(out_mult),
                            ctypes.c_float(softcap), K._p(cand), K._p(value), K._stream())
    K._check(rc, "df_topk")


def rerank(head: torch.Tensor, x: torch.Tensor, rows: int, used: int, ids: torch.Tensor, c: int, k: int,
           cand: torch.Tensor, value: torch.Tensor):
    """Exact logits of each row's ``c`` candidate ids against the bf16 ``head`` rows (``x``: normalised hidden rows),
    then the ``k`` best of them in the same order rule."""
    rc = K.lib().b2_df_rerank(K._p(head), K._p(x), ctypes.c_longlong(x.stride(0)), rows, head.shape[1], used, K._p(ids), c, k,
                              K._p(cand), K._p(value), K._stream())
    K._check(rc, "df_rerank")


def select(cand: torch.Tensor, score: torch.Tensor, rows: int, k: int, temperature: float, seed: int, out_ids: torch.Tensor,
           out_chosen: torch.Tensor, ctrl: Optional[torch.Tensor] = None, pos0: int = 0,
           ctrl_tokens: Optional[torch.Tensor] = None):
    """One token per row out of its ``k`` candidates: the best score at temperature 0, else the arg-max of
    ``score / T + Gumbel`` whose noise is a function of (seed, position, token id) alone."""
    rc = K.lib().b2_df_select(K._p(cand), K._p(score), rows, k, ctypes.c_float(temperature), ctypes.c_uint(seed & 0xFFFFFFFF),
                              K._p(ctrl), pos0, K._p(out_ids), K._p(out_chosen), K._p(ctrl_tokens), K._stream())
    K._check(rc, "df_select")


def keyed_hash(seed: int, pos: int, token: int) -> int:
    fn = K.lib().b2_df_keyed_hash
    fn.restype = ctypes.c_uint
    return int(fn(ctypes.c_uint(seed & 0xFFFFFFFF), ctypes.c_uint(pos & 0xFFFFFFFF), ctypes.c_uint(token & 0xFFFFFFFF)))


def gumbel_of(seed: int, pos: int, token: int) -> float:
    """The noise the selector adds for (seed, position, token) -- the host twin of the kernel's arithmetic (fp32)."""
    import numpy as np
    h = keyed_hash(seed, (pos + DRAFT_SALT) & 0xFFFFFFFF, token)
    u = np.float32((np.float32(h >> 8) + np.float32(0.5)) * np.float32(1.0 / 16777216.0))
    return float(-np.log(-np.log1p(-u, dtype=np.float32), dtype=np.float32))
