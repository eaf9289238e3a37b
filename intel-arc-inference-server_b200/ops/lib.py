"""ctypes bindings of the sm_100a kernel library.

The library exports plain C entry points that take raw device pointers and a
``cudaStream_t``; the wrappers here pass ``tensor.data_ptr()`` and the current
torch stream, so the kernels are captured by ``torch.cuda.CUDAGraph`` like any
other work on that stream.  There is no PyTorch fallback: on a machine with a
GPU a missing library is an error, never a silent eager path.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build as _build

_lib: Optional[ctypes.CDLL] = None
_UNITS = ("gemv", "decode", "gemm", "attn", "attnrows", "moe", "comm", "ep", "spec", "sampler", "gdn", "mega", "dflash")

# Control block layout (int32 words) -- mirrors decode_ops.cu
CTRL_N_ROWS = 0
CTRL_ROW_REQ = 16
CTRL_ROW_POS = 80
CTRL_CUR_TOKEN = 144
CTRL_OUT_TOKEN = 208
CTRL_OUT_VALUE = 272
CTRL_ROW_BLOCK = 336     # [64] 1: the row attends to every position of its request's rows (block drafter)
CTRL_WORDS = 512
MAX_ROWS = 64

launch_count = 0    # kernels launched through this module (bench.py reports it)


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build.LIB
        if not os.path.exists(path) or not _build.is_current():
            try:
                path = _build.build()
            except Exception as e:  # no nvcc on this machine: use the shipped binary if there is one
                if not os.path.exists(_build.LIB):
                    raise KernelError(f"kernel library is not built and cannot be built here: {e}") from e
                path = _build.LIB
        _lib = ctypes.CDLL(path)
    return _lib


def available() -> bool:
    return torch.cuda.is_available()


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc: int, what: str):
    global launch_count
    launch_count += 1
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


def status() -> dict:
    """Reads every translation unit's status word; {} when no kernel recorded an error."""
    out = {}
    L = lib()
    for u in _UNITS:
        fn = getattr(L, f"b2_status_{u}", None)
        if fn is None:
            continue
        buf = (ctypes.c_uint * 4)()
        rc = fn(buf)
        if rc != 0:
            raise KernelError(f"status read failed ({u}): cuda error {rc}")
        if buf[0]:
            out[u] = {"code": hex(buf[0]), "detail": buf[1], "count": buf[2]}
    return out


def status_clear():
    L = lib()
    for u in _UNITS:
        fn = getattr(L, f"b2_status_clear_{u}", None)
        if fn is not None:
            fn()
    for t in _fail_words.values():
        t.zero_()


_fail_words: dict = {}      # device index -> pinned host word the kernels' first error code is also written to


def arm_failure_word() -> torch.Tensor:
    """Gives every kernel unit of the current device a word in pinned host memory for its first bounded-wait
    failure, so that ``failed_fast()`` after a step costs a host read, not a copy per unit.  Idempotent."""
    dev = torch.cuda.current_device()
    if dev not in _fail_words:
        word = torch.zeros(1, dtype=torch.int32).pin_memory()
        L = lib()
        for u in _UNITS:
            fn = getattr(L, f"b2_status_hostflag_{u}", None)
            if fn is not None:
                rc = fn(ctypes.c_void_p(word.data_ptr()))
                if rc != 0:
                    raise KernelError(f"cannot arm the failure word ({u}): cuda error {rc}")
        _fail_words[dev] = word
    return _fail_words[dev]


def failed_fast() -> bool:
    """True when some kernel of the current device has recorded a failure since the last ``status_clear()``
    (meaningful after a synchronize; needs ``arm_failure_word()`` once per device)."""
    w = _fail_words.get(torch.cuda.current_device()) if torch.cuda.is_available() else None
    return w is not None and int(w[0]) != 0


def check_status():
    s = status()
    if s:
        raise KernelError(f"device kernels reported bounded-wait failures: {s}")


# ----------------------------------------------------------------------------- decode ops
def gemv_splits(n: int, k: int) -> int:
    return lib().b2_gemv_w4_splits(n, k)


def gemv_w4(w4b: torch.Tensor, x: torch.Tensor, out: torch.Tensor, m: int, n: int, k: int, splits: int,
            x_mode: int = 0, s_in: int = 1, x_slice: int = 0, ldx: Optional[int] = None):
    """``out[s][m][n]`` fp32 partial sums of ``x @ W^T`` for a W4B weight.

    ``x_mode`` 0: ``x`` is bf16 ``[m][k]``.  ``x_mode`` 1: ``x`` is fp32 ``[s_in][m][2k]``
    split-K slices of a gate‖up projection (interleave16); the kernel folds them and applies
    SiLU(gate) * up while staging the activations.
    """
    if ldx is None:
        ldx = k if x_mode == 0 else 2 * k
    rc = lib().b2_gemv_w4(_p(w4b), _p(x), _p(out), m, n, k, splits, ldx, n, x_mode, s_in,
                          ctypes.c_longlong(x_slice), _stream())
    _check(rc, "gemv_w4")


def gemv_w4_fused(w4b, x, out, m, n, k, splits, *, x_mode=0, s_in=1, x_slice=0, ldx=None, norm_w=None, norm_ssq=None,
                  norm_eps=0.0, fold_tickets=None, fold_resid=None, fold_ssq=None, tp=None, tp_mcap=0):
    """The GEMV with its neighbours folded in.  ``x_mode`` 2: ``x`` is the bf16 residual stream and the
    kernel applies RMSNorm (``norm_w``, per-block sums of squares ``norm_ssq``) while staging it.
    ``fold_*``: the last split CTA of each 128-column block adds the split-K slices to ``fold_resid``
    in place and leaves that block's sum of squares in ``fold_ssq`` ``[m][n/128]``.  ``tp`` (a wire of
    ``parallel.symm``) makes the fold all-reduce the ranks' partial sums over NVLink first."""
    if ldx is None:
        ldx = 2 * k if x_mode == 1 else k
    tpw = tp is not None and tp.world > 1
    rc = lib().b2_gemv_w4_fused(_p(w4b), _p(x), _p(out), m, n, k, splits, ldx, x_mode, s_in, ctypes.c_longlong(x_slice),
                                _p(norm_w), _p(norm_ssq), ctypes.c_float(norm_eps), _p(fold_tickets), _p(fold_resid),
                                _p(fold_resid), _p(fold_ssq), _p(tp.table) if tpw else None, _p(tp.epoch) if tpw else None,
                                tp.world if tpw else 1, tp.rank if tpw else 0, tp_mcap, _stream())
    _check(rc, "gemv_w4_fused")


def gemv_w4_qkv_rope(w4b, x, out, m, k, splits, *, x_mode, norm_w, norm_ssq, norm_eps, tickets, q_out, cos_t, sin_t, ctrl,
                     block_table, max_blocks, n_q, n_kv, k_plane, v_plane):
    """The qkv projection whose last split CTA per head also sums the slices, applies RoPE and writes the q rows / the
    rows' slots of the paged bf16 cache (head size 128): the separate RoPE + append launch disappears."""
    rc = lib().b2_gemv_w4_qkv_rope(_p(w4b), _p(x), _p(out), m, k, splits, k, x_mode, _p(norm_w), _p(norm_ssq),
                                   ctypes.c_float(norm_eps), _p(tickets), _p(q_out), _p(cos_t), _p(sin_t), _p(ctrl),
                                   _p(block_table), max_blocks, n_q, n_kv, _p(k_plane), _p(v_plane), _stream())
    _check(rc, "gemv_w4_qkv_rope")


def quant_slots(m: int) -> int:
    """Token slots per 64-k group in ``xq_gs`` for ``m`` rows: 8 per row tile of the GEMV (8, 16, 32 or 64)."""
    return 8 if m <= 8 else (16 if m <= 16 else (32 if m <= 32 else 64))


def quant_x(x, m, k, xq, xq_gs, *, x_mode=0, s_in=1, x_slice=0, ldx=None, norm_w=None, norm_ssq=None, norm_eps=0.0):
    """Quantises ``m`` activation rows once for ``gemv_w4_fused(..., x_mode=3)``: 15-bit two-limb integers per
    64-k group in the GEMV's operand order (``xq``) and the groups' {scale, -8 sum} (``xq_gs``)."""
    if ldx is None:
        ldx = 2 * k if x_mode == 1 else k
    if m > 64 or xq.numel() * xq.element_size() < m * (k // 64) * 128 \
            or xq_gs.numel() * xq_gs.element_size() < quant_slots(m) * (k // 64) * 8:
        raise ValueError(f"quant_x: buffers too small for {m} rows of {k} (xq_gs holds {quant_slots(m)} token slots per group)")
    rc = lib().b2_quant_x(_p(x), m, k, ldx, x_mode, s_in, ctypes.c_longlong(x_slice), _p(norm_w), _p(norm_ssq),
                          ctypes.c_float(norm_eps), _p(xq), _p(xq_gs), _stream())
    _check(rc, "quant_x")


def decode_mega_sms() -> int:
    """CTAs of the whole-step decode kernel: one per SM of the current device."""
    n = lib().b2_decode_mega_sms()
    if n <= 0:
        raise KernelError("decode_mega: cannot read the SM count of the current device")
    return n


def decode_mega_plan(n_cta: int, m: int, h: int, n_q: int, n_kv: int, ffn: int) -> Optional[dict]:
    """Schedule constants of the whole-step decode kernel for ``m`` rows of this shape (pure host arithmetic; also
    checks that the CTAs' runs cover every ring stage of every linear exactly once).  None: the kernel does not
    cover the shape."""
    out = (ctypes.c_int * 5)()
    pf = ctypes.c_longlong(0)
    rc = lib().b2_decode_mega_plan(n_cta, m, h, n_q, n_kv, ffn, out, ctypes.byref(pf))
    if rc in (-1, -2, -3):
        return None
    if rc != 0:
        raise KernelError(f"decode_mega_plan: schedule self-check failed with code {rc}")
    return {"rows": out[0], "nsplit": out[1], "max_nb": out[2], "stages": out[3], "smem": out[4], "part_floats": pf.value}


def decode_mega(layers_table, n_layers, m, h, n_q, n_kv, ffn, ctrl, block_table, max_blocks, num_pages, planes, embed,
                vocab, flag, cos_t, sin_t, k_cache, v_cache, resid, ssq, xq, gs, part, tickets, q, o_part, ml_part,
                attn_tickets, bar, eps, scale, span_pages, n_cta, n_phases: int = 0, cooperative: bool = True, dbg=None):
    """Embedding + ``n_layers`` dense layers of one decode / verify step (``m`` <= 8 consecutive rows of one request)
    in one launch.  ``xq`` / ``gs``: three quantised-row buffers and their group scales (hidden-wide, o-proj input,
    down-proj input); ``bar``: three zeroed uint32 words.  ``n_phases`` > 0 stops after that many phases (1 embed +
    5 per layer: qkv, attention, o, gate||up, down) -- a debugging cut."""
    rc = lib().b2_decode_mega(_p(layers_table), n_layers, m, h, n_q, n_kv, ffn, _p(ctrl), _p(block_table), max_blocks,
                              num_pages, planes, _p(embed), vocab, _p(flag), _p(cos_t), _p(sin_t), _p(k_cache), _p(v_cache),
                              _p(resid), _p(ssq), _p(xq[0]), _p(xq[1]), _p(xq[2]), _p(gs[0]), _p(gs[1]), _p(gs[2]),
                              _p(part), _p(tickets), _p(q), _p(o_part), _p(ml_part), _p(attn_tickets), _p(bar),
                              ctypes.c_float(eps), ctypes.c_float(scale), span_pages, n_phases, n_cta,
                              1 if cooperative else 0, _p(dbg), _stream())
    _check(rc, "decode_mega")


def resid_norm(mode: int, m: int, h: int, w: torch.Tensor, eps: float, resid_out: torch.Tensor,
               x_out: Optional[torch.Tensor], *, embed=None, ctrl=None, vocab=0, resid_in=None, part=None,
               part_slice=0, splits=0, flag=None):
    rc = lib().b2_resid_norm(_p(embed), _p(ctrl), _p(resid_in), _p(part), ctypes.c_longlong(part_slice), splits, m, h,
                             mode, vocab, _p(w), ctypes.c_float(eps), _p(resid_out), _p(x_out), _p(flag), _stream())
    _check(rc, "resid_norm")


def draft_front(embed, ctrl, vocab, hidden, w_e, w_h, eps, m, h, xcat, flag=None):
    """Input of a draft head's fc projection for ``m`` rows: ``xcat[i] = [norm(embed[cur_token[i]]) | norm(hidden[i])]``
    (bf16 ``[m][2h]``); the tokens are read from the control block."""
    rc = lib().b2_draft_front(_p(embed), _p(ctrl), vocab, _p(hidden), ctypes.c_longlong(hidden.stride(0)), _p(w_e),
                              _p(w_h), ctypes.c_float(eps), m, h, _p(xcat), _p(flag), _stream())
    _check(rc, "draft_front")


def rope_append(qkv_part, slice_elems, splits, m, ctrl, block_table, max_blocks, cos_t, sin_t, n_q, n_kv, d, q_out,
                k_cache, v_cache, k_scale=None, v_scale=None, kv_int8=False, req=0, pos0=0):
    """With ``ctrl`` None the ``m`` rows are consecutive positions ``pos0..`` of request ``req`` (prompt chunks)."""
    rc = lib().b2_rope_append(_p(qkv_part), ctypes.c_longlong(slice_elems), splits, m, _p(ctrl), _p(block_table),
                              max_blocks, _p(cos_t), _p(sin_t), n_q, n_kv, d, _p(q_out), _p(k_cache), _p(v_cache),
                              _p(k_scale), _p(v_scale), int(kv_int8), req, pos0, _stream())
    _check(rc, "rope_append")


def attn_decode(q, k_cache, v_cache, block_table, ctrl, o_part, ml_part, out, m, n_q, n_kv, d, nsplit, max_blocks,
                scale, k_scale=None, v_scale=None, kv_int8=False, tickets=None):
    """Split-KV decode attention.  With ``tickets`` (zeroed int32 ``[rows][n_kv]``) the last split CTA of
    each (row, KV head) merges the splits inside the kernel; without, a second kernel merges."""
    global launch_count
    rc = lib().b2_attn_decode(_p(q), _p(k_cache), _p(v_cache), _p(k_scale), _p(v_scale), _p(block_table), _p(ctrl),
                              _p(o_part), _p(ml_part), _p(out), m, n_q, n_kv, d, nsplit, max_blocks,
                              ctypes.c_float(scale), int(kv_int8), _p(tickets), _stream())
    launch_count += 0 if tickets is not None else 1
    _check(rc, "attn_decode")


def attn_rows(q, k_cache, v_cache, block_table, ctrl, o_part, ml_part, out, tickets, m, n_q, n_kv, d, nsplit,
              max_blocks, scale, span_pages: int = 0, k_scale=None, v_scale=None, kv_int8: bool = False, window: int = 0,
              one_request: bool = False, xq=None, xq_gs=None):
    """Decode / verify attention that serves consecutive rows of one request together on the tensor cores
    (bf16 or int8 KV, head size 128); same split-KV partial buffers and in-kernel merge as ``attn_decode``.
    ``window`` > 0: every row attends to its last ``window`` positions only; ``window`` = -1: the rows are a block whose
    rows all attend to every position up to the block's last one (no causal mask inside the block).
    ``one_request``: the caller knows that all ``m`` rows are one request's, at consecutive positions; the launch then
    has one CTA column per group of rows instead of one per row (most of which would leave at once).
    ``xq`` / ``xq_gs`` (with ``tickets=None``): the merge also writes the rows in the quantised form of ``quant_x`` for
    K = n_q * d, so that the o projection's GEMV can read them without that launch."""
    rc = lib().b2_attn_rows(_p(q), _p(k_cache), _p(v_cache), _p(k_scale), _p(v_scale), 1 if kv_int8 else 0,
                            _p(block_table), _p(ctrl), _p(o_part), _p(ml_part),
                            _p(out), _p(tickets), m, n_q, n_kv, d, nsplit, max_blocks, ctypes.c_float(scale), span_pages,
                            k_cache.numel() // (n_kv * 16 * d), window, 1 if one_request else 0, _stream())
    _check(rc, "attn_rows")
    if tickets is None:     # many rows: the merge is its own launch, one CTA per row and head
        if xq is not None:
            rc = lib().b2_attn_merge_quant(_p(o_part), _p(ml_part), _p(out), m, n_q, nsplit, d, _p(xq), _p(xq_gs),
                                           quant_slots(m), _stream())
        else:
            rc = lib().b2_attn_merge(_p(o_part), _p(ml_part), _p(out), m, n_q, nsplit, d, _stream())
        _check(rc, "attn_merge")


def gdn_conv(part, splits, m, n, conv_ch, ctrl, conv_w, conv_state, act, slot: int = -1):
    """Folds the split-K partials of a gated delta-net layer's input projection into ``act`` [m][n]; the first
    ``conv_ch`` columns pass through the slot's 4-tap causal convolution (state [slots][conv_ch][3]) and SiLU.
    ``ctrl`` maps rows to slots (decode / verify rows); ``ctrl=None`` with ``slot``: a prompt chunk of one slot."""
    _check(lib().b2_gdn_conv(_p(part), splits, m, n, conv_ch, _p(ctrl), slot, _p(conv_w), _p(conv_state), _p(act),
                             _stream()), "gdn_conv")


def gdn_step(act, m, n, n_k, n_v, head_dim, ctrl, a_log, dt_bias, norm_w, eps, state, out, slot: int = -1):
    """One recurrent step per row and value head over ``state`` [slots][n_v][128][128]; ``out`` [m][n_v * 128] bf16
    is the gated, normalised read-out."""
    _check(lib().b2_gdn_step(_p(act), m, n, n_k, n_v, head_dim, _p(ctrl), slot, _p(a_log), _p(dt_bias), _p(norm_w),
                             ctypes.c_float(eps), _p(state), _p(out), _stream()), "gdn_step")


def gdn_chunk(act, m, n, n_k, n_v, head_dim, slot, a_log, dt_bias, norm_w, eps, state, out):
    """A prompt chunk of ``m`` rows of ``slot`` through a gated delta-net layer's recurrence (after ``gdn_conv``):
    normalisation and gates in parallel over the rows, one sequential scan per value head, gated norm in parallel.
    ``act`` is overwritten with intermediate values."""
    _check(lib().b2_gdn_chunk(_p(act), m, n, n_k, n_v, head_dim, slot, _p(a_log), _p(dt_bias), _p(norm_w),
                              ctypes.c_float(eps), _p(state), _p(out), _stream()), "gdn_chunk")


def gdn_wy_block_bytes() -> int:
    """Workspace bytes the chunked scan needs per (64-row chunk, value head)."""
    return int(lib().b2_gdn_wy_block_bytes())


def gdn_chunk_wy(act, m, n, n_k, n_v, head_dim, slot, a_log, dt_bias, norm_w, eps, state, out, ws):
    """``gdn_chunk`` with the recurrence in its chunked form on the tensor cores: per 64-row chunk the rows' deltas come
    from a triangular solve that does not involve the state (all chunks in parallel), and the scan over the chunks
    is four small matrix products per chunk and value head.  ``ws``: uint8 workspace of
    ``ceil(m / 64) * n_v * gdn_wy_block_bytes()`` bytes."""
    _check(lib().b2_gdn_chunk_wy(_p(act), m, n, n_k, n_v, head_dim, slot, _p(a_log), _p(dt_bias), _p(norm_w),
                                 ctypes.c_float(eps), _p(state), _p(out), _p(ws),
                                 ctypes.c_longlong(ws.numel() * ws.element_size()), _stream()), "gdn_chunk_wy")


def sample_rows(logits, m, n_valid, temperature, top_k, top_p, seed, token, status, penalty=None, hist=None,
                hist_len=None, kept=None):
    """One token per row of ``logits`` [m][ld] by the host sampler's rule (temperature, top-k, top-p, optional
    repetition penalty over ``hist`` [m][cap] ids, ``seed`` uint64 per row as int64 storage).  ``status[i] = 1``
    marks a row that must be sampled on the host (filtered set wider than 1024 candidates)."""
    rc = lib().b2_sample_rows(_p(logits), m, logits.stride(0) if logits.dim() == 2 else logits.numel() // m, n_valid,
                              _p(temperature), _p(top_k), _p(top_p), _p(seed), _p(penalty), _p(hist), _p(hist_len),
                              hist.shape[1] if hist is not None else 0, _p(token), _p(status), _p(kept), _stream())
    _check(rc, "sample_rows")


def kv_convert(k16, v16, table16, k8, v8, ks, vs, table8, pos0, tokens, n_kv, d, to_int8: bool):
    """Rows of positions ``pos0 .. pos0 + tokens`` between bf16 pages (``table16``) and int8 pages + per-row scales
    (``table8``), one direction per call."""
    rc = lib().b2_kv_convert(_p(k16), _p(v16), _p(table16), _p(k8), _p(v8), _p(ks), _p(vs), _p(table8), pos0, tokens,
                             n_kv, d, 1 if to_int8 else 0, _stream())
    _check(rc, "kv_convert")


def head_ncand(n: int) -> int:
    return lib().b2_head_ncand(n)


def head_gemv(w, x, out, m, n, k, cand_val=None, cand_idx=None, n_valid=None, wscale=None):
    global launch_count
    rc = lib().b2_head_gemv(_p(w), _p(wscale), int(wscale is not None), _p(x), _p(out), m, n, k, n, _p(cand_val),
                            _p(cand_idx), n if n_valid is None else n_valid, _stream())
    launch_count += (m + 7) // 8 - 1
    _check(rc, "head_gemv")


def argmax_finish(cand_val, cand_idx, ncand, m, ctrl, advance: bool):
    rc = lib().b2_argmax_finish(_p(cand_val), _p(cand_idx), ncand, m, _p(ctrl), int(advance), _stream())
    _check(rc, "argmax_finish")


def argmax_finish_tp(cand_val, cand_idx, ncand, m, vocab_offset, ctrl, advance: bool, wire, mcap: int):
    """Vocabulary-parallel arg-max: local reduce, exchange over the wire, merge on the device."""
    rc = lib().b2_argmax_finish_tp(_p(cand_val), _p(cand_idx), ncand, m, vocab_offset, _p(ctrl), 1 if advance else 0,
                                   _p(wire.table), _p(wire.epoch), wire.world, wire.rank, mcap, _stream())
    _check(rc, "argmax_finish_tp")


def allreduce_rows(x, out, m, n, wire, mcap: int):
    """One-shot all-reduce of fp32 ``x[m][n]`` into ``out`` (rank-order fold, same bits on every rank)."""
    rc = lib().b2_allreduce_rows(_p(x), _p(out), m, n, _p(wire.table), _p(wire.epoch), wire.world, wire.rank, mcap,
                                 _stream())
    _check(rc, "allreduce_rows")


def rs_fold(rs, rs_expect: int, nsrc: int, done, resid, norm_w, eps: float, xw, h: int, tpr: int, c: int):
    """Owner side of GEMM -> reduce-scatter: wait for the m-tiles' arrivals, fold the partial sums and the
    residual in rank order, RMSNorm, push the rows into every rank's gathered activations (wire ``xw``)."""
    rc = lib().b2_rs_fold(_p(rs.land), _p(rs.flags), _p(done), rs_expect, nsrc, _p(resid), _p(norm_w),
                          ctypes.c_float(eps), _p(xw.table), xw.world, xw.rank, h, tpr, c, _stream())
    _check(rc, "rs_fold")


def wire_wait(cnt: torch.Tensor, expect: int):
    """Stream-ordered bounded wait until ``cnt[0] >= expect``."""
    rc = lib().b2_wire_wait(_p(cnt), expect, _stream())
    _check(rc, "wire_wait")


def attn_prefill(q, k_cache, v_cache, block_table_row, out, c, pos0, n_q, n_kv, d, num_pages, max_blocks, scale,
                 window: int = 0):
    """Causal flash attention of a prompt chunk (``c`` rows at positions ``pos0..``) over the paged bf16 cache;
    ``window`` > 0: every row attends to its last ``window`` positions only."""
    rc = lib().b2_attn_prefill(_p(q), _p(k_cache), _p(v_cache), _p(block_table_row), _p(out), c, pos0, n_q, n_kv, d,
                               num_pages, max_blocks, ctypes.c_float(scale), window, _stream())
    _check(rc, "attn_prefill")
