"""GPU decoder: the layer walk of one decode / verify step over the sm_100a kernels.

``DecoderModel.step_rows(M)`` enqueues one forward pass for M rows (M <= 64)
on the current stream; every kernel reads row positions, request slots and input
tokens from the device control block, so the enqueued sequence can be captured
once per M in a CUDA graph and replayed without host writes -- the role of the
reference's capture walk (src/runtime/capture.cc:1332-1510: gdn_layer / fa_layer /
mlp / head) with CUDA graphs in place of closed Level Zero command lists.

Launches per dense layer: resid_norm, qkv GEMV, rope_append, attn_decode,
attn_merge, o GEMV, resid_norm, gate_up GEMV, down GEMV (SiLU*up folded into its
activation load) = 9; the reference's list has 12 per layer (774 for 64 layers).
"""
from __future__ import annotations

import os

import math
from dataclasses import dataclass
from typing import List, Optional

import torch

from ..ops import lib as K
from .config import ModelConfig
from .oracle import rope_tables
from .weights import ModelWeights, LayerWeights, QLinear


@dataclass
class LinearPlan:
    ql: QLinear
    splits: int
    part: torch.Tensor     # fp32 [splits * max_rows * n] scratch


class StepBuffers:
    """Activations and split-K scratch of one step, sized once for ``max_rows``."""

    def __init__(self, cfg: ModelConfig, max_rows: int, nsplit_attn: int, device, head_rows: Optional[int] = None):
        bf, f32 = torch.bfloat16, torch.float32
        h = cfg.hidden
        head_rows = cfg.vocab if head_rows is None else head_rows
        self.max_rows = max_rows
        self.resid = torch.zeros(max_rows, h, dtype=bf, device=device)
        self.x = torch.zeros(max_rows, h, dtype=bf, device=device)
        self.q = torch.zeros(max_rows, cfg.q_dim, dtype=bf, device=device)
        self.attn_out = torch.zeros(max_rows, cfg.q_dim, dtype=bf, device=device)
        self.o_part = torch.zeros(max_rows * cfg.n_q_heads * nsplit_attn * cfg.head_dim, dtype=f32, device=device)
        self.ml_part = torch.zeros(max_rows * cfg.n_q_heads * nsplit_attn * 2, dtype=f32, device=device)
        self.logits = torch.zeros(max_rows, head_rows, dtype=f32, device=device)
        self.ncand = K.head_ncand(head_rows)
        self.cand_val = torch.zeros(max_rows * self.ncand, dtype=f32, device=device)
        self.cand_idx = torch.zeros(max_rows * self.ncand, dtype=torch.int32, device=device)
        self.flag = torch.zeros(4, dtype=torch.int32, device=device)
        self.tickets = torch.zeros(max_rows * cfg.n_kv_heads, dtype=torch.int32, device=device)
        self.fold_tickets = torch.zeros((h + 127) // 128, dtype=torch.int32, device=device)
        self.qkv_tickets = torch.zeros(max((cfg.qkv_dim + 127) // 128, 8), dtype=torch.int32, device=device)   # per head of the qkv projection
        self.ssq = torch.zeros(max_rows * ((h + 127) // 128), dtype=f32, device=device)
        kmax = max(2 * h, cfg.q_dim, cfg.ffn, cfg.expert_ffn, cfg.shared_ffn, cfg.gdn_value_dim)
        if cfg.n_gdn_layers:
            self.gdn_act = torch.zeros(max_rows, cfg.gdn_proj_dim, dtype=f32, device=device)
            self.gdn_out = torch.zeros(max_rows, cfg.gdn_value_dim, dtype=bf, device=device)
        self.xq = torch.zeros(max_rows * (kmax // 64) * 128, dtype=torch.uint8, device=device)    # pre-quantised rows
        self.xq_gs = torch.zeros(K.quant_slots(max_rows) * (kmax // 64) * 2, dtype=torch.int32, device=device)   # {scale, -8 sum} per group and token slot
        self._parts = {}
        self.device = device

    def part(self, name: str, splits: int, n: int) -> torch.Tensor:
        key = (name, splits, n)
        if key not in self._parts:
            self._parts[key] = torch.zeros(splits * self.max_rows * n, dtype=torch.float32, device=self.device)
        return self._parts[key]


def attn_splits(n_kv_heads: int, depth: int) -> int:
    """KV splits of the decode attention for contexts around ``depth``: KV heads x splits CTAs fill the 2 x 148
    resident slots of the multi-row kernel in one wave, a split keeps at least 64 keys (the merge reads every
    split), and the partial buffers hold at most 64 splits.  Measured on the 27B shape (8 KV heads), 16 layers:
    depth 1024 1.41 / 1.43 / 1.45 ms with 16 / 32 / 37 splits, depth 4096 1.50 / 1.49 ms with 32 / 37, depth
    32768 (8 layers) 1.10 / 1.17 ms with 37 / 64."""
    return max(4, min(64, 296 // max(1, n_kv_heads), max(depth, 64) // 64))


class KVCache:
    """Paged KV: per layer ``[page][kv_head][16][D]`` for K and for V (bf16 or int8 + fp32 scales)."""

    def __init__(self, cfg: ModelConfig, n_layers: int, num_pages: int, device, kv_dtype: str = "bf16", n_slots: int = 1):
        self.kv_int8 = kv_dtype == "int8"
        dt = torch.int8 if self.kv_int8 else torch.bfloat16
        self.num_pages = num_pages
        self.n_layers = n_layers                # layers addressed by ``layer`` (trunk + draft-head layers)
        # gated delta-net layers hold no KV: only the others get a plane of the cache
        self._plane = {}
        for li in range(n_layers):
            if not cfg.is_gdn_layer(li):
                self._plane[li] = len(self._plane)
        planes = max(1, len(self._plane))
        self.k = torch.zeros(planes, num_pages, cfg.n_kv_heads, cfg.page_size, cfg.head_dim, dtype=dt, device=device)
        self.v = torch.zeros_like(self.k)
        if self.kv_int8:
            self.k_scale = torch.zeros(planes, num_pages, cfg.n_kv_heads, cfg.page_size, dtype=torch.float32, device=device)
            self.v_scale = torch.zeros_like(self.k_scale)
        else:
            self.k_scale = self.v_scale = None
        # gated delta-net layers keep, per slot, the last three convolution inputs and one fp32 state per value head
        self.gdn_conv = self.gdn_state = None
        if cfg.n_gdn_layers:
            g = cfg.n_gdn_layers
            self.gdn_conv = torch.zeros(g, n_slots, cfg.gdn_conv_channels, 3, dtype=torch.float32, device=device)
            self.gdn_state = torch.zeros(g, n_slots, cfg.gdn_v_heads, cfg.gdn_head_dim, cfg.gdn_head_dim,
                                         dtype=torch.float32, device=device)

    def reset_slot(self, slot: int):
        if self.gdn_conv is not None:
            self.gdn_conv[:, slot].zero_()
            self.gdn_state[:, slot].zero_()

    def layer(self, li: int):
        j = self._plane[li]
        ks = self.k_scale[j] if self.kv_int8 else None
        vs = self.v_scale[j] if self.kv_int8 else None
        return self.k[j], self.v[j], ks, vs


class DecoderModel:
    def __init__(self, weights: ModelWeights, max_rows: int = 64, max_pos: int = 8192, nsplit_attn: int = 32,
                 int8_head: bool = False, tp=None, nccl=None):
        """``tp``: the wires of a tensor-parallel group (``parallel.symm.TpWires``); ``weights`` then hold this
        rank's shard (``cfg.tp_shard``) and ``lm_head`` this rank's rows of the vocabulary."""
        self.w = weights
        self.cfg = cfg = weights.cfg
        self.device = weights.embed.device
        self.max_rows = max_rows
        self.nsplit_attn = nsplit_attn
        self.tp = tp if tp is not None and tp.world > 1 else None
        # ``nccl`` = (rank, world, group): the comparison path -- the same kernels, unfused, with NCCL
        # all-reduces after the row-parallel linears and an NCCL gather for the arg-max
        self.nccl = nccl if nccl is not None and nccl[1] > 1 else None
        if self.nccl is not None:
            self.vocab_offset_nccl = self.nccl[0] * ((cfg.vocab + self.nccl[1] - 1) // self.nccl[1])
        self.head_rows = weights.lm_head.shape[0]
        self.vocab_offset = 0
        if self.tp is not None:
            per = (cfg.vocab + tp.world - 1) // tp.world
            self.vocab_offset = tp.rank * per
            if max_rows > tp.mcap:
                raise ValueError(f"max_rows {max_rows} exceeds the wires' row capacity {tp.mcap}")
        self.buf = StepBuffers(cfg, max_rows, nsplit_attn, self.device, self.head_rows)
        cos, sin = rope_tables(cfg.head_dim, cfg.rope_theta, max_pos)
        self.cos_t, self.sin_t = cos.to(self.device).contiguous(), sin.to(self.device).contiguous()
        self.max_pos = max_pos
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        self.int8_head = int8_head
        if int8_head and weights.lm_head_i8 is None:
            wf = weights.lm_head.float()
            sc = wf.abs().amax(dim=1).clamp_min(1e-8) / 127.0
            weights.lm_head_i8 = (torch.round(wf / sc[:, None]).clamp_(-127, 127).to(torch.int8).contiguous(), sc.contiguous())
        self._splits = {}
        # from this many rows up the activations are quantised once by their own kernel instead of in every
        # CTA of the GEMV (whose prologue repeats the rows' work per 128 output columns)
        self.prequant_rows = int(os.environ.get("B2_PREQUANT_ROWS", "3"))
        self.merge_quant = os.environ.get("B2_MERGE_QUANT", "1") == "1"   # the attention merge writes the o projection's quantised rows
        self.attn_rows_min = int(os.environ.get("B2_ATTN_ROWS_MIN", "1"))
        self.rows_one_request = False    # set by the engine around a step whose rows are one request's, consecutive
        self.block_rows = False      # set by a block drafter around its layers: flagged rows attend non-causally
        self.attn_merge_inkernel_rows = int(os.environ.get("B2_ATTN_MERGE_INKERNEL_ROWS", "0"))
        # fixed KV split spans make a row's attention bits independent of the rows it is verified with (speculation
        # then reproduces plain decoding exactly); off, the splits adapt to the context (fastest at any depth)
        self.attn_fixed_spans = False
        self.fused = self.nccl is None and os.environ.get("B2_UNFUSED", "0") != "1"     # dense layers: residual folds and norms ride inside the GEMVs
        # whole-step kernel (one launch for embedding + all dense layers of a one-request step of up to 8 rows).
        # Off unless asked for (B2_MEGA=1, or the attribute): on the 27B shape at depth 4096 it takes 6.6 ms per
        # step against 5.1 ms for the launch-per-linear walk, whose several CTAs per SM hide the latency of the
        # fold / barrier chain between two linears better than one resident CTA per SM does
        self.use_mega = os.environ.get("B2_MEGA", "0") == "1"
        # the qkv projection's last split CTA per head can apply RoPE and append K / V itself (bf16 cache, head size
        # 128): one launch fewer per layer.  Measured neutral on the 27B step (4.73 vs 4.70 ms: the fold's latency
        # replaces the small kernel's), so it is opt-in
        self.rope_fold = os.environ.get("B2_ROPE_FOLD", "0") == "1"
        self.ep = None      # parallel.ep.EpMoe with the row form enabled: MoE layers of a decode step go through it
        self.mega_cooperative = os.environ.get("B2_MEGA_COOP", "1") != "0"
        self._mega_bufs = {}
        self._mega_tables = {}
        self._mega_shared = None
        if self.nccl is not None:
            self._red = torch.zeros(max_rows * cfg.hidden, dtype=torch.float32, device=self.device)
            self._gather = torch.zeros(self.nccl[1], max_rows, 2, dtype=torch.float32, device=self.device)

    # ------------------------------------------------------------------ pieces
    def _gemv(self, name: str, ql: QLinear, x: torch.Tensor, m: int, x_mode=0, s_in=1, x_slice=0):
        key = (ql.n, ql.k)
        s = self._splits.get(key)
        if s is None:
            s = self._splits[key] = K.gemv_splits(ql.n, ql.k)
        part = self.buf.part(name, s, ql.n)
        if m >= self.prequant_rows:
            b = self.buf
            K.quant_x(x, m, ql.k, b.xq, b.xq_gs, x_mode=x_mode, s_in=s_in, x_slice=x_slice)
            K.gemv_w4_fused(ql.w4b, b.xq, part, m, ql.n, ql.k, s, x_mode=3, norm_ssq=b.xq_gs)
        else:
            K.gemv_w4(ql.w4b, x, part, m, ql.n, ql.k, s, x_mode=x_mode, s_in=s_in, x_slice=x_slice)
        return part, s

    def _attention(self, m: int, ctrl, block_table, max_blocks, kv: KVCache, kc, vc, ks, vs, window: int = 0,
                   quant_out: bool = False) -> bool:
        """Split-KV attention of the step's rows into ``buf.attn_out``.  Head size 128 (bf16 or int8 KV) goes to the
        tensor-core kernel that serves a request's consecutive rows together; the rest to the per-row kernel."""
        cfg, b = self.cfg, self.buf
        if window == -1 and (cfg.head_dim != 128 or self.nsplit_attn > 64 or cfg.gqa > 16):
            raise NotImplementedError("block rows need the multi-row attention kernel (head size 128)")
        if (m >= self.attn_rows_min or window == -1) and cfg.head_dim == 128 and self.nsplit_attn <= 64 and cfg.gqa <= 16:
            inkernel = m <= self.attn_merge_inkernel_rows    # few rows: the last split CTA merges; many: a merge launch
            # ``quant_out``: the caller's next launch is the o projection on pre-quantised rows; the merge writes them
            quant = quant_out and not inkernel and m >= self.prequant_rows and self.merge_quant
            K.attn_rows(b.q, kc, vc, block_table, ctrl, b.o_part, b.ml_part, b.attn_out, b.tickets if inkernel else None,
                        m, cfg.n_q_heads,
                        cfg.n_kv_heads, cfg.head_dim, self.nsplit_attn, max_blocks, self.scale,
                        span_pages=(max_blocks + self.nsplit_attn - 1) // self.nsplit_attn if self.attn_fixed_spans else 0,
                        k_scale=ks, v_scale=vs, kv_int8=kv.kv_int8, window=window, one_request=self.rows_one_request and m > 1,
                        xq=b.xq if quant else None, xq_gs=b.xq_gs if quant else None)
            return quant
        else:
            if window > 0:
                raise NotImplementedError("sliding-window layers need the multi-row attention kernel (head size 128)")
            K.attn_decode(b.q, kc, vc, block_table, ctrl, b.o_part, b.ml_part, b.attn_out, m, cfg.n_q_heads,
                          cfg.n_kv_heads, cfg.head_dim, self.nsplit_attn, max_blocks, self.scale, ks, vs, kv.kv_int8,
                          tickets=b.tickets)
        return False

    def gdn_block(self, lw: LayerWeights, li: int, m: int, ctrl, kv: KVCache):
        """A gated delta-net layer's mixer for the step's rows: projection GEMV, convolution + SiLU, the recurrent
        step per value head, output projection (partials, like the attention block's)."""
        cfg, b, g = self.cfg, self.buf, lw.gdn
        gi = cfg.gdn_index(li)
        part, s = self._gemv("gdn_in", g.in_proj, b.x, m)
        n = cfg.gdn_proj_dim
        K.gdn_conv(part, s, m, n, cfg.gdn_conv_channels, ctrl, g.conv_w, kv.gdn_conv[gi], b.gdn_act)
        K.gdn_step(b.gdn_act, m, n, cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim, ctrl, g.a_log, g.dt_bias,
                   g.norm_w, cfg.rms_eps, kv.gdn_state[gi], b.gdn_out)
        return self._gemv("gdn_out", g.out_proj, b.gdn_out, m)

    def _window(self, li: int) -> int:
        if li < self.cfg.n_layers:
            return self.cfg.window_of(li)
        return -1 if self.block_rows else 0    # draft-head layers: the whole context; -1: block rows as flagged

    def attention_block(self, lw: LayerWeights, li: int, m: int, ctrl, block_table, max_blocks, kv: KVCache):
        cfg, b = self.cfg, self.buf
        part, s = self._gemv("qkv", lw.qkv, b.x, m)
        kc, vc, ks, vs = kv.layer(li)
        K.rope_append(part, m * cfg.qkv_dim, s, m, ctrl, block_table, max_blocks, self.cos_t, self.sin_t,
                      cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, b.q, kc, vc, ks, vs, kv.kv_int8)
        self._attention(m, ctrl, block_table, max_blocks, kv, kc, vc, ks, vs, self._window(li))
        return self._gemv("o", lw.o, b.attn_out, m)

    def ffn_block(self, lw: LayerWeights, m: int):
        cfg, b = self.cfg, self.buf
        gu, s_gu = self._gemv("gate_up", lw.gate_up, b.x, m)
        return self._gemv("down", lw.down, gu, m, x_mode=1, s_in=s_gu, x_slice=m * 2 * cfg.ffn)

    def _gemv_fused(self, name: str, ql: QLinear, x, m: int, norm_w=None, fold: bool = False, x_mode=0, s_in=1,
                    x_slice=0, tp_fold: bool = True, prequantised: bool = False):
        """``tp_fold`` False: a linear every rank holds whole (a draft head's front) folds locally, without the
        ranks' all-reduce."""
        key = (ql.n, ql.k)
        s = self._splits.get(key)
        if s is None:
            s = self._splits[key] = K.gemv_splits(ql.n, ql.k)
        b = self.buf
        part = b.part(name, s, ql.n)
        if prequantised:        # ``buf.xq`` / ``buf.xq_gs`` already hold these rows (written by the attention merge)
            x, x_mode, norm_w, xq_gs = b.xq, 3, None, b.xq_gs
        elif m >= self.prequant_rows:
            K.quant_x(x, m, ql.k, b.xq, b.xq_gs, x_mode=x_mode, s_in=s_in, x_slice=x_slice, norm_w=norm_w,
                      norm_ssq=b.ssq if norm_w is not None else None, norm_eps=self.cfg.rms_eps)
            x, x_mode, norm_w, xq_gs = b.xq, 3, None, b.xq_gs
        else:
            xq_gs = None
        K.gemv_w4_fused(ql.w4b, x, part, m, ql.n, ql.k, s, x_mode=x_mode, s_in=s_in, x_slice=x_slice,
                        norm_w=norm_w, norm_ssq=xq_gs if xq_gs is not None else (b.ssq if norm_w is not None else None),
                        norm_eps=self.cfg.rms_eps,
                        fold_tickets=b.fold_tickets if fold else None, fold_resid=b.resid if fold else None,
                        fold_ssq=b.ssq if fold else None,
                        tp=self.tp.fold if (fold and tp_fold and self.tp is not None) else None,
                        tp_mcap=self.tp.mcap if self.tp is not None else 0)
        return part, s

    def _qkv_rope(self, lw: LayerWeights, m: int, ctrl, block_table, max_blocks, kc, vc, x_ready: bool):
        """qkv projection + RoPE + KV append in one launch (the GEMV's last split CTA per head does the rest)."""
        cfg, b = self.cfg, self.buf
        ql = lw.qkv
        key = (ql.n, ql.k)
        s = self._splits.get(key)
        if s is None:
            s = self._splits[key] = K.gemv_splits(ql.n, ql.k)
        part = b.part("qkv", s, ql.n)
        x, x_mode, norm_w, aux = (b.x, 0, None, None) if x_ready else (b.resid, 2, lw.input_norm, b.ssq)
        if m >= self.prequant_rows:
            K.quant_x(x, m, ql.k, b.xq, b.xq_gs, x_mode=x_mode, norm_w=norm_w, norm_ssq=aux, norm_eps=cfg.rms_eps)
            x, x_mode, norm_w, aux = b.xq, 3, None, b.xq_gs
        K.gemv_w4_qkv_rope(ql.w4b, x, part, m, ql.k, s, x_mode=x_mode, norm_w=norm_w, norm_ssq=aux, norm_eps=cfg.rms_eps,
                           tickets=b.qkv_tickets, q_out=b.q, cos_t=self.cos_t, sin_t=self.sin_t, ctrl=ctrl,
                           block_table=block_table, max_blocks=max_blocks, n_q=ql.n // 128 - 2 * cfg.n_kv_heads,
                           n_kv=cfg.n_kv_heads, k_plane=kc, v_plane=vc)

    def dense_layer_fused(self, lw: LayerWeights, li: int, m: int, ctrl, block_table, max_blocks, kv: KVCache,
                          x_ready: bool):
        """One dense layer in six launches: the residual folds ride in the o / down GEMVs' last CTAs and the
        two RMSNorms in the qkv / gate‖up GEMVs' activation staging.  ``x_ready``: ``buf.x`` already holds
        the normalised input (first layer, after the embedding kernel); otherwise ``buf.resid`` and
        ``buf.ssq`` do."""
        cfg, b = self.cfg, self.buf
        kc, vc, ks, vs = kv.layer(li)
        if self.rope_fold and not kv.kv_int8 and cfg.head_dim == 128 and lw.qkv.n == cfg.qkv_dim:
            self._qkv_rope(lw, m, ctrl, block_table, max_blocks, kc, vc, x_ready)
        else:
            if x_ready:
                part, s = self._gemv("qkv", lw.qkv, b.x, m)
            else:
                part, s = self._gemv_fused("qkv", lw.qkv, b.resid, m, norm_w=lw.input_norm, x_mode=2)
            K.rope_append(part, m * cfg.qkv_dim, s, m, ctrl, block_table, max_blocks, self.cos_t, self.sin_t,
                          cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, b.q, kc, vc, ks, vs, kv.kv_int8)
        q8 = self._attention(m, ctrl, block_table, max_blocks, kv, kc, vc, ks, vs, self._window(li),
                             quant_out=lw.o.k == cfg.n_q_heads * 128)
        self._gemv_fused("o", lw.o, b.attn_out, m, fold=True, prequantised=q8)
        gu, s_gu = self._gemv_fused("gate_up", lw.gate_up, b.resid, m, norm_w=lw.post_norm, x_mode=2)
        self._gemv_fused("down", lw.down, gu, m, fold=True, x_mode=1, s_in=s_gu, x_slice=m * 2 * cfg.ffn)

    def gdn_layer_fused(self, lw: LayerWeights, li: int, m: int, ctrl, kv: KVCache, x_ready: bool):
        """A gated delta-net layer with a dense FFN in six launches: projection GEMV (input RMSNorm in its staging),
        convolution + SiLU, recurrent step, output projection (residual fold in its last CTAs), gate||up (post norm in
        its staging), down (fold).  ``x_ready`` as in ``dense_layer_fused``."""
        cfg, b, g = self.cfg, self.buf, lw.gdn
        gi = cfg.gdn_index(li)
        if x_ready:
            part, s = self._gemv("gdn_in", g.in_proj, b.x, m)
        else:
            part, s = self._gemv_fused("gdn_in", g.in_proj, b.resid, m, norm_w=lw.input_norm, x_mode=2)
        n = cfg.gdn_proj_dim
        K.gdn_conv(part, s, m, n, cfg.gdn_conv_channels, ctrl, g.conv_w, kv.gdn_conv[gi], b.gdn_act)
        K.gdn_step(b.gdn_act, m, n, cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim, ctrl, g.a_log, g.dt_bias,
                   g.norm_w, cfg.rms_eps, kv.gdn_state[gi], b.gdn_out)
        self._gemv_fused("gdn_out", g.out_proj, b.gdn_out, m, fold=True)
        gu, s_gu = self._gemv_fused("gate_up", lw.gate_up, b.resid, m, norm_w=lw.post_norm, x_mode=2)
        self._gemv_fused("down", lw.down, gu, m, fold=True, x_mode=1, s_in=s_gu, x_slice=m * 2 * cfg.ffn)

    def moe_layer_fused(self, lw: LayerWeights, li: int, m: int, ctrl, block_table, max_blocks, kv: KVCache, x_ready: bool):
        """One mixture-of-experts layer in ten launches (eleven unfused): the input RMSNorm rides in the qkv GEMV's
        staging, the attention branch's residual fold in the o GEMV's last CTAs, and the experts' weighted sum is
        added to the residual rows by the combine kernel, which also leaves the sums of squares the next layer's
        qkv GEMV normalises with.  ``x_ready`` as in ``dense_layer_fused``."""
        from . import moe as _moe
        cfg, b = self.cfg, self.buf
        kc, vc, ks, vs = kv.layer(li)
        if self.rope_fold and not kv.kv_int8 and cfg.head_dim == 128 and lw.qkv.n == cfg.qkv_dim:
            self._qkv_rope(lw, m, ctrl, block_table, max_blocks, kc, vc, x_ready)
        else:
            if x_ready:
                part, s = self._gemv("qkv", lw.qkv, b.x, m)
            else:
                part, s = self._gemv_fused("qkv", lw.qkv, b.resid, m, norm_w=lw.input_norm, x_mode=2)
            K.rope_append(part, m * cfg.qkv_dim, s, m, ctrl, block_table, max_blocks, self.cos_t, self.sin_t,
                          cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, b.q, kc, vc, ks, vs, kv.kv_int8)
        q8 = self._attention(m, ctrl, block_table, max_blocks, kv, kc, vc, ks, vs, self._window(li),
                             quant_out=lw.o.k == cfg.n_q_heads * 128)
        self._gemv_fused("o", lw.o, b.attn_out, m, fold=True, prequantised=q8)
        # the experts and the router read normalised rows
        K.resid_norm(1, m, cfg.hidden, lw.post_norm, cfg.rms_eps, b.resid, b.x, resid_in=b.resid, splits=0)
        _moe.moe_block_rows(self, lw, m, fold=True)

    def _moe_fusable(self, layers: List[LayerWeights]) -> bool:
        cfg = self.cfg
        if not self.fused or self.tp is not None or self.nccl is not None or self.ep is not None or cfg.hidden % 128:
            return False
        return all(lw.experts_gate_up_w4b is not None and lw.gdn is None and lw.qkv is not None and
                   (lw.shared is None or (cfg.shared_ffn == cfg.expert_ffn and
                                          lw.shared.gate_up.w4b.numel() == lw.experts_gate_up_w4b[0].numel()))
                   for lw in layers)

    # ------------------------------------------------------------------ whole-step kernel
    def mega_plan(self, layers: List[LayerWeights], m: int, kv: KVCache):
        """The schedule of the whole-step kernel for ``m`` rows, or None when this step is outside what it covers:
        dense SwiGLU layers with full softmax attention, head size 128, bf16 KV, one GPU, at most 8 rows."""
        cfg = self.cfg
        if not (self.use_mega and self.fused and self.tp is None and self.nccl is None and m <= 8):
            return None
        if kv.kv_int8 or cfg.head_dim != 128 or cfg.hidden % 128 or cfg.ffn % 128 or cfg.ffn <= 0:
            return None
        if any(lw.gate_up is None or lw.gdn is not None or lw.qkv is None for lw in layers):
            return None
        if any(lw.qkv.n != cfg.qkv_dim or lw.gate_up.n != 2 * cfg.ffn for lw in layers):
            return None
        if cfg.sliding_window > 0:
            return None
        key = (m, cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads, cfg.ffn)
        if key not in self._mega_bufs:
            n_cta = K.decode_mega_sms()
            plan = K.decode_mega_plan(n_cta, m, cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads, cfg.ffn)
            if plan is not None:
                plan["n_cta"] = n_cta
                dev, u8, i32, f32 = self.device, torch.uint8, torch.int32, torch.float32
                ks = (cfg.hidden // 64, cfg.q_dim // 64, cfg.ffn // 64)     # groups of the three quantised-row buffers
                plan["xq"] = [torch.zeros(g * plan["rows"] * 144, dtype=u8, device=dev) for g in ks]
                plan["gs"] = [torch.zeros(g * 8 * 2, dtype=i32, device=dev) for g in ks]
                plan["part"] = torch.zeros(plan["part_floats"], dtype=f32, device=dev)
                plan["o_part"] = torch.zeros(m * cfg.n_q_heads * plan["nsplit"] * 128, dtype=f32, device=dev)
                plan["ml_part"] = torch.zeros(m * cfg.n_q_heads * plan["nsplit"] * 2, dtype=f32, device=dev)
                if self._mega_shared is None:
                    self._mega_shared = {"tickets": torch.zeros(max(plan["max_nb"], 8), dtype=i32, device=dev),
                                         "attn_tickets": torch.zeros(max(cfg.n_kv_heads, 8), dtype=i32, device=dev),
                                         "bar": torch.zeros(4, dtype=i32, device=dev)}
            self._mega_bufs[key] = plan
        return self._mega_bufs[key]

    def mega_reset(self):
        """Zeroes the kernel's ticket and barrier words (after a bounded wait ran out in the middle of a step)."""
        if self._mega_shared is not None:
            for t in self._mega_shared.values():
                t.zero_()

    def _mega_table(self, layers: List[LayerWeights], kv: KVCache, kv_layer0: int) -> torch.Tensor:
        key = (tuple(id(lw) for lw in layers), id(kv), kv_layer0)
        t = self._mega_tables.get(key)
        if t is None:
            rows = []
            for i, lw in enumerate(layers):
                rows.append([lw.qkv.w4b.data_ptr(), lw.o.w4b.data_ptr(), lw.gate_up.w4b.data_ptr(), lw.down.w4b.data_ptr(),
                             lw.input_norm.data_ptr(), lw.post_norm.data_ptr(), kv._plane[kv_layer0 + i], 0])
            t = torch.tensor(rows, dtype=torch.int64).to(self.device)
            self._mega_tables[key] = t
        return t

    def mega_layers(self, layers: List[LayerWeights], m: int, ctrl, block_table, max_blocks, kv: KVCache, plan,
                    kv_layer0: int = 0, n_phases: int = 0):
        """Embedding + ``layers`` for the step's rows in one launch; leaves the folded residual stream in
        ``buf.resid`` and its per-block sums of squares in ``buf.ssq``."""
        cfg, b, sh = self.cfg, self.buf, self._mega_shared
        span = (max_blocks + plan["nsplit"] - 1) // plan["nsplit"] if self.attn_fixed_spans else 0
        K.decode_mega(self._mega_table(layers, kv, kv_layer0), len(layers), m, cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads,
                      cfg.ffn, ctrl, block_table, max_blocks, kv.num_pages, kv.k.shape[0], self.w.embed, cfg.vocab, b.flag,
                      self.cos_t, self.sin_t, kv.k, kv.v, b.resid, b.ssq, plan["xq"], plan["gs"], plan["part"],
                      sh["tickets"], b.q, plan["o_part"], plan["ml_part"], sh["attn_tickets"], sh["bar"], cfg.rms_eps,
                      self.scale, span, plan["n_cta"], n_phases=n_phases, cooperative=self.mega_cooperative,
                      dbg=getattr(self, "mega_dbg", None))

    def layers_walk(self, layers: List[LayerWeights], m: int, ctrl, block_table, max_blocks, kv: KVCache,
                    first_from_embed: bool = True, kv_layer0: int = 0, resid_ready: bool = False,
                    one_request: bool = False):
        """Runs ``layers``; returns the (partials, splits) of the last residual branch, not yet folded.
        ``resid_ready``: ``buf.resid`` and ``buf.ssq`` already hold the folded residual rows and their per-block
        sums of squares (a later pipeline stage that received them from the stage before)."""
        cfg, b = self.cfg, self.buf
        h = cfg.hidden
        pend = None
        embedded = False
        self.rows_one_request = bool(one_request)     # the attention launch then counts row groups, not rows
        if self.fused and resid_ready and all(lw.gate_up is not None and lw.gdn is None for lw in layers) and h % 128 == 0:
            for i, lw in enumerate(layers):
                self.dense_layer_fused(lw, kv_layer0 + i, m, ctrl, block_table, max_blocks, kv, x_ready=False)
            return None, 0
        if one_request and first_from_embed:
            # rows of ONE request at consecutive positions: the whole walk is one persistent kernel
            plan = self.mega_plan(layers, m, kv)
            if plan is not None:
                self.mega_layers(layers, m, ctrl, block_table, max_blocks, kv, plan, kv_layer0)
                return None, 0
        if self.fused and first_from_embed and all(lw.gate_up is not None and lw.gdn is None for lw in layers) and h % 128 == 0:
            K.resid_norm(0, m, h, layers[0].input_norm, cfg.rms_eps, b.resid, b.x, embed=self.w.embed, ctrl=ctrl,
                         vocab=cfg.vocab, flag=b.flag)
            for i, lw in enumerate(layers):
                self.dense_layer_fused(lw, kv_layer0 + i, m, ctrl, block_table, max_blocks, kv, x_ready=(i == 0))
            return None, 0      # the residual stream is already folded
        if (self.fused and first_from_embed and self.tp is None and self.nccl is None and h % 128 == 0 and
                any(lw.gdn is not None for lw in layers) and all(lw.gate_up is not None for lw in layers) and
                cfg.gdn_value_dim % 64 == 0):
            # hybrid model: gated delta-net layers and attention layers, both on their fused forms
            K.resid_norm(0, m, h, layers[0].input_norm, cfg.rms_eps, b.resid, b.x, embed=self.w.embed, ctrl=ctrl,
                         vocab=cfg.vocab, flag=b.flag)
            for i, lw in enumerate(layers):
                if lw.gdn is not None:
                    self.gdn_layer_fused(lw, kv_layer0 + i, m, ctrl, kv, x_ready=(i == 0))
                else:
                    self.dense_layer_fused(lw, kv_layer0 + i, m, ctrl, block_table, max_blocks, kv, x_ready=(i == 0))
            return None, 0
        if first_from_embed and self._moe_fusable(layers):
            K.resid_norm(0, m, h, layers[0].input_norm, cfg.rms_eps, b.resid, b.x, embed=self.w.embed, ctrl=ctrl,
                         vocab=cfg.vocab, flag=b.flag)
            for i, lw in enumerate(layers):
                self.moe_layer_fused(lw, kv_layer0 + i, m, ctrl, block_table, max_blocks, kv, x_ready=(i == 0))
            return None, 0      # the residual stream is already folded
        if self.tp is not None:
            raise NotImplementedError("tensor parallel decode covers dense models whose hidden size is a multiple of 128")
        for i, lw in enumerate(layers):
            if pend is None:
                if first_from_embed and not embedded:
                    embedded = True
                    K.resid_norm(0, m, h, lw.input_norm, cfg.rms_eps, b.resid, b.x, embed=self.w.embed, ctrl=ctrl,
                                 vocab=cfg.vocab, flag=b.flag)
                else:   # resid already holds the layer input
                    K.resid_norm(1, m, h, lw.input_norm, cfg.rms_eps, b.resid, b.x, resid_in=b.resid, splits=0)
            else:
                K.resid_norm(1, m, h, lw.input_norm, cfg.rms_eps, b.resid, b.x, resid_in=b.resid, part=pend[0],
                             part_slice=m * h, splits=pend[1])
            if lw.gdn is not None:
                po, so = self.gdn_block(lw, kv_layer0 + i, m, ctrl, kv)
            else:
                po, so = self.attention_block(lw, kv_layer0 + i, m, ctrl, block_table, max_blocks, kv)
            po, so = self._nccl_reduce(po, so, m)
            K.resid_norm(1, m, h, lw.post_norm, cfg.rms_eps, b.resid, b.x, resid_in=b.resid, part=po,
                         part_slice=m * h, splits=so)
            if lw.gate_up is not None:
                pend = self.ffn_block(lw, m)
            elif self.ep is not None:
                # experts spread over the ranks: the block adds its result to the residual rows itself
                self.ep.block_rows(lw, m, b.x, b.resid)
                pend = None
                continue
            else:
                from . import moe as _moe
                pend = _moe.moe_block_rows(self, lw, m)
            pend = self._nccl_reduce(pend[0], pend[1], m)
        return pend if pend is not None else (None, 0)

    def _nccl_reduce(self, part, splits: int, m: int):
        """Comparison path: sum the split slices, all-reduce the ranks' partial sums with NCCL."""
        if self.nccl is None:
            return part, splits
        import torch.distributed as dist
        n = m * self.cfg.hidden
        red = self._red[:n]
        torch.sum(part[: splits * n].view(splits, n), dim=0, out=red)
        dist.all_reduce(red, group=self.nccl[2])
        return red, 1

    def head(self, m: int, pend, ctrl, advance: bool, final_norm: Optional[torch.Tensor] = None):
        cfg, b = self.cfg, self.buf
        h = cfg.hidden
        fn = self.w.final_norm if final_norm is None else final_norm
        K.resid_norm(1, m, h, fn, cfg.rms_eps, b.resid, b.x, resid_in=b.resid, part=pend[0],
                     part_slice=m * h, splits=pend[1])
        nv = self.head_rows
        if self.int8_head:
            w8, sc = self.w.lm_head_i8
            K.head_gemv(w8, b.x, b.logits, m, nv, h, b.cand_val, b.cand_idx, wscale=sc)
        else:
            K.head_gemv(self.w.lm_head, b.x, b.logits, m, nv, h, b.cand_val, b.cand_idx)
        if self.nccl is not None:
            self._head_nccl(m, ctrl, advance)
        elif self.tp is not None:   # vocabulary-parallel: exchange (value, id) and merge on the device
            K.argmax_finish_tp(b.cand_val, b.cand_idx, b.ncand, m, self.vocab_offset, ctrl, advance, self.tp.head,
                               self.tp.mcap)
        else:
            K.argmax_finish(b.cand_val, b.cand_idx, b.ncand, m, ctrl, advance)

    def _head_nccl(self, m: int, ctrl, advance: bool):
        """Comparison path of the vocabulary-parallel arg-max: local arg-max, NCCL all-gather, torch merge."""
        import torch.distributed as dist
        b = self.buf
        rank, world, group = self.nccl
        cv = b.cand_val[: m * b.ncand].view(m, b.ncand)
        ci = b.cand_idx[: m * b.ncand].view(m, b.ncand)
        best = cv.max(dim=1).values
        tie = torch.where(cv == best[:, None], ci, torch.full_like(ci, 0x7fffffff)).min(dim=1).values
        mine = torch.stack([best, (tie + self.vocab_offset_nccl).view(torch.float32)], dim=1).contiguous()
        dist.all_gather_into_tensor(self._gather_flat(m), mine, group=group)
        g = self._gather_flat(m).view(world, m, 2)
        vals, ids = g[:, :, 0], g[:, :, 1].contiguous().view(torch.int32)
        top = vals.max(dim=0).values
        tok = torch.where(vals == top[None, :], ids, torch.full_like(ids, 0x7fffffff)).min(dim=0).values
        ctrl[K.CTRL_OUT_TOKEN: K.CTRL_OUT_TOKEN + m] = tok
        ctrl[K.CTRL_OUT_VALUE: K.CTRL_OUT_VALUE + m] = top.view(torch.int32)
        if advance:
            ctrl[K.CTRL_CUR_TOKEN: K.CTRL_CUR_TOKEN + m] = tok
            ctrl[K.CTRL_ROW_POS: K.CTRL_ROW_POS + m] += 1

    def _gather_flat(self, m: int):
        return self._gather.view(-1)[: self.nccl[1] * m * 2]

    # ------------------------------------------------------------------ whole step
    def step_rows(self, m: int, ctrl, block_table, max_blocks, kv: KVCache, advance: bool, one_request: bool = False):
        """One forward pass for the ``m`` rows described by ``ctrl``; the arg-max of each row lands in
        ``ctrl[out_token]``; with ``advance`` the rows' tokens and positions move on for the next replay.
        ``one_request``: the rows are consecutive positions of one request (plain decode, verify rows)."""
        assert 1 <= m <= self.max_rows
        pend = self.layers_walk(self.w.layers, m, ctrl, block_table, max_blocks, kv, one_request=one_request)
        self.head(m, pend, ctrl, advance)
