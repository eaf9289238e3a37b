"""Weight containers shared by the CPU oracle and the GPU models.

A quantised linear is held in the kernel ("W4B") layout only; the oracle
dequantises it on demand.  ``random_weights`` builds a whole random-init model
either by quantising fp32 normal(0, 0.02) matrices (exact, used for the tiny
configurations and for writing synthetic checkpoints) or by drawing nibbles and
scales directly on the device (used for the full-size benchmark shapes).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..utils import quant as Q
from .config import ModelConfig


@dataclass
class QLinear:
    """W4A16 linear in W4B layout. ``w4b`` is uint8 ``[ceil(n/128)][k/64][4352]``."""
    w4b: torch.Tensor
    n: int
    k: int
    _w_f32: Optional[torch.Tensor] = None     # oracle cache
    _w_bf16: Optional[torch.Tensor] = None    # resident bf16 copy for the prefill GEMM
    _w_i8: Optional[tuple] = None             # (int8 [n][k], fp32 row scale) for the int8 prefill GEMM

    def dequant_f32(self) -> torch.Tensor:
        if self._w_f32 is None:
            self._w_f32 = Q.dequant_w4b(self.w4b.cpu(), self.n)
        return self._w_f32

    @property
    def nbytes(self) -> int:
        return self.w4b.numel()

    @staticmethod
    def from_f32(w: torch.Tensor, device="cpu") -> "QLinear":
        q, s = Q.quantize_rtn(w)
        return QLinear(Q.to_w4b(q, s).to(device), w.shape[0], w.shape[1])

    @staticmethod
    def random(n: int, k: int, device, seed: int, std: float = 0.02) -> "QLinear":
        return QLinear(Q.random_w4b(n, k, device, seed, std), n, k)


def interleave16(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Fuse gate and up rows in alternating runs of 16 (``g0..15, u0..15, g16..``).

    With this order a GEMM epilogue thread that owns 32 consecutive output
    columns holds 16 gate values and their 16 up values, so SiLU(g)*u is
    computed without a second pass (the reference fuses gate‖up the same way,
    src/loader/loader.cc:308).
    """
    i, k = gate.shape
    assert i % 16 == 0
    return torch.stack([gate.reshape(i // 16, 16, k), up.reshape(i // 16, 16, k)], dim=1).reshape(2 * i, k)


def deinterleave16(x: torch.Tensor):
    """Split the last dim of ``x`` (2*I, interleave16 order) into (gate, up)."""
    *lead, n = x.shape
    v = x.reshape(*lead, n // 32, 2, 16)
    return v[..., 0, :].reshape(*lead, n // 2), v[..., 1, :].reshape(*lead, n // 2)


@dataclass
class ExpertWeights:
    gate_up: QLinear      # [2*expert_ffn][hidden], interleave16
    down: QLinear         # [hidden][expert_ffn]


@dataclass
class GdnWeights:
    """A gated delta-net layer: fused input projection [ q | k | v | z | b | a ], depthwise 4-tap convolution over
    q, k, v, per-head decay parameters, the gated output norm and the output projection."""
    in_proj: QLinear               # [gdn_proj_dim][hidden]
    conv_w: torch.Tensor           # fp32 [conv_channels][4]; tap 3 multiplies the newest input
    a_log: torch.Tensor            # fp32 [n_v]
    dt_bias: torch.Tensor          # fp32 [n_v]
    norm_w: torch.Tensor           # fp32 [head_dim]
    out_proj: QLinear              # [hidden][value_dim]


@dataclass
class LayerWeights:
    input_norm: torch.Tensor       # fp32 [hidden]
    post_norm: torch.Tensor        # fp32 [hidden]
    qkv: Optional[QLinear]         # None on gated delta-net layers
    o: Optional[QLinear]
    gate_up: Optional[QLinear] = None
    down: Optional[QLinear] = None
    router: Optional[torch.Tensor] = None          # bf16 [n_experts][hidden]
    experts: Optional[List[ExpertWeights]] = None
    shared: Optional[ExpertWeights] = None
    shared_gate: Optional[torch.Tensor] = None     # bf16 [1][hidden]
    # experts stacked for the grouped kernels: uint8 [E][nb][kg][4352]
    experts_gate_up_w4b: Optional[torch.Tensor] = None
    experts_down_w4b: Optional[torch.Tensor] = None
    gdn: Optional[GdnWeights] = None               # set instead of qkv / o on gated delta-net layers


@dataclass
class MtpWeights:
    """Multi-token-prediction head: fc over [norm(embed) ‖ norm(hidden)] then decoder layers."""
    pre_norm_embed: torch.Tensor
    pre_norm_hidden: torch.Tensor
    fc: QLinear                    # [hidden][2*hidden]
    layers: List[LayerWeights]
    norm: torch.Tensor
    mask_token: Optional[int] = None    # a block drafter's "not drafted yet" token (default: the last vocabulary id)


@dataclass
class ModelWeights:
    cfg: ModelConfig
    embed: torch.Tensor            # bf16 [vocab][hidden]
    lm_head: torch.Tensor          # bf16 [vocab][hidden]
    final_norm: torch.Tensor       # fp32 [hidden]
    layers: List[LayerWeights]
    mtp: Optional[MtpWeights] = None
    lm_head_i8: Optional[tuple] = None    # (int8 [vocab][hidden], fp32 [vocab]) when the int8 head is on

    def nbytes(self) -> int:
        tot = self.embed.numel() * 2 + self.lm_head.numel() * 2
        for lw in self.layers + (self.mtp.layers if self.mtp else []):
            for ql in (lw.qkv, lw.o, lw.gate_up, lw.down):
                if ql is not None:
                    tot += ql.nbytes
            if lw.gdn is not None:
                tot += lw.gdn.in_proj.nbytes + lw.gdn.out_proj.nbytes
            if lw.experts_gate_up_w4b is not None:
                tot += lw.experts_gate_up_w4b.numel() + lw.experts_down_w4b.numel()
            if lw.shared is not None:
                tot += lw.shared.gate_up.nbytes + lw.shared.down.nbytes
        return tot


def _norm_weight(h, device, gen=None):
    return torch.ones(h, dtype=torch.float32, device=device)


def _rand_layer(cfg: ModelConfig, device, seed: int, exact: bool, std=0.02, gdn: bool = False) -> LayerWeights:
    h = cfg.hidden
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)

    def lin(n, k, sub):
        if exact:
            return QLinear.from_f32(torch.randn(n, k, generator=g) * std, device)
        return QLinear.random(n, k, device, seed * 131 + sub, std)

    def lin_gate_up(i, k, sub):
        if exact:
            gate = torch.randn(i, k, generator=g) * std
            up = torch.randn(i, k, generator=g) * std
            return QLinear.from_f32(interleave16(gate, up), device)
        return QLinear.random(2 * i, k, device, seed * 131 + sub, std)

    if gdn:
        nv = cfg.gdn_v_heads
        lw = LayerWeights(input_norm=_norm_weight(h, device), post_norm=_norm_weight(h, device), qkv=None, o=None)
        lw.gdn = GdnWeights(
            in_proj=lin(cfg.gdn_proj_dim, h, 1),
            conv_w=(torch.randn(cfg.gdn_conv_channels, 4, generator=g) * 0.5).to(device),
            a_log=torch.log(torch.rand(nv, generator=g) * 4.0 + 0.5).to(device),
            dt_bias=(torch.randn(nv, generator=g) * 0.5).to(device),
            norm_w=(1.0 + 0.1 * torch.randn(cfg.gdn_head_dim, generator=g)).to(device),
            out_proj=lin(h, cfg.gdn_value_dim, 2))
    else:
        lw = LayerWeights(
            input_norm=_norm_weight(h, device), post_norm=_norm_weight(h, device),
            qkv=lin(cfg.qkv_dim, h, 1), o=lin(h, cfg.q_dim, 2))
    if exact:
        # non-trivial norm weights so the norm kernels are actually exercised
        lw.input_norm = (1.0 + 0.1 * torch.randn(h, generator=g)).to(device)
        lw.post_norm = (1.0 + 0.1 * torch.randn(h, generator=g)).to(device)
    if cfg.is_moe:
        lw.router = (torch.randn(cfg.n_experts, h, generator=g) * (1.0 / h ** 0.5)).to(torch.bfloat16).to(device) \
            if exact else (torch.randn(cfg.n_experts, h, device=device) * (1.0 / h ** 0.5)).to(torch.bfloat16)
        if exact:
            lw.experts = [ExpertWeights(lin_gate_up(cfg.expert_ffn, h, 10 + 2 * e), lin(h, cfg.expert_ffn, 11 + 2 * e))
                          for e in range(cfg.n_experts)]
            lw.experts_gate_up_w4b = torch.stack([e.gate_up.w4b for e in lw.experts]).contiguous()
            lw.experts_down_w4b = torch.stack([e.down.w4b for e in lw.experts]).contiguous()
        else:
            e = cfg.n_experts
            gu = Q.random_w4b(e * 2 * cfg.expert_ffn, h, device, seed * 131 + 7, std)
            dn = Q.random_w4b(e * h, cfg.expert_ffn, device, seed * 131 + 8, std)
            lw.experts_gate_up_w4b = gu.reshape(e, 2 * cfg.expert_ffn // 128, h // 64, Q.BLOCK_BYTES)
            lw.experts_down_w4b = dn.reshape(e, h // 128, cfg.expert_ffn // 64, Q.BLOCK_BYTES)
        if cfg.shared_ffn:
            lw.shared = ExpertWeights(lin_gate_up(cfg.shared_ffn, h, 3), lin(h, cfg.shared_ffn, 4))
            lw.shared_gate = (torch.randn(1, h, generator=g) * (1.0 / h ** 0.5)).to(torch.bfloat16).to(device)
    else:
        lw.gate_up = lin_gate_up(cfg.ffn, h, 5)
        lw.down = lin(h, cfg.ffn, 6)
    return lw


def random_weights(cfg: ModelConfig, device="cpu", seed: int = 0, exact: Optional[bool] = None,
                   std: float = 0.02, head_rows: Optional[int] = None) -> ModelWeights:
    """Random-init model. ``exact`` (default: on for < 100M parameters) quantises real fp32 matrices.
    ``head_rows``: rows of the lm_head this rank holds (vocabulary-parallel head)."""
    if exact is None:
        exact = cfg.param_count() < 100_000_000
    h = cfg.hidden
    hr = cfg.vocab if head_rows is None else head_rows
    if exact:
        g = torch.Generator(device="cpu")
        g.manual_seed(seed)
        embed = (torch.randn(cfg.vocab, h, generator=g) * std).to(torch.bfloat16).to(device)
        head = (torch.randn(cfg.vocab, h, generator=g) * std)[:hr].to(torch.bfloat16).to(device).contiguous()
    else:
        embed = torch.empty(cfg.vocab, h, dtype=torch.bfloat16, device=device).normal_(0, std)
        head = torch.empty(hr, h, dtype=torch.bfloat16, device=device).normal_(0, std)
    layers = [_rand_layer(cfg, device, seed * 1000 + 1 + i, exact, std, gdn=cfg.is_gdn_layer(i)) for i in range(cfg.n_layers)]
    mw = ModelWeights(cfg, embed, head, _norm_weight(h, device), layers)
    if cfg.mtp_layers:
        dense_cfg = cfg
        if exact:
            g2 = torch.Generator(device="cpu")
            g2.manual_seed(seed * 1000 + 777)
            fc = QLinear.from_f32(torch.randn(h, 2 * h, generator=g2) * std, device)
        else:
            fc = QLinear.random(h, 2 * h, device, seed * 1000 + 777, std)
        mw.mtp = MtpWeights(_norm_weight(h, device), _norm_weight(h, device), fc,
                            [_rand_layer(dense_cfg, device, seed * 1000 + 800 + i, exact, std)
                             for i in range(cfg.mtp_layers)], _norm_weight(h, device))
    return mw
