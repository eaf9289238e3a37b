"""fp32 CPU oracle: the model math restated with plain PyTorch ops.

Every GPU kernel and the whole engine are judged against this file.  It plays
the role of the reference's Python oracle (tools/oracle/) and of its host
twins (tests/kernels/*_ref.h): dequantised fp32 matmuls, RMSNorm, rotate-half
RoPE, causal GQA softmax attention, SwiGLU, MoE routing (softmax over all
experts -> top-k with ties to the lower id -> renormalise, as in
src/kernels/moe.cl:20-36), greedy argmax with ties to the lower id
(src/kernels/argmax.cl).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn.functional as F

from .config import ModelConfig
from .weights import ModelWeights, LayerWeights, QLinear, deinterleave16


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float().cpu()


def rope_tables(head_dim: int, theta: float, max_pos: int):
    """cos / sin ``[max_pos][head_dim/2]`` computed in float64 then rounded to fp32
    (the reference builds its table the same way, src/loader/loader.cc:703)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float(), ang.sin().float()


def apply_rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half RoPE. ``x`` is ``[T][heads][head_dim]``, ``pos`` int ``[T]``."""
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
    ang = pos.double()[:, None] * inv[None, :]
    cos, sin = ang.cos().float()[:, None, :], ang.sin().float()[:, None, :]
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def argmax_low_tie(logits: torch.Tensor) -> torch.Tensor:
    """Argmax along the last dim; equal maxima resolve to the lowest index."""
    m = logits.max(dim=-1, keepdim=True).values
    idx = torch.arange(logits.shape[-1]).expand_as(logits)
    big = torch.full_like(idx, logits.shape[-1])
    return torch.where(logits == m, idx, big).min(dim=-1).values


def moe_route(logits: torch.Tensor, top_k: int):
    """softmax over all experts -> top-k (ties to lower id) -> renormalise to sum 1."""
    p = F.softmax(logits.float(), dim=-1)
    # stable sort on (-p, id): sort by id first (already ordered), then a stable sort by -p
    order = torch.sort(-p, dim=-1, stable=True).indices
    idx = order[..., :top_k]
    w = torch.gather(p, -1, idx)
    w = w / w.sum(-1, keepdim=True)
    return idx, w


class OracleKV:
    def __init__(self, cfg: ModelConfig, n_layers: Optional[int] = None):
        n = cfg.n_layers if n_layers is None else n_layers
        self.k: List[Optional[torch.Tensor]] = [None] * n
        self.v: List[Optional[torch.Tensor]] = [None] * n
        self.gdn = {}      # layer -> (conv inputs [channels][3], state [n_v][dk][dv]) of gated delta-net layers

    def length(self) -> int:
        for k in self.k:
            if k is not None:
                return k.shape[0]
        return 0

    def truncate(self, n: int):
        for i in range(len(self.k)):
            if self.k[i] is not None:
                self.k[i] = self.k[i][:n]
                self.v[i] = self.v[i][:n]


class OracleModel:
    def __init__(self, weights: ModelWeights):
        self.w = weights
        self.cfg = weights.cfg

    # ---- pieces ----
    def linear(self, ql: QLinear, x: torch.Tensor) -> torch.Tensor:
        return x.float() @ ql.dequant_f32().t()

    def swiglu(self, gate_up: QLinear, down: QLinear, x: torch.Tensor) -> torch.Tensor:
        g, u = deinterleave16(self.linear(gate_up, x))
        return self.linear(down, F.silu(g) * u)

    def attention(self, lw: LayerWeights, x: torch.Tensor, pos: torch.Tensor, kv: OracleKV, li: int):
        c = self.cfg
        t = x.shape[0]
        qkv = self.linear(lw.qkv, x)
        q = qkv[:, : c.q_dim].reshape(t, c.n_q_heads, c.head_dim)
        k = qkv[:, c.q_dim: c.q_dim + c.kv_dim].reshape(t, c.n_kv_heads, c.head_dim)
        v = qkv[:, c.q_dim + c.kv_dim:].reshape(t, c.n_kv_heads, c.head_dim)
        q = apply_rope(q, pos, c.rope_theta)
        k = apply_rope(k, pos, c.rope_theta)
        if kv.k[li] is None:
            kv.k[li], kv.v[li] = k, v
        else:
            kv.k[li] = torch.cat([kv.k[li], k]); kv.v[li] = torch.cat([kv.v[li], v])
        kk, vv = kv.k[li], kv.v[li]
        s_len = kk.shape[0]
        kk = kk.repeat_interleave(c.gqa, dim=1)
        vv = vv.repeat_interleave(c.gqa, dim=1)
        scores = torch.einsum("thd,shd->hts", q, kk) / math.sqrt(c.head_dim)
        key_pos = torch.arange(s_len)
        mask = key_pos[None, :] > pos[:, None]
        win = c.window_of(li) if li < c.n_layers else 0      # draft-head layers attend to the whole context
        if win > 0:
            mask = mask | (key_pos[None, :] <= pos[:, None] - win)
        scores = scores.masked_fill(mask[None], float("-inf"))
        p = F.softmax(scores, dim=-1)
        o = torch.einsum("hts,shd->thd", p, vv).reshape(t, c.q_dim)
        return self.linear(lw.o, o)

    def moe(self, lw: LayerWeights, x: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        logits = x.float() @ lw.router.float().cpu().t()
        idx, wts = moe_route(logits, c.top_k)
        out = torch.zeros_like(x, dtype=torch.float32)
        for e in range(c.n_experts):
            sel = (idx == e)
            rows = sel.any(-1).nonzero().flatten()
            if rows.numel() == 0:
                continue
            we = (wts * sel).sum(-1)[rows]
            ex = lw.experts[e]
            out[rows] += we[:, None] * self.swiglu(ex.gate_up, ex.down, x[rows])
        if lw.shared is not None:
            gate = torch.sigmoid(x.float() @ lw.shared_gate.float().cpu().t())
            out += gate * self.swiglu(lw.shared.gate_up, lw.shared.down, x)
        return out

    def gdn(self, lw: LayerWeights, x: torch.Tensor, kv: OracleKV, li: int) -> torch.Tensor:
        """Gated delta-net layer, token by token (the recurrence the device kernel runs: ops/csrc/gdn.cu)."""
        c, g = self.cfg, lw.gdn
        dh, nk, nv = c.gdn_head_dim, c.gdn_k_heads, c.gdn_v_heads
        kd, vd, cc = c.gdn_key_dim, c.gdn_value_dim, c.gdn_conv_channels
        proj = self.linear(g.in_proj, x)
        conv_w, a_log, dt_bias, norm_w = (t.float().cpu() for t in (g.conv_w, g.a_log, g.dt_bias, g.norm_w))
        conv, S = kv.gdn.get(li, (torch.zeros(cc, 3), torch.zeros(nv, dh, dh)))
        outs = []
        for t in range(x.shape[0]):
            hist = torch.cat([conv, proj[t, :cc, None]], dim=1)
            y = F.silu((hist * conv_w).sum(dim=1))
            conv = hist[:, 1:]
            q, k, v = y[:kd].view(nk, dh), y[kd: 2 * kd].view(nk, dh), y[2 * kd:].view(nv, dh)
            z = proj[t, cc: cc + vd].view(nv, dh)
            b, a = proj[t, cc + vd: cc + vd + nv], proj[t, cc + vd + nv:]
            q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dh ** -0.5
            k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
            q, k = q.repeat_interleave(nv // nk, dim=0), k.repeat_interleave(nv // nk, dim=0)
            beta = torch.sigmoid(b)
            decay = torch.exp(-torch.exp(a_log) * F.softplus(a + dt_bias))
            S = S * decay[:, None, None]
            delta = (v - torch.einsum("hij,hi->hj", S, k)) * beta[:, None]
            S = S + torch.einsum("hi,hj->hij", k, delta)
            o = torch.einsum("hij,hi->hj", S, q)
            o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + c.rms_eps) * norm_w * F.silu(z)
            outs.append(o.reshape(vd))
        kv.gdn[li] = (conv, S)
        return self.linear(g.out_proj, torch.stack(outs))

    def layer(self, lw: LayerWeights, h: torch.Tensor, pos: torch.Tensor, kv: OracleKV, li: int):
        c = self.cfg
        xin = rmsnorm(h, lw.input_norm, c.rms_eps)
        h = h + (self.gdn(lw, xin, kv, li) if lw.gdn is not None else self.attention(lw, xin, pos, kv, li))
        x = rmsnorm(h, lw.post_norm, c.rms_eps)
        if lw.experts is not None:
            h = h + self.moe(lw, x)
        else:
            h = h + self.swiglu(lw.gate_up, lw.down, x)
        return h

    # ---- whole model ----
    def forward(self, ids: torch.Tensor, kv: Optional[OracleKV] = None, start: int = 0, return_hidden=False):
        """Run ``ids`` (int ``[T]``) at positions ``start..``; returns logits ``[T][vocab]`` fp32."""
        c = self.cfg
        if kv is None:
            kv = OracleKV(c)
        pos = torch.arange(start, start + ids.shape[0])
        h = self.w.embed.float().cpu()[ids]
        for li, lw in enumerate(self.w.layers):
            h = self.layer(lw, h, pos, kv, li)
        hn = rmsnorm(h, self.w.final_norm, c.rms_eps)
        logits = hn @ self.w.lm_head.float().cpu().t()
        if return_hidden:
            return logits, h
        return logits

    def mtp_forward(self, hidden: torch.Tensor, next_ids: torch.Tensor, kv: OracleKV, start: int):
        """MTP head: ``hidden`` ``[T][H]`` is the trunk's pre-final-norm state at positions
        ``start..``; ``next_ids`` are the tokens at positions ``start+1..``.  Returns logits that
        predict positions ``start+2..`` and the head's own hidden state (to chain deeper drafts)."""
        c, m = self.cfg, self.w.mtp
        e = rmsnorm(self.w.embed.float().cpu()[next_ids], m.pre_norm_embed, c.rms_eps)
        hh = rmsnorm(hidden, m.pre_norm_hidden, c.rms_eps)
        h = self.linear(m.fc, torch.cat([e, hh], dim=-1))
        pos = torch.arange(start, start + next_ids.shape[0])
        for li, lw in enumerate(m.layers):
            h = self.layer(lw, h, pos, kv, li)
        logits = rmsnorm(h, m.norm, c.rms_eps) @ self.w.lm_head.float().cpu().t()
        return logits, h

    def generate(self, prompt: torch.Tensor, n_new: int):
        """Greedy decode. Returns (token ids ``[n_new]``, logits ``[n_new][vocab]``)."""
        kv = OracleKV(self.cfg)
        logits = self.forward(prompt, kv, 0)[-1:]
        toks, rows = [], []
        pos = prompt.shape[0]
        for _ in range(n_new):
            t = argmax_low_tie(logits)
            toks.append(int(t)); rows.append(logits[0])
            logits = self.forward(t.reshape(1), kv, pos)
            pos += 1
        return torch.tensor(toks), torch.stack(rows)
