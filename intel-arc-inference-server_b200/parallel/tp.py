"""Tensor parallelism: one process per GPU, every rank drives the same Engine calls over its shard.

Column-parallel qkv / gate‖up (whole heads, whole interleave runs), row-parallel o / down whose
partial sums are all-reduced INSIDE the GEMV's fold epilogue over NVLink peer stores, and a
vocabulary-parallel lm_head whose arg-max is merged on the device.  The reference's two-card form:
src/runtime/tp_engine.h:98-292, src/kernels/tp.cl:98-202, src/model/model_desc.cc:252-285.  Here the
group is 2, 4 or 8 ranks behind an NVSwitch, so the crossing is a one-shot push to every peer plus a
local fold in rank order (latency-bound messages of 20 KB per row).

``mode="fused"`` is the product; ``mode="nccl"`` runs the same kernels unfused with NCCL
all-reduces, the comparison every speed-up is quoted against.
"""
from __future__ import annotations

import dataclasses
import os
from typing import Optional, Tuple

import torch

from ..models.config import ModelConfig
from ..models.weights import ExpertWeights, LayerWeights, ModelWeights, MtpWeights, QLinear, random_weights
from ..utils import quant as Q


def init_dist(backend: Optional[str] = None) -> Tuple[int, int, int]:
    """Joins the process group described by the launcher's environment; returns (rank, world, local_rank)."""
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {"device_id": torch.device("cuda", local)} if backend == "nccl" else {}
        dist.init_process_group(backend, rank=rank, world_size=world, **kw)
    return rank, world, local


# ---------------------------------------------------------------------- sharding existing weights
def _cols(ql: QLinear, lo: int, hi: int, device) -> QLinear:
    """Output rows lo:hi of a W4B linear (a column-parallel slice)."""
    q, s = Q.from_w4b(ql.w4b, ql.n)
    return QLinear(Q.to_w4b(q[:, lo:hi].contiguous().to(device), s[:, lo:hi].contiguous().to(device)), hi - lo, ql.k)


def _rows(ql: QLinear, lo: int, hi: int, device) -> QLinear:
    """Input channels lo:hi (a row-parallel slice); lo and hi are multiples of the group size."""
    q, s = Q.from_w4b(ql.w4b, ql.n)
    return QLinear(Q.to_w4b(q[lo:hi].contiguous().to(device), s[lo // 64: hi // 64].contiguous().to(device)), ql.n, hi - lo)


def _cat_cols(parts, device) -> QLinear:
    qs, ss = zip(*[Q.from_w4b(p.w4b, p.n) for p in parts])
    q, s = torch.cat(qs, dim=1), torch.cat(ss, dim=1)
    return QLinear(Q.to_w4b(q.to(device), s.to(device)), q.shape[1], q.shape[0])


def shard_layer(lw: LayerWeights, cfg: ModelConfig, rank: int, world: int, device) -> LayerWeights:
    hd = cfg.head_dim
    qh, kh = cfg.n_q_heads // world, cfg.n_kv_heads // world
    q0, k0, v0 = 0, cfg.q_dim, cfg.q_dim + cfg.kv_dim
    qkv = _cat_cols([_cols(lw.qkv, q0 + rank * qh * hd, q0 + (rank + 1) * qh * hd, device),
                     _cols(lw.qkv, k0 + rank * kh * hd, k0 + (rank + 1) * kh * hd, device),
                     _cols(lw.qkv, v0 + rank * kh * hd, v0 + (rank + 1) * kh * hd, device)], device)
    o = _rows(lw.o, rank * qh * hd, (rank + 1) * qh * hd, device)
    out = LayerWeights(input_norm=lw.input_norm.to(device), post_norm=lw.post_norm.to(device), qkv=qkv, o=o)
    if lw.gate_up is not None:
        f = cfg.ffn // world
        # gate‖up rows alternate in runs of 16: FFN channels lo:hi are rows 2 lo : 2 hi
        out.gate_up = _cols(lw.gate_up, 2 * rank * f, 2 * (rank + 1) * f, device)
        out.down = _rows(lw.down, rank * f, (rank + 1) * f, device)
    else:
        raise NotImplementedError("tensor-parallel sharding of MoE layers")
    return out


def shard_weights(full: ModelWeights, rank: int, world: int, device=None) -> ModelWeights:
    """This rank's shard of a whole model (tests and small models; big checkpoints are sliced by the loader)."""
    cfg = full.cfg
    device = device or full.embed.device
    local = cfg.tp_shard(world)
    per = (cfg.vocab + world - 1) // world
    head = full.lm_head[rank * per: min(cfg.vocab, (rank + 1) * per)].to(device).contiguous()
    layers = [shard_layer(lw, cfg, rank, world, device) for lw in full.layers]
    return ModelWeights(local, full.embed.to(device), head, full.final_norm.to(device), layers)


def random_shard(cfg: ModelConfig, rank: int, world: int, device, seed: int = 0) -> ModelWeights:
    """Random-init shard made directly on the device (full-size shapes; no whole model anywhere)."""
    local = cfg.tp_shard(world)
    per = (cfg.vocab + world - 1) // world
    rows = min(cfg.vocab, (rank + 1) * per) - rank * per
    return random_weights(local, device=device, seed=seed * 16 + rank, exact=False, head_rows=rows)


def make_engine(weights: ModelWeights, mode: str = "fused", group=None, **kw):
    """Engine over this rank's shard.  ``mode``: "fused" (peer-memory wires) or "nccl" (comparison)."""
    import torch.distributed as dist
    from ..runtime.engine import Engine
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if world == 1:
        return Engine(weights, **kw)
    if mode == "fused":
        from .symm import TpWires
        wires = TpWires(weights.cfg.hidden, kw.get("max_rows", 64), group, weights.embed.device)
        return Engine(weights, tp=wires, **kw)
    if mode == "nccl":
        return Engine(weights, nccl=(rank, world, group), **kw)
    raise ValueError(f"unknown tensor-parallel mode {mode!r}")
