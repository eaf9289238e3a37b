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
    if lw.gdn is not None:
        raise NotImplementedError("gated delta-net layers are not sliced for tensor parallelism")
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
    out = ModelWeights(local, full.embed.to(device), head, full.final_norm.to(device), layers)
    if full.mtp is not None:      # the draft head: its layers are sliced like the trunk's, its front is held whole
        from ..models.weights import MtpWeights
        t = full.mtp
        out.mtp = MtpWeights(t.pre_norm_embed.to(device), t.pre_norm_hidden.to(device),
                             QLinear(t.fc.w4b.to(device), t.fc.n, t.fc.k),
                             [shard_layer(lw, cfg, rank, world, device) for lw in t.layers], t.norm.to(device))
    return out


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


# ---------------------------------------------------------------------- timing (CUDA events, max over ranks)
def _max_over_ranks(x: float, dev) -> float:
    import torch.distributed as dist
    t = torch.tensor([x], device=dev, dtype=torch.float64)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def _sync_all():
    import torch.distributed as dist
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    torch.cuda.synchronize()


def bench_decode(cfg: ModelConfig, mode: str, depth: int, steps: int, warmup: int, rows: int = 1, windows: int = 1,
                 e2e: bool = False, kv_dtype: str = "bf16") -> dict:
    """Graph-replayed decode steps of ``rows`` requests at context ``depth``; ms per step is the max over ranks of
    the median of ``windows`` timed windows of ``steps`` steps.  ``e2e``: also time steps driven from the host through
    ``Engine.forward_rows`` -- every step copies the rows' control words from pinned host memory and reads the
    tokens back."""
    import torch.distributed as dist
    from ..ops import lib as K
    from ..runtime.engine import Row
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    w = random_weights(cfg, device=dev, seed=0, exact=False) if world == 1 else random_shard(cfg, rank, world, dev)
    total = depth + (windows + (3 if e2e else 0) + 2) * (steps + warmup) + 64
    eng = make_engine(w, mode=mode, max_seqs=rows, max_len=total, kv_dtype=kv_dtype)
    local = eng.cfg
    for layer in range(local.n_layers):   # context at depth: random KV pages (the timing needs the reads only)
        kc, vc, ks, vs = eng.kv.layer(layer)
        if eng.kv.kv_int8:
            kc.copy_(torch.randint(-127, 128, kc.shape, device=dev, dtype=torch.int8))
            vc.copy_(torch.randint(-127, 128, vc.shape, device=dev, dtype=torch.int8))
            ks.fill_(0.5 / 127)
            vs.fill_(0.5 / 127)
        else:
            kc.normal_(0, 0.5)
            vc.normal_(0, 0.5)
    for s in range(rows):
        eng._ensure_pages(s, depth)
        eng.seq_len[s] = depth
    eng.decode_begin(list(range(rows)), [1 + s for s in range(rows)])
    for _ in range(warmup):
        eng.decode_step(read=False)
    win = []
    for _ in range(max(1, windows)):
        _sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            eng.decode_step(read=False)
        e1.record()
        _sync_all()
        win.append(e0.elapsed_time(e1) / steps)
    ms = _max_over_ranks(sorted(win)[len(win) // 2], dev)
    out = {"ms_per_step": ms, "tokens_per_s": rows / (ms / 1e3), "rows": rows, "depth": depth,
           "launches_per_step": eng.launches(rows, True), "kv_cache": kv_dtype, "windows_ms_per_step": [round(x, 4) for x in win]}
    if e2e:
        toks = eng._read_out(rows)
        for _ in range(warmup):
            toks = eng.forward_rows([Row(s, eng.seq_len[s], toks[s]) for s in range(rows)], advance=False, read=True)
        win = []
        for _ in range(min(3, max(1, windows))):
            _sync_all()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                toks = eng.forward_rows([Row(s, eng.seq_len[s], toks[s]) for s in range(rows)], advance=False, read=True)
            e1.record()
            _sync_all()
            win.append(e0.elapsed_time(e1) / steps)
        out["e2e_ms_per_step"] = _max_over_ranks(sorted(win)[len(win) // 2], dev)
        out["h2d_bytes_per_step"] = K.CTRL_WORDS * 4
        out["d2h_bytes_per_step"] = K.CTRL_WORDS * 4
    K.check_status()
    eng.close()
    del eng, w
    torch.cuda.empty_cache()
    return out


def bench_spec_mtp(cfg: ModelConfig, depth: int, iters: int = 12, k: int = 3, accept: int = 3) -> dict:
    """Draft-and-verify iterations with an MTP head under tensor parallelism (fused wires), FORCED acceptance so the
    time does not depend on what a random-init head proposes: prompt pass of ``depth`` tokens (the head ingests it from
    the gathered hidden rows), then ``iters`` iterations of k chained drafts + one verify step of k + 1 rows on every
    rank in lockstep.  Device time, max over ranks; tokens/s = (accept + 1) / iteration."""
    import torch.distributed as dist
    from ..ops import lib as K
    from ..runtime.spec import SpecAdapter
    from ..server.adapter import EngineAdapter
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    w = random_shard(dataclasses.replace(cfg, mtp_layers=1), rank, world, dev)
    eng = make_engine(w, mode="fused", max_seqs=1, max_len=depth + (k + 1) * (iters + 8) + 64, extra_kv_layers=1)
    ad = SpecAdapter(EngineAdapter(eng), "mtp", k)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab - 1, (depth,), generator=g).tolist()
    pending = ad.prefill(0, ids)

    def iteration(pending):
        drafts = ad.draft(0, pending, k)
        res = ad.step({0: [pending] + drafts})[0]
        keep = min(accept, len(drafts))
        if keep < len(drafts):
            ad.truncate(0, ad.length(0) - (len(drafts) - keep))
        return res[keep]

    for _ in range(3):
        pending = iteration(pending)
    _sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        pending = iteration(pending)
    e1.record()
    _sync_all()
    ms = _max_over_ranks(e0.elapsed_time(e1) / iters, dev)
    K.check_status()
    if hasattr(eng, "close"):
        eng.close()
    return {"world": world, "depth": depth, "k": k, "accepted": accept, "ms_per_iteration": ms,
            "tokens_per_s": (accept + 1) / ms * 1e3, "rows_verified": k + 1}


def bench_prefill(cfg: ModelConfig, mode: str, n: int, reps: int = 4, kv_dtype: str = "bf16") -> dict:
    """Whole prompt passes of ``n`` tokens through ``Engine.prefill``; ms is the max over ranks."""
    import torch.distributed as dist
    from ..ops import lib as K
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    w = random_weights(cfg, device=dev, seed=0, exact=False) if world == 1 else random_shard(cfg, rank, world, dev)
    eng = make_engine(w, mode=mode, max_seqs=1, max_len=n + 64, use_graphs=False, prefill_backend="bf16-resident",
                      kv_dtype=kv_dtype)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab, (n,), generator=g).tolist()
    for _ in range(3):
        eng.reset(0)
        eng.prefill(0, ids)
    _sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n0 = K.launch_count
    e0.record()
    for _ in range(reps):
        eng.reset(0)
        eng.prefill(0, ids)
    e1.record()
    _sync_all()
    ms = _max_over_ranks(e0.elapsed_time(e1) / reps, dev)
    K.check_status()
    launches = (K.launch_count - n0) // reps
    eng.close()
    del eng, w
    torch.cuda.empty_cache()
    return {"ms": ms, "tokens": n, "tokens_per_s": n / (ms / 1e3), "launches": launches, "kv_cache": kv_dtype}


def bench_fused_ops(cfg: ModelConfig, c: int = 4096, reps: int = 20, peaks: Optional[dict] = None) -> dict:
    """The two fused GEMM+collective kernels alone, at the model's down / gate‖up shapes over a ``c``-row chunk:
    time (max over ranks) against the slower of the GEMM at the measured cuBLAS peak and the bytes that must
    cross NVLink at the measured 770 GB/s per direction."""
    import torch.distributed as dist
    from ..ops import gemm as G
    from ..ops import lib as K
    from .symm import Wire
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    peaks = peaks or {}
    tf = float(peaks.get("bf16_tflops", 1590.0)) * 1e12
    link = 770e9
    h, f = cfg.hidden, cfg.ffn // world
    tiles = (c + 127) // 128
    tpr = (tiles + world - 1) // world
    rows_cap = tpr * 128
    rs = Wire(world * rows_cap * h * 2, world * tpr, 0, None, dev)
    xw = Wire(world * rows_cap * h * 2, world * tpr, 0, None, dev)
    x_full = xw.buf.view(torch.bfloat16, 0, world * rows_cap * h).view(world * rows_cap, h)
    own = torch.zeros(rows_cap, h, dtype=torch.bfloat16, device=dev)
    done = torch.zeros(tpr, dtype=torch.int32, device=dev)
    act = torch.randn(c, f, device=dev).to(torch.bfloat16)
    w_down = (torch.randn(h, f, device=dev) * 0.02).to(torch.bfloat16)
    w_gu = (torch.randn(2 * f, h, device=dev) * 0.02).to(torch.bfloat16)
    out_gu = torch.empty(c, f, dtype=torch.bfloat16, device=dev)
    norm_w = torch.ones(h, device=dev)
    state = {"ag": 0}

    def rs_step():
        arr = G.gemm_tp(act, w_down, None, G.EPI_RS_PUSH, rs=rs, rs_tpr=tpr)
        K.rs_fold(rs, arr, world, done, own, norm_w, 1e-6, xw, h, tpr, c)
        state["ag"] += 1

    def ag_step():
        G.gemm_tp(x_full[:c], w_gu, out_gu, G.EPI_SILU_MUL, ag_cnt=xw.flags, ag_expect=128 * state["ag"])

    def timed(fn):
        for _ in range(3):
            fn()
        _sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        _sync_all()
        return _max_over_ranks(e0.elapsed_time(e1) / reps, dev)

    def both():
        rs_step()
        ag_step()

    t_pair = timed(both)
    K.check_status()
    flops_rs = 2.0 * c * h * f
    flops_ag = 2.0 * c * (2 * f) * h
    bytes_rs = c * h * 2.0 * (world - 1) / world       # bf16 partial tiles leaving this rank
    bytes_ag = c * h * 2.0 * (world - 1) / world       # this rank's normalised rows to every peer
    floor_ms = (max(flops_rs / tf, bytes_rs / link) + max(flops_ag / tf, bytes_ag / link)) * 1e3
    rs.close()
    xw.close()
    return {"chunk_rows": c, "hidden": h, "ffn_local": f, "world": world,
            "gemm_rs_fold_ag_gemm_ms": t_pair, "roofline_floor_ms": floor_ms, "fraction_of_roofline": floor_ms / t_pair,
            "roofline": "slower of FLOPs at measured cuBLAS bf16 peak and NVLink bytes at measured 770 GB/s per direction",
            "peak_tflops_used": tf / 1e12}
