"""Expert parallelism for the mixture-of-experts prompt pass.

Attention, router and shared expert are replicated and run data-parallel (every rank serves its own
requests); the routed experts are spread over the ranks, ``E / world`` each.  A block's tokens go to
their experts' ranks and come back through the fused kernels of ``ops/csrc/ep.cu`` and the
expert-parallel forms of the grouped GEMM (``ops/csrc/gemm_tc.cu``):

    route -> count -> counts exchange -> plan -> dispatch (peer stores, per-block arrival counters)
          -> grouped gate‖up GEMM (starts a block when its rows are in) -> grouped down GEMM whose
             epilogue stores each row into its source rank's return buffer
          -> weighted sum of a token's slots in slot order (+ shared expert + residual).

``mode="nccl"`` is the comparison: the same GEMMs around ``all_to_all_single`` with host-read counts.
The reference has no expert parallelism (docs/17-running-models.md:455-470).
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ..models.config import ModelConfig
from ..models.moe import router_cat
from ..models.weights import ModelWeights, random_weights
from ..ops import gemm as G
from ..ops import lib as K
from ..ops import moe as M
from ..utils import quant as Q
from .symm import MAX_RANKS, SymmBuffer, Wire


def ep_shard_weights(full: ModelWeights, rank: int, world: int) -> ModelWeights:
    """This rank's experts of a whole model (tests; views of the stacked tensors, nothing is copied twice)."""
    cfg = full.cfg
    el = cfg.n_experts // world
    layers = []
    for lw in full.layers:
        l2 = dataclasses.replace(lw)
        if lw.experts is not None:
            l2.experts = lw.experts[rank * el: (rank + 1) * el]
            l2.experts_gate_up_w4b = lw.experts_gate_up_w4b[rank * el: (rank + 1) * el].contiguous()
            l2.experts_down_w4b = lw.experts_down_w4b[rank * el: (rank + 1) * el].contiguous()
        layers.append(l2)
    return ModelWeights(cfg, full.embed, full.lm_head, full.final_norm, layers)


def random_ep_shard(cfg: ModelConfig, rank: int, world: int, device, seed: int = 0) -> ModelWeights:
    """Random-init weights with only this rank's experts materialised (full-size shapes)."""
    el = cfg.n_experts // world
    local = dataclasses.replace(cfg, n_experts=el)
    w = random_weights(local, device=device, seed=seed * 16 + rank, exact=False)
    g = torch.Generator(device=device)
    g.manual_seed(seed)            # the router is the same on every rank
    for lw in w.layers:
        if lw.router is not None:
            lw.router = (torch.randn(cfg.n_experts, cfg.hidden, generator=g, device=device) * cfg.hidden ** -0.5).to(torch.bfloat16)
            if hasattr(lw, "_router_cat"):
                delattr(lw, "_router_cat")
    w.cfg = cfg
    return w


class EpMoe:
    def __init__(self, cfg: ModelConfig, max_tokens: int, group=None, device=None, mode: str = "fused",
                 overflow: Optional[float] = None):
        import torch.distributed as dist
        self.cfg, self.group, self.mode = cfg, group, mode
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.dev = device or torch.device("cuda", torch.cuda.current_device())
        e, k, h, i = cfg.n_experts, cfg.top_k, cfg.hidden, cfg.expert_ffn
        if e % self.world:
            raise ValueError(f"expert parallel {self.world} does not divide {e} experts")
        self.el = e // self.world
        t = self.t_cap = max_tokens
        # receive buffer: by default the worst case (every rank sends all its rows here), so routing skew can
        # never overflow it; `overflow` (a multiple of the uniform-routing T k rows) trades memory for the
        # risk -- a rank that is sent more than its buffer holds reports it in the status word and drops rows
        if overflow is None:
            overflow = float(self.world)
        self.cap_rows = (int(t * k * overflow) + self.el * 128 + 127) // 128 * 128
        self.max_blk = self.cap_rows // 128
        i32, f32, bf = torch.int32, torch.float32, torch.bfloat16
        dev = self.dev
        self.ld = (e + (1 if cfg.shared_ffn else 0) + 7) // 8 * 8
        self.logits = torch.empty(t, self.ld, dtype=f32, device=dev)
        self.topk_idx = torch.empty(t * k, dtype=i32, device=dev)
        self.topk_w = torch.empty(t * k, dtype=f32, device=dev)
        self.counts = torch.zeros(e, dtype=i32, device=dev)
        self.rank_in = torch.empty(t * k, dtype=i32, device=dev)
        self.send_base = torch.zeros(e, dtype=i32, device=dev)
        self.blk_expert = torch.zeros(self.max_blk, dtype=i32, device=dev)
        self.blk_row0 = torch.zeros(self.max_blk, dtype=i32, device=dev)
        self.blk_rows = torch.zeros(self.max_blk, dtype=i32, device=dev)
        self.n_blk = torch.zeros(1, dtype=i32, device=dev)
        self.total_rows = torch.zeros(1, dtype=i32, device=dev)
        self.act = torch.zeros(self.cap_rows, i, dtype=bf, device=dev)
        self.shared_y = torch.empty(t, h, dtype=bf, device=dev) if cfg.shared_ffn else None
        self.ident = torch.arange(t * k, dtype=i32, device=dev)     # slot s of token t is row t k + s of the return buffer
        self.epoch = 0
        self.slab_gu = self.slab_dn = None
        if mode == "fused":
            w = self.world
            self.cntw = Wire(w * e * 4, w, 0, group, dev)
            self.recvw = Wire(self.cap_rows * h * 2, 2 * self.max_blk, 0, group, dev)
            self.srcb = SymmBuffer(self.cap_rows * 4, group, dev)
            tab = [0] * MAX_RANKS
            for r in range(w):
                tab[r] = self.srcb.ptrs[r]
            self.src_table = torch.tensor(tab, dtype=torch.int64, device=dev)
            self.retw = Wire(t * k * h * 2, w, 0, group, dev)
            self.recv_x = self.recvw.buf.view(bf, 0, self.cap_rows * h).view(self.cap_rows, h)
            self.recv_src = self.srcb.view(i32, 0, self.cap_rows)
            self.ret = self.retw.buf.view(bf, 0, t * k * h).view(t * k, h)
        else:
            self.y = torch.zeros(self.cap_rows, h, dtype=bf, device=dev)
            self.xs = torch.zeros(self.cap_rows, h, dtype=bf, device=dev)
            self.rank2 = torch.empty(self.cap_rows, dtype=i32, device=dev)
            self.counts2 = torch.zeros(self.el, dtype=i32, device=dev)
            self.expert_base = torch.zeros(self.el, dtype=i32, device=dev)
            self.row_of = torch.empty(self.cap_rows, dtype=i32, device=dev)

    # ------------------------------------------------------------------ decode rows
    def enable_rows(self, max_rows: int):
        """Buffers of the decode / verify form (at most ``max_rows`` rows per rank and step): on the experts' owner
        the received rows go through the batched W4 GEMV, one (row, expert) pair per batch, reading int4 weights."""
        cfg, dev = self.cfg, self.dev
        k, h, i = cfg.top_k, cfg.hidden, cfg.expert_ffn
        if max_rows > self.t_cap:
            raise ValueError("more decode rows than the exchange buffers were sized for")
        self.rows_cap = max_rows
        self.cap_pairs = max_rows * k * self.world            # every pair of every rank could land here
        if self.cap_pairs > 65535:
            raise ValueError("too many (row, expert) pairs for one batched GEMV launch")
        i32, f32, bf = torch.int32, torch.float32, torch.bfloat16
        self.cx = torch.zeros(self.cap_pairs, h, dtype=bf, device=dev)
        self.cexp = torch.full((self.cap_pairs,), -1, dtype=i32, device=dev)
        self.csrc = torch.zeros(self.cap_pairs, dtype=i32, device=dev)
        self.n_valid = torch.zeros(1, dtype=i32, device=dev)
        self.s_gu, self.s_dn = K.gemv_splits(2 * i, h), K.gemv_splits(h, i)
        self.part_gu = torch.zeros(self.cap_pairs * self.s_gu * 2 * i, dtype=f32, device=dev)
        self.part_dn = torch.zeros(self.cap_pairs * self.s_dn * h, dtype=f32, device=dev)
        self.rows_act = torch.empty(max_rows, max(cfg.shared_ffn, 8), dtype=bf, device=dev) if cfg.shared_ffn else None

    def block_rows(self, lw, c: int, x, resid):
        """``resid[:c] += MoE(x[:c])`` for the ``c`` rows of a decode / verify step (``c`` may differ between ranks,
        every rank calls this once per MoE layer).  Fused mode only: route -> counts exchange -> plan -> dispatch as in the
        prompt form; the owner gathers the rows that arrived, runs gate‖up and down as batched int4 GEMVs, and stores
        each result row into its source's return buffer; the source sums a row's slots in slot order."""
        if self.mode != "fused":
            raise NotImplementedError("decode rows under expert parallelism use the fused wire")
        cfg = self.cfg
        e, k, h, i = cfg.n_experts, cfg.top_k, cfg.hidden, cfg.expert_ffn
        x, resid = x[:c], resid[:c]
        logits = self.logits[:c]
        rc = router_cat(lw, cfg)
        if c > 0:
            K.head_gemv(rc, x, logits, c, rc.shape[0], h)
            M.route(logits, self.ld, c, e, k, self.topk_idx, self.topk_w)
        self.epoch += 1
        ep, par = self.epoch, self.epoch & 1
        self.counts.zero_()
        if c > 0:
            M.count(self.topk_idx, c * k, self.counts, self.rank_in)
        L = K.lib()
        K._check(L.b2_ep_counts_push(K._p(self.counts), e, K._p(self.cntw.table), self.world, self.rank, ep, K._stream()),
                 "ep_counts_push")
        blk_cnt = self.recvw.flags
        K._check(L.b2_ep_plan(K._p(self.cntw.table), ep, e, self.world, self.rank, self.max_blk, self.cap_rows,
                              K._p(self.send_base), K._p(self.blk_expert), K._p(self.blk_row0), K._p(self.blk_rows),
                              K._p(self.n_blk), K._p(self.total_rows), K._p(blk_cnt[(par ^ 1) * self.max_blk:]),
                              K._stream()), "ep_plan")
        if c > 0:
            K._check(L.b2_ep_dispatch(K._p(self.topk_idx), K._p(self.rank_in), K._p(self.send_base), K._p(x), c, k, h, e,
                                      self.world, self.rank, self.cap_rows, par, self.max_blk, K._p(self.recvw.table),
                                      K._p(self.src_table), K._stream()), "ep_dispatch")
        K._check(L.b2_ep_rows_gather(K._p(self.blk_expert), K._p(self.blk_row0), K._p(self.blk_rows), K._p(self.n_blk),
                                     self.max_blk, K._p(blk_cnt[par * self.max_blk:]), K._p(self.recv_x), K._p(self.recv_src),
                                     h, self.cap_pairs, K._p(self.cx), K._p(self.cexp), K._p(self.csrc), K._p(self.n_valid),
                                     K._stream()), "ep_rows_gather")
        gu_bytes = lw.experts_gate_up_w4b[0].numel()
        dn_bytes = lw.experts_down_w4b[0].numel()
        M.gemv_experts(lw.experts_gate_up_w4b, gu_bytes, self.cexp, self.cap_pairs, self.cx, 1, h * 2, self.part_gu, 2 * i, h,
                       self.s_gu, h, sparse=True)
        M.gemv_experts(lw.experts_down_w4b, dn_bytes, self.cexp, self.cap_pairs, self.part_gu, 1, self.s_gu * 2 * i * 4,
                       self.part_dn, h, i, self.s_dn, 2 * i, x_mode=1, s_in=self.s_gu, x_slice=2 * i, sparse=True)
        K._check(L.b2_ep_rows_return(K._p(self.part_dn), K._p(self.cexp), K._p(self.csrc), self.cap_pairs, self.s_dn, h,
                                     K._p(self.retw.table), K._stream()), "ep_rows_return")
        K._check(L.b2_ep_flag_all(K._p(self.retw.table), self.world, self.rank, ep, K._stream()), "ep_flag_all")
        shared_y, gate = None, None
        if lw.shared is not None and c > 0:
            act = self.rows_act[:c, : cfg.shared_ffn]
            G.gemm_w4(x, lw.shared.gate_up.w4b, lw.shared.gate_up.n, lw.shared.gate_up.k, act, epi=G.EPI_SILU_MUL)
            shared_y = self.shared_y[:c]
            G.gemm_w4(act, lw.shared.down.w4b, lw.shared.down.n, lw.shared.down.k, shared_y, epi=G.EPI_BF16)
            gate = logits[:, e:]
        ep_wait_all(self.retw, self.epoch)
        if c > 0:
            M.combine(self.ret, self.ident, self.topk_w, c, k, h, shared_y, gate, self.ld, resid, resid)

    # ------------------------------------------------------------------ expert weights (bf16 forms)
    def _expert_bf16(self, runner, lw):
        cfg = self.cfg
        h, i, el = cfg.hidden, cfg.expert_ffn, self.el
        cached = getattr(lw, "_experts_bf16", None)
        if cached is not None:
            return cached
        if runner.backend == "bf16-resident":
            gu = G.dequant_w4b(lw.experts_gate_up_w4b.view(-1, h // 64, Q.BLOCK_BYTES), el * 2 * i, h).view(el, 2 * i, h)
            dn = G.dequant_w4b(lw.experts_down_w4b.view(-1, i // 64, Q.BLOCK_BYTES), el * h, i).view(el, h, i)
            lw._experts_bf16 = (gu, dn)
            return lw._experts_bf16
        if self.slab_gu is None:
            self.slab_gu = torch.empty(el, 2 * i, h, dtype=torch.bfloat16, device=self.dev)
            self.slab_dn = torch.empty(el, h, i, dtype=torch.bfloat16, device=self.dev)
        G.dequant_w4b(lw.experts_gate_up_w4b, el * 2 * i, h, self.slab_gu)
        G.dequant_w4b(lw.experts_down_w4b, el * h, i, self.slab_dn)
        return self.slab_gu, self.slab_dn

    # ------------------------------------------------------------------ one block
    def block_prefill(self, runner, lw, c: int):
        """``runner.resid[:c] += MoE(runner.x[:c])`` with the experts of all ranks."""
        cfg = self.cfg
        e, k, h = cfg.n_experts, cfg.top_k, cfg.hidden
        x, resid = runner.x[:c], runner.resid[:c]
        logits = self.logits[:c]
        G.gemm_bf16(x, router_cat(lw, cfg), logits, epi=G.EPI_F32)
        M.route(logits, self.ld, c, e, k, self.topk_idx, self.topk_w)
        shared_y, gate = None, None
        if self.mode == "fused":
            self._fused(runner, lw, c, x)
            y, row_of = self.ret, self.ident
        else:
            y, row_of = self._nccl(runner, lw, c, x)
        if lw.shared is not None:
            act = runner.act[:c, : cfg.shared_ffn]
            runner.linear(lw.shared.gate_up, x, act, G.EPI_SILU_MUL)
            shared_y = self.shared_y[:c]
            runner.linear(lw.shared.down, act, shared_y, G.EPI_BF16)
            gate = logits[:, e:]
        if self.mode == "fused":
            ep_wait_all(self.retw, self.epoch)
        M.combine(y, row_of, self.topk_w, c, k, h, shared_y, gate, self.ld, resid, resid)

    def _fused(self, runner, lw, c: int, x):
        cfg = self.cfg
        e, k, h = cfg.n_experts, cfg.top_k, cfg.hidden
        self.epoch += 1
        ep, par = self.epoch, self.epoch & 1
        self.counts.zero_()
        M.count(self.topk_idx, c * k, self.counts, self.rank_in)
        L = K.lib()
        K._check(L.b2_ep_counts_push(K._p(self.counts), e, K._p(self.cntw.table), self.world, self.rank, ep, K._stream()),
                 "ep_counts_push")
        blk_cnt = self.recvw.flags
        K._check(L.b2_ep_plan(K._p(self.cntw.table), ep, e, self.world, self.rank, self.max_blk, self.cap_rows,
                              K._p(self.send_base), K._p(self.blk_expert), K._p(self.blk_row0), K._p(self.blk_rows),
                              K._p(self.n_blk), K._p(self.total_rows), K._p(blk_cnt[(par ^ 1) * self.max_blk:]),
                              K._stream()), "ep_plan")
        K._check(L.b2_ep_dispatch(K._p(self.topk_idx), K._p(self.rank_in), K._p(self.send_base), K._p(x), c, k, h, e,
                                  self.world, self.rank, self.cap_rows, par, self.max_blk, K._p(self.recvw.table),
                                  K._p(self.src_table), K._stream()), "ep_dispatch")
        gu, dn = self._expert_bf16(runner, lw)
        blocks = (self.blk_expert, self.blk_row0, self.blk_rows, self.n_blk, self.max_blk)
        G.gemm_grouped_ep(self.recv_x, gu, self.act, blocks, G.EPI_SILU_MUL, blk_wait=blk_cnt[par * self.max_blk:])
        G.gemm_grouped_ep(self.act, dn, None, blocks, G.EPI_EP_RETURN, row_src=self.recv_src, ret_table=self.retw.table)
        K._check(L.b2_ep_flag_all(K._p(self.retw.table), self.world, self.rank, ep, K._stream()), "ep_flag_all")

    def _nccl(self, runner, lw, c: int, x):
        """Comparison: sort by destination on the device, read the counts on the host, NCCL all-to-all both ways."""
        import torch.distributed as dist
        cfg = self.cfg
        e, k, h, el, w = cfg.n_experts, cfg.top_k, cfg.hidden, self.el, self.world
        idx = self.topk_idx[: c * k].long()
        order = torch.argsort(idx, stable=True)                    # rows sorted by expert = by destination
        send_x = x[order // k]
        send_e = idx[order].to(torch.int32)
        per_dest = torch.bincount(idx // el, minlength=w)
        recv_counts = torch.empty_like(per_dest)
        if w > 1:
            dist.all_to_all_single(recv_counts, per_dest, group=self.group)
        else:
            recv_counts.copy_(per_dest)
        ins, outs = per_dest.tolist(), recv_counts.tolist()        # host reads the counts (a sync per block)
        n_in = sum(outs)
        if n_in > self.cap_rows - el * 128:
            raise RuntimeError("expert-parallel receive buffer is too small for this routing")
        rx = torch.empty(n_in, h, dtype=x.dtype, device=x.device)
        re = torch.empty(n_in, dtype=torch.int32, device=x.device)
        if w > 1:
            dist.all_to_all_single(rx, send_x, outs, ins, group=self.group)
            dist.all_to_all_single(re, send_e, outs, ins, group=self.group)
        else:
            rx.copy_(send_x)
            re.copy_(send_e)
        if n_in == 0:      # nothing was routed to this rank's experts: only the exchange back remains
            back = rx
        re_local = (re - self.rank * el).contiguous()
        self.counts2.zero_()
        if n_in > 0:
            M.sort(re_local, n_in, 1, el, self.max_blk, self.counts2, self.rank2, self.expert_base, self.blk_expert,
                   self.blk_row0, self.blk_rows, self.n_blk, self.total_rows)
            M.scatter(re_local, self.rank2, self.expert_base, n_in, 1, rx, h, self.row_of, self.xs)
            gu, dn = self._expert_bf16(runner, lw)
            blocks = (self.blk_expert, self.blk_row0, self.blk_rows, self.n_blk, self.max_blk)
            G.gemm_grouped_bf16(self.xs, gu, self.act, blocks, epi=G.EPI_SILU_MUL)
            G.gemm_grouped_bf16(self.act, dn, self.y, blocks, epi=G.EPI_BF16)
            back = self.y[self.row_of[:n_in].long()]
        ret_sorted = torch.empty(c * k, h, dtype=x.dtype, device=x.device)
        if w > 1:
            dist.all_to_all_single(ret_sorted, back, ins, outs, group=self.group)
        else:
            ret_sorted.copy_(back)
        row_of = torch.empty(c * k, dtype=torch.int32, device=x.device)
        row_of[order] = torch.arange(c * k, dtype=torch.int32, device=x.device)
        return ret_sorted, row_of

    def close(self):
        if self.mode == "fused":
            self.recv_x = self.recv_src = self.ret = None
            for b in (self.cntw, self.recvw, self.retw):
                b.close()
            self.srcb.close()


def ep_wait_all(wire: Wire, epoch: int):
    K._check(K.lib().b2_ep_wait_all(K._p(wire.table), wire.world, wire.rank, epoch, K._stream()), "ep_wait_all")


def bench_prefill(cfg: ModelConfig, n: int, modes=("fused", "nccl"), reps: int = 4) -> dict:
    """Every rank ingests its own ``n``-token prompt: data-parallel attention, expert-parallel MoE.  Returns the
    group's tokens/s per mode (CUDA events, max over ranks)."""
    import torch.distributed as dist
    from ..runtime.engine import Engine
    from ..runtime.prefill import PrefillRunner
    from .tp import _max_over_ranks, _sync_all
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    out = {}
    w = random_ep_shard(cfg, rank, world, dev)
    g = torch.Generator().manual_seed(100 + rank)
    ids = torch.randint(0, cfg.vocab, (n,), generator=g).tolist()
    for mode in modes:
        eng = Engine(w, max_seqs=1, max_len=n + 64, use_graphs=False, prefill_backend="bf16-resident")
        runner = PrefillRunner(eng, max_chunk=min(n, 4096))
        runner.ep = EpMoe(cfg, min(n, 4096), mode=mode)
        for _ in range(2):
            eng.reset(0)
            runner.run(0, ids)
        _sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            eng.reset(0)
            runner.run(0, ids)
        e1.record()
        _sync_all()
        ms = _max_over_ranks(e0.elapsed_time(e1) / reps, dev)
        K.check_status()
        out[f"prefill_{mode}"] = {"ms": ms, "tokens": n * world, "tokens_per_s": n * world / (ms / 1e3),
                                  "parallelism": f"dp{world} attention + ep{world} experts"}
        runner.ep.close()
        del eng, runner
        torch.cuda.empty_cache()
    return out


def attach_rows(engine, max_rows: int) -> "EpMoe":
    """Makes ``engine`` (which holds only this rank's experts) run the MoE layers of its decode / verify steps through
    the expert-parallel row form.  Such an engine steps eagerly: the exchange's call numbers are launch arguments."""
    if engine.use_graphs:
        raise ValueError("an expert-parallel decode engine runs without CUDA graphs (use_graphs=False)")
    ep = EpMoe(engine.cfg, max(max_rows, 8), mode="fused")
    ep.enable_rows(max_rows)
    engine.model.ep = ep
    return ep


def bench_decode_rows(cfg: ModelConfig, rows_per_rank: int, depth: int, steps: int = 32, warmup: int = 4) -> dict:
    """Batched decode with the experts spread over the ranks: every rank serves ``rows_per_rank`` requests of its own
    at context ``depth`` (data-parallel attention); one step emits ``world * rows_per_rank`` tokens.  CUDA events,
    max over ranks."""
    import torch.distributed as dist
    from ..runtime.engine import Engine, Row
    from .tp import _max_over_ranks, _sync_all
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    w = random_ep_shard(cfg, rank, world, dev)
    eng = Engine(w, max_seqs=rows_per_rank, max_len=depth + steps + warmup + 64, use_graphs=False)
    ep = attach_rows(eng, rows_per_rank)
    eng.kv.k.normal_(0, 0.5)
    eng.kv.v.normal_(0, 0.5)
    for slot in range(rows_per_rank):
        eng._ensure_pages(slot, depth)
        eng.seq_len[slot] = depth
    toks = [17 + slot for slot in range(rows_per_rank)]

    def step(toks):
        return eng.forward_rows([Row(slot, eng.seq_len[slot], toks[slot]) for slot in range(rows_per_rank)])
    for _ in range(warmup):
        toks = step(toks)
    _sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        toks = step(toks)
    e1.record()
    _sync_all()
    ms = _max_over_ranks(e0.elapsed_time(e1) / steps, dev)
    K.check_status()
    out = {"ms_per_step": ms, "rows_total": world * rows_per_rank, "tokens_per_s": world * rows_per_rank / (ms / 1e3),
           "depth": depth, "parallelism": f"dp{world} attention + ep{world} experts",
           "note": "eager steps (no CUDA graph), each with its host round trip"}
    ep.close()
    return out
