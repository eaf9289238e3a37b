"""Pipeline parallelism: contiguous layer ranges per rank, activations handed on with NCCL p2p.

Stage ``s`` holds layers ``[a_s, b_s)``; stage 0 also embeds, the last stage also runs the head.  The
hand-off after a stage's last layer is the FOLDED residual rows (bf16 ``[M][hidden]``) plus their per-block
sums of squares (fp32 ``[M][hidden / 128]``), about 10 KB per row at hidden 5120 -- the cut the reference
chose for its two-card pipeline so that the norm is not recomputed (src/runtime/pipeline_engine.h:25-67,
pipeline_plan.h:11-33,61-66).  ``send`` / ``recv`` are stream-ordered NCCL calls: a stage enqueues its send
and goes on to its next micro-batch or prompt chunk while the next stage computes, which is the overlap a
chunk pipeline needs.  The sampled tokens come back from the last stage with one small broadcast per step.

Prompt pass: every stage runs the tcgen05 prompt kernels over its own layers, chunk by chunk; chunk ``c`` is handed
on as soon as the stage's last layer is done with it and the host never waits in between, so stage ``s`` works on
chunk ``c`` while stage ``s + 1`` works on chunk ``c - 1`` (src/runtime/prefill/pipeline_prefill.cc has the same
shape).  Decode: the compute between two hand-offs (the stage's layers, the head on the last stage) is a captured
CUDA graph per row count; only the hand-offs themselves are enqueued call by call.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence, Tuple

import torch

from ..models.config import ModelConfig
from ..models.weights import ModelWeights, random_weights
from ..ops import lib as K
from ..runtime.engine import Engine, Row


def split_layers(n_layers: int, stages: int, head_cost: float = 1.5) -> List[Tuple[int, int]]:
    """Contiguous ranges balanced by bytes read per token; the head counts as ``head_cost`` layers on the last
    stage (pipeline_plan.h:11-33 balances the same way)."""
    total = n_layers + head_cost
    out, a = [], 0
    for s in range(stages):
        target = total * (s + 1) / stages
        b = n_layers if s == stages - 1 else max(a + 1, min(n_layers - (stages - 1 - s), round(target)))
        out.append((a, b))
        a = b
    return out


def stage_weights(full: ModelWeights, a: int, b: int) -> ModelWeights:
    cfg = dataclasses.replace(full.cfg, n_layers=b - a, name=f"{full.cfg.name}/layers{a}-{b}")
    return ModelWeights(cfg, full.embed, full.lm_head, full.final_norm, full.layers[a:b])


def random_stage(cfg: ModelConfig, a: int, b: int, device, seed: int = 0) -> ModelWeights:
    local = dataclasses.replace(cfg, n_layers=b - a, name=f"{cfg.name}/layers{a}-{b}")
    return random_weights(local, device=device, seed=seed * 16 + a, exact=False)


class PipelineEngine(Engine):
    """One stage of the pipeline; every rank makes the same calls in the same order."""

    def __init__(self, weights: ModelWeights, stage: int, stages: int, group=None, **kw):
        kw["use_graphs"] = False       # NCCL p2p between the stages: steps are enqueued, not replayed
        kw.setdefault("prefill_backend", "rows")
        super().__init__(weights, **kw)
        self.stage, self.stages, self.group = stage, stages, group
        self.first, self.last = stage == 0, stage == stages - 1
        self.sent_bytes = 0
        self.stage_graphs = True
        self._stage_graph = {}
        self._pp_runner = None
        self._land = None

    def _peer(self, s: int) -> int:
        import torch.distributed as dist
        return dist.get_global_rank(self.group, s) if self.group is not None else s

    def _enqueue(self, m: int, advance: bool):
        import torch.distributed as dist
        mdl, b = self.model, self.model.buf
        h = self.cfg.hidden
        nb = (h + 127) // 128
        if not self.first:
            dist.recv(b.resid[:m], src=self._peer(self.stage - 1), group=self.group)
            dist.recv(b.ssq[: m * nb], src=self._peer(self.stage - 1), group=self.group)
        self._stage_compute(m, advance)
        if not self.last:
            dist.send(b.resid[:m], dst=self._peer(self.stage + 1), group=self.group)
            dist.send(b.ssq[: m * nb], dst=self._peer(self.stage + 1), group=self.group)
            self.sent_bytes += m * h * 2 + m * nb * 4
        # the tokens (and logit values) return to every stage; stage 0 needs them for the next embedding
        out = self.ctrl[K.CTRL_OUT_TOKEN: K.CTRL_OUT_VALUE + 64]
        dist.broadcast(out, src=self._peer(self.stages - 1), group=self.group)
        if advance and not self.last:
            self.ctrl[K.CTRL_CUR_TOKEN: K.CTRL_CUR_TOKEN + m] = self.ctrl[K.CTRL_OUT_TOKEN: K.CTRL_OUT_TOKEN + m]
            self.ctrl[K.CTRL_ROW_POS: K.CTRL_ROW_POS + m] += 1

    def _stage_body(self, m: int, advance: bool):
        mdl = self.model
        mdl.layers_walk(mdl.w.layers, m, self.ctrl, self.block_table, self.max_blocks, self.kv,
                        first_from_embed=self.first, resid_ready=not self.first)
        if self.last:
            mdl.head(m, (None, 0), self.ctrl, advance)

    def _stage_compute(self, m: int, advance: bool):
        """The stage's layers (and the head on the last stage) as one captured graph per (rows, advance): between two
        hand-offs the host issues one launch instead of several hundred."""
        if not self.stage_graphs or self.kv.gdn_state is not None:
            return self._stage_body(m, advance)
        key = (m, advance)
        g = self._stage_graph.get(key)
        if g is None:
            # warm-up outside capture (function attributes, scratch), then put back what it changed: the control
            # block, and on a later stage the rows it received (the walk folds into them in place)
            b = self.model.buf
            saved = self.ctrl.clone()
            rows_in = None if self.first else (b.resid[:m].clone(), b.ssq.clone())
            self._stage_body(m, advance)
            torch.cuda.current_stream().synchronize()
            self.ctrl.copy_(saved)
            if rows_in is not None:
                b.resid[:m].copy_(rows_in[0])
                b.ssq.copy_(rows_in[1])
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._stage_body(m, advance)
            self.ctrl.copy_(saved)
            self._stage_graph[key] = g
        g.replay()

    # ------------------------------------------------------------------ prompt pass
    def prefill(self, slot: int, ids: Sequence[int], chunk: Optional[int] = None) -> int:
        ids = list(ids)
        if len(ids) <= self.max_rows or self.cfg.head_dim != 128 or self.kv.kv_int8 or self.cfg.n_gdn_layers:
            return super().prefill(slot, ids, chunk)      # short prompts and the forms without a tcgen05 path: row steps
        return self._prefill_chunks(slot, ids, chunk)

    def _prefill_chunks(self, slot: int, ids: List[int], chunk: Optional[int]) -> int:
        import torch.distributed as dist
        from ..runtime.prefill import PrefillRunner
        self.require_ok()
        cfg, mdl = self.cfg, self.model
        if self._pp_runner is None:
            saved, self.prefill_backend = self.prefill_backend, "auto"
            self._pp_runner = PrefillRunner(self)
            self.prefill_backend = saved
            r = self._pp_runner
            # two landing buffers: a chunk that is still being sent is not overwritten by the next one
            self._land = [r.resid, torch.empty_like(r.resid)]
        r = self._pp_runner
        chunk = min(chunk or r.max_chunk, r.max_chunk)
        start, n = self.seq_len[slot], len(ids)
        buf = None
        for ci, c0 in enumerate(range(0, n, chunk)):
            part = ids[c0: c0 + chunk]
            c, pos0 = len(part), start + c0
            self._ensure_pages(slot, pos0 + c)
            buf = self._land[ci & 1][:c]
            if self.first:
                host = r.ids_stage.begin()
                host[:c] = torch.as_tensor(part, dtype=torch.int64)
                r.ids_stage.push(r.ids_dev[:c], host[:c])
                torch.index_select(mdl.w.embed, 0, r.ids_dev[:c], out=buf)
            else:
                dist.recv(buf, src=self._peer(self.stage - 1), group=self.group)
            x = r.x[:c]
            for li, lw in enumerate(mdl.w.layers):
                r.layer(lw, li, slot, c, pos0, buf, x)
            if not self.last:
                dist.send(buf, dst=self._peer(self.stage + 1), group=self.group)
                self.sent_bytes += c * cfg.hidden * 2
            self.seq_len[slot] = max(self.seq_len[slot], pos0 + c)
        if self.last:
            mdl.buf.resid[0].copy_(buf[(n - 1) % chunk])
            r._head_of_row0()
        out = self.ctrl[K.CTRL_OUT_TOKEN: K.CTRL_OUT_VALUE + 64]
        dist.broadcast(out, src=self._peer(self.stages - 1), group=self.group)
        self.last_prefill_row = 0
        self.check_failed("prompt pass")
        return self._read_out(1)[0]


def bench_pp(cfg: ModelConfig, prompt_len: int, steps: int = 32, warmup: int = 4) -> dict:
    """The ranks as pipeline stages of ONE model: prompt pass of ``prompt_len`` tokens (tokens/s), then plain decode of
    that request (ms per token).  CUDA events around each part, max over ranks."""
    import torch.distributed as dist
    from .tp import _max_over_ranks, _sync_all
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    a, b = split_layers(cfg.n_layers, world)[rank]
    eng = PipelineEngine(random_stage(cfg, a, b, dev), rank, world, max_seqs=1, max_len=prompt_len + steps + warmup + 64)
    g = torch.Generator().manual_seed(9)
    ids = torch.randint(0, cfg.vocab, (prompt_len,), generator=g).tolist()
    eng.prefill(0, ids[:8192])          # builds the runner, its resident weights and the kernels' attributes
    eng.reset(0)
    _sync_all()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    e[0].record()
    tok = eng.prefill(0, ids)
    e[1].record()
    eng.decode_begin([0], [tok])
    for _ in range(warmup):
        eng.decode_step()
    _sync_all()
    e[2].record()
    for _ in range(steps):
        eng.decode_step()
    e[3].record()
    _sync_all()
    K.check_status()
    pms = _max_over_ranks(e[0].elapsed_time(e[1]), dev)
    dms = _max_over_ranks(e[2].elapsed_time(e[3]) / steps, dev)
    return {"stages": world, "layers": [a, b], "prompt_tokens": prompt_len, "prompt_ms": pms,
            "prompt_tokens_per_s": prompt_len / (pms / 1e3), "decode_ms_per_step": dms, "decode_tokens_per_s": 1e3 / dms,
            "depth": prompt_len, "hand_off_bytes": eng.sent_bytes}
