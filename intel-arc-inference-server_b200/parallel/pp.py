"""Pipeline parallelism: contiguous layer ranges per rank, activations handed on with NCCL p2p.

Stage ``s`` holds layers ``[a_s, b_s)``; stage 0 also embeds, the last stage also runs the head.  The
hand-off after a stage's last layer is the FOLDED residual rows (bf16 ``[M][hidden]``) plus their per-block
sums of squares (fp32 ``[M][hidden / 128]``), about 10 KB per row at hidden 5120 -- the cut the reference
chose for its two-card pipeline so that the norm is not recomputed (src/runtime/pipeline_engine.h:25-67,
pipeline_plan.h:11-33,61-66).  ``send`` / ``recv`` are stream-ordered NCCL calls: a stage enqueues its send
and goes on to its next micro-batch or prompt chunk while the next stage computes, which is the overlap a
chunk pipeline needs.  The sampled tokens come back from the last stage with one small broadcast per step.
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
        mdl.layers_walk(mdl.w.layers, m, self.ctrl, self.block_table, self.max_blocks, self.kv,
                        first_from_embed=self.first, resid_ready=not self.first)
        if not self.last:
            dist.send(b.resid[:m], dst=self._peer(self.stage + 1), group=self.group)
            dist.send(b.ssq[: m * nb], dst=self._peer(self.stage + 1), group=self.group)
            self.sent_bytes += m * h * 2 + m * nb * 4
        else:
            mdl.head(m, (None, 0), self.ctrl, advance)
        # the tokens (and logit values) return to every stage; stage 0 needs them for the next embedding
        out = self.ctrl[K.CTRL_OUT_TOKEN: K.CTRL_OUT_VALUE + 64]
        dist.broadcast(out, src=self._peer(self.stages - 1), group=self.group)
        if advance and not self.last:
            self.ctrl[K.CTRL_CUR_TOKEN: K.CTRL_CUR_TOKEN + m] = self.ctrl[K.CTRL_OUT_TOKEN: K.CTRL_OUT_TOKEN + m]
            self.ctrl[K.CTRL_ROW_POS: K.CTRL_ROW_POS + m] += 1
