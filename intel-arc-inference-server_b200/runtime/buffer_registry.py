"""One table for every device buffer of a decode step: which memory-plan group pays for it, whether ``reset`` clears
it and whether it belongs to a session snapshot.

The reference ties its buffers to its planner at compile time: every buffer must have a size member annotated with
plan group / reset / snapshot, or the build fails (src/runtime/gpu_state.h:1-80, negative compile test
tests/runtime/gpu_state_fail.cc).  Python has no compile step, so the same promise is an audit that runs in the
tests and at engine start-up under ``B200SERVE_AUDIT=1``: a tensor attribute that is not in the table, or a group
that holds more bytes than the planner budgets for it, raises.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..models.config import ModelConfig
from . import memory_plan as MP

# attribute -> (plan group, cleared by Engine.reset(slot), part of save_kv / load_kv snapshots)
STEP_BUFFERS: Dict[str, Tuple[str, bool, bool]] = {
    "resid": ("step", False, False), "x": ("step", False, False), "q": ("step", False, False),
    "attn_out": ("step", False, False), "o_part": ("step", False, False), "ml_part": ("step", False, False),
    "logits": ("step", False, False), "cand_val": ("step", False, False), "cand_idx": ("step", False, False),
    "flag": ("step", False, False), "tickets": ("step", False, False), "fold_tickets": ("step", False, False), "qkv_tickets": ("step", False, False),
    "ssq": ("step", False, False), "xq": ("step", False, False), "xq_gs": ("step", False, False),
    "gdn_act": ("step", False, False), "gdn_out": ("step", False, False),
}
KV_BUFFERS: Dict[str, Tuple[str, bool, bool]] = {
    "k": ("kv", False, True), "v": ("kv", False, True), "k_scale": ("kv", False, True), "v_scale": ("kv", False, True),
    "gdn_conv": ("state", True, True), "gdn_state": ("state", True, True),
}


def _tensors(obj):
    return {n: v for n, v in vars(obj).items() if isinstance(v, torch.Tensor)}


def audit(buf, kv, cfg: ModelConfig, kv_dtype: str = "bf16", max_seqs: int = 1) -> Dict[str, int]:
    """Checks ``buf`` (StepBuffers) and ``kv`` (KVCache) against the tables and the planner; returns bytes per group."""
    groups = {"step": 0, "kv": 0, "state": 0}
    for obj, table, what in ((buf, STEP_BUFFERS, "StepBuffers"), (kv, KV_BUFFERS, "KVCache")):
        for name, t in _tensors(obj).items():
            if name not in table:
                raise AssertionError(f"{what}.{name} has no entry in runtime/buffer_registry.py: the memory planner does "
                                     "not know this buffer")
            groups[table[name][0]] += t.numel() * t.element_size()
    for t in getattr(buf, "_parts", {}).values():      # split-K partial sums, allocated on first use per linear
        groups["step"] += t.numel() * t.element_size()
    nsplit = buf.o_part.numel() // max(1, buf.max_rows * cfg.n_q_heads * cfg.head_dim)
    planned_step = MP.step_scratch_bytes(cfg, buf.max_rows, nsplit)
    if groups["step"] > planned_step:
        raise AssertionError(f"step buffers hold {groups['step']} bytes, the planner budgets {planned_step}")
    planes = max(1, kv.k.shape[0])
    per_page = MP.kv_bytes_per_page(cfg, kv_dtype) // max(1, cfg.n_layers - cfg.n_gdn_layers + cfg.mtp_layers) * planes
    planned_kv = kv.num_pages * per_page
    if groups["kv"] != planned_kv:
        raise AssertionError(f"KV pool holds {groups['kv']} bytes, the planner counts {planned_kv} for {kv.num_pages} pages")
    planned_state = max_seqs * MP.gdn_state_bytes_per_slot(cfg)
    if groups["state"] > planned_state:
        raise AssertionError(f"recurrent state holds {groups['state']} bytes, the planner budgets {planned_state}")
    return groups
