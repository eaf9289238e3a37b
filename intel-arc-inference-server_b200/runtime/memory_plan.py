"""Device-free memory arithmetic: what fits, before anything is allocated.

The role of the reference's planner (src/runtime/memory_plan.h:117-254): from the model
descriptor and the serving options compute the bytes of weights, KV pool, step scratch and
prompt-pass scratch; choose ``max_len`` for ``--max-len auto`` as the largest context whose pool
fits beside the rest with a fixed reserve; refuse at start-up with the numbers when the request
cannot fit.  One source of sizes for the planner and the allocator keeps the two honest.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..models.config import ModelConfig

RESERVE_BYTES = int(1.5 * 2 ** 30)        # left free for the CUDA context, NCCL, fragmentation
HBM_BYTES = 183_359 * 2 ** 20             # what nvidia-smi reports for a B200 (used when no device can be asked)


def device_budget() -> int:
    """Total memory of the current CUDA device as the driver reports it; the B200 figure on a machine without one."""
    try:
        import torch
        if torch.cuda.is_available():
            return int(torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory)
    except Exception:  # noqa: BLE001
        pass
    return HBM_BYTES


@dataclass
class MemoryPlan:
    weights: int
    kv_pool: int
    step_scratch: int
    prefill_scratch: int
    resident_bf16: int
    total: int
    budget: int
    max_len: int
    max_seqs: int
    num_pages: int

    def line(self) -> str:
        g = 2 ** 30
        return (f"memory: model {self.weights / g:.2f} GiB, kv {self.kv_pool / g:.2f} GiB ({self.num_pages} pages, "
                f"{self.max_seqs} x {self.max_len}), decode state {self.step_scratch / g:.2f} GiB, prompt scratch "
                f"{self.prefill_scratch / g:.2f} GiB, total {self.total / g:.2f} of {self.budget / g:.2f} GiB")


def weight_bytes(cfg: ModelConfig, int8_head: bool = False, tp: int = 1, ep: int = 1) -> int:
    h = cfg.hidden
    int4 = 0.5 + 2.0 / 64
    per = cfg._mixer_params() * int4 / tp      # attention projections, or a gated delta-net layer's (mean over layers)
    if cfg.is_moe:
        per += cfg.n_experts * 3 * cfg.expert_ffn * h * int4 / ep + cfg.n_experts * h * 2
        per += 3 * cfg.shared_ffn * h * int4 / tp
    else:
        per += 3 * cfg.ffn * h * int4 / tp
    layers = cfg.n_layers + cfg.mtp_layers
    head = cfg.vocab * h * (1 if int8_head else 2) / tp + (cfg.vocab * h * 2 if int8_head else 0) * 0
    return int(layers * per + cfg.vocab * h * 2 + head)


def kv_bytes_per_page(cfg: ModelConfig, kv_dtype: str, tp: int = 1) -> int:
    per_tok_head = cfg.head_dim * (1 if kv_dtype == "int8" else 2) + (4 if kv_dtype == "int8" else 0)
    return (cfg.n_layers - cfg.n_gdn_layers + cfg.mtp_layers) * 2 * (cfg.n_kv_heads // tp) * per_tok_head * cfg.page_size


def gdn_state_bytes_per_slot(cfg: ModelConfig) -> int:
    """Recurrent state (fp32, one head_dim x head_dim matrix per value head) and convolution window of the gated
    delta-net layers of one sequence slot; twice, for the copy that rewinds rejected rows."""
    if not cfg.n_gdn_layers:
        return 0
    per = cfg.gdn_v_heads * cfg.gdn_head_dim * cfg.gdn_head_dim * 4 + cfg.gdn_conv_channels * 3 * 4
    return 2 * cfg.n_gdn_layers * per


def step_scratch_bytes(cfg: ModelConfig, max_rows: int = 64, nsplit: int = 32) -> int:
    h = cfg.hidden
    b = max_rows * (2 * h * 2 + 2 * cfg.q_dim * 2 + cfg.vocab * 4)
    b += max_rows * cfg.n_q_heads * nsplit * (cfg.head_dim + 2) * 4
    b += 16 * max_rows * (cfg.qkv_dim + 2 * h + 2 * max(cfg.ffn, cfg.expert_ffn * max(cfg.top_k, 1))) * 4
    kmax = max(2 * h, cfg.q_dim, cfg.ffn, cfg.expert_ffn, cfg.shared_ffn, cfg.gdn_value_dim)
    b += max_rows * (kmax // 64) * (128 + 8) + (1 << 16)      # quantised rows + group scales, small control words
    if cfg.n_gdn_layers:
        b += max_rows * (cfg.gdn_proj_dim * 4 + cfg.gdn_value_dim * 2)
    return int(b)


def prefill_scratch_bytes(cfg: ModelConfig, chunk: int, backend: str) -> int:
    h = cfg.hidden
    ffn = cfg.ffn if not cfg.is_moe else max(cfg.expert_ffn, cfg.shared_ffn)
    b = chunk * (2 * h * 2 + cfg.qkv_dim * 4 + 2 * cfg.q_dim * 2 + ffn * 2)
    biggest = max(cfg.qkv_dim * h, h * cfg.q_dim, 2 * ffn * h)
    if backend in ("bf16", "auto"):
        b += biggest * 2
        if cfg.is_moe:
            b += cfg.n_experts * 3 * cfg.expert_ffn * h * 2
    if cfg.is_moe:
        rows = (chunk * cfg.top_k // 128 + cfg.n_experts) * 128
        b += rows * (2 * h + cfg.expert_ffn) * 2
    return int(b)


def plan(cfg: ModelConfig, max_seqs: int, max_len, kv_dtype: str = "bf16", int8_head: bool = False,
         prefill_backend: str = "auto", prefill_chunk: int = 4096, tp: int = 1, ep: int = 1,
         budget: int = 0) -> MemoryPlan:
    """``max_len`` an int or "auto"; ``budget`` 0: what the current device reports.  Raises ValueError with the
    numbers when it cannot fit."""
    budget = budget or device_budget()
    w = weight_bytes(cfg, int8_head, tp, ep)
    resident = 0
    if prefill_backend == "auto":    # the prompt pass keeps bf16 copies when they take at most 45 % of the memory
        prefill_backend = "bf16-resident" if 2 * cfg.param_count() / max(tp * ep, 1) <= 0.45 * budget else "bf16"
    if prefill_backend == "bf16-resident":
        resident = (w - 2 * cfg.vocab * cfg.hidden * 2) * 4      # int4 -> bf16 copies of the linears
    elif prefill_backend in ("int8", "l0-int8"):
        resident = (w - 2 * cfg.vocab * cfg.hidden * 2) * 2
    st = step_scratch_bytes(cfg)
    pf = prefill_scratch_bytes(cfg, prefill_chunk, prefill_backend)
    page = kv_bytes_per_page(cfg, kv_dtype, tp)
    fixed = w + resident + st + pf + RESERVE_BYTES + max_seqs * gdn_state_bytes_per_slot(cfg)
    if fixed >= budget:
        raise ValueError(f"{cfg.name}: weights and scratch need {fixed / 2**30:.1f} GiB of {budget / 2**30:.1f} GiB "
                         "before any KV cache")
    if max_len == "auto":
        pages = (budget - fixed) // page
        max_len = int(min(262144, (pages - 1) // max_seqs * cfg.page_size))
        if max_len < 2 * cfg.page_size:
            raise ValueError(f"{cfg.name}: no room for a KV cache of {max_seqs} sequences")
    max_len = int(max_len)
    num_pages = max_seqs * ((max_len + cfg.page_size - 1) // cfg.page_size) + 1
    kv = num_pages * page
    total = fixed + kv
    if total > budget:
        fit = ((budget - fixed) // page - 1) // max_seqs * cfg.page_size
        raise ValueError(f"{cfg.name}: {max_seqs} x {max_len} positions of {kv_dtype} KV need {kv / 2**30:.1f} GiB; "
                         f"{(budget - fixed) / 2**30:.1f} GiB are free after the model: at most {fit} positions fit")
    return MemoryPlan(w, kv, st, pf, resident, total, budget, max_len, max_seqs, num_pages)
