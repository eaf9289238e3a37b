"""Memory planner arithmetic (CPU)."""
import pytest

from b200serve.models.config import dense_27b, moe_35b_a3b, tiny_dense
from b200serve.runtime.memory_plan import kv_bytes_per_page, plan, weight_bytes


def test_27b_numbers():
    cfg = dense_27b()
    w = weight_bytes(cfg)
    assert 13.5e9 < w < 15.5e9                       # int4 + scales + bf16 embed and head
    assert kv_bytes_per_page(cfg, "bf16") == 64 * 2 * 8 * 128 * 2 * 16
    assert kv_bytes_per_page(cfg, "int8") < kv_bytes_per_page(cfg, "bf16") * 0.53
    p = plan(cfg, 8, 32768 + 256, kv_dtype="int8")
    assert p.max_len == 33024 and p.total < p.budget and "kv" in p.line()
    auto = plan(cfg, 1, "auto")
    assert auto.max_len == 262144                    # one sequence: capped by the context limit, not by memory
    auto8 = plan(cfg, 64, "auto")
    assert auto8.max_len % 16 == 0 and auto8.max_len * 64 * 256 * 1024 < auto8.budget
    with pytest.raises(ValueError, match="at most"):
        plan(cfg, 64, 262144)
    with pytest.raises(ValueError, match="before any KV"):
        plan(cfg, 1, 1024, budget=8 * 2 ** 30)


def test_tp_and_moe_shrink_per_gpu_bytes():
    cfg = dense_27b()
    assert weight_bytes(cfg, tp=8) < weight_bytes(cfg) * 0.3
    moe = moe_35b_a3b()
    assert weight_bytes(moe, ep=8) < weight_bytes(moe) * 0.25
    assert plan(moe, 16, 131072 + 64, kv_dtype="int8").total < plan(moe, 16, 131072 + 64, kv_dtype="int8").budget
    with pytest.raises(ValueError):
        plan(moe, 16, 131072 + 64)      # the same in bf16 does not fit one GPU
    assert plan(tiny_dense(), 2, 512).num_pages == 2 * 32 + 1
