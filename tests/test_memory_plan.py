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


def test_vram_probe_with_fake_nvml():
    """The memory / BAR1 / NVLink probe over a fake NVML: two NVLink-connected GPUs and one behind PCIe."""
    from types import SimpleNamespace as NS
    from b200serve.utils import vram

    class FakeNvml:
        NVML_P2P_CAPS_INDEX_NVLINK = 2
        NVML_P2P_STATUS_OK = 0
        calls = []

        def nvmlDeviceGetCount(self): return 3
        def nvmlDeviceGetHandleByIndex(self, i): return i
        def nvmlDeviceGetName(self, h): return b"NVIDIA B200"
        def nvmlDeviceGetMemoryInfo(self, h): return NS(total=180 << 30, free=(170 - 60 * h) << 30, used=0)

        def nvmlDeviceGetBAR1MemoryInfo(self, h):
            if h == 2:
                raise RuntimeError("not supported")
            return NS(bar1Total=(256 << 30) if h == 0 else (64 << 30), bar1Free=1 << 30)

        def nvmlDeviceGetNvLinkState(self, h, link):
            if link >= 18:
                raise RuntimeError("invalid link")
            return 1 if h < 2 else 0

        def nvmlDeviceGetP2PStatus(self, a, b, idx):
            assert idx == self.NVML_P2P_CAPS_INDEX_NVLINK
            return 0 if (a < 2 and b < 2) else 5

        def __getattr__(self, name):        # anything that would change a setting is a test failure
            raise AssertionError(f"unexpected NVML call {name}")

    g = vram.probe(FakeNvml())
    assert [x.index for x in g] == [0, 1, 2]
    assert g[0].bar1_covers_memory and not g[1].bar1_covers_memory and g[2].bar1_total == 0
    assert g[0].nvlinks_up == 18 and g[2].nvlinks_up == 0
    assert g[0].peers_nvlink == {1: True, 2: False}
    lines = vram.describe(g)
    assert "NVLink peers [1]" in lines[0] and "NOT over NVLink [2]" in lines[0] and "covers the memory" in lines[0]
    assert vram.check_placement(g[:2], need_bytes=100 << 30, need_nvlink=False) == []
    two = vram.probe(FakeNvml(), indices=[0, 1])
    assert vram.check_placement(two, need_nvlink=True) == []
    bad = vram.check_placement(g, need_bytes=100 << 30, need_nvlink=True)
    assert any("GPU 2" in b and "GiB free" in b for b in bad) and any("not connected by NVLink" in b for b in bad)


def test_plan_counts_the_recurrent_state_of_hybrid_models():
    from b200serve.models.config import preset
    from b200serve.runtime import memory_plan as MP
    dense, hyb = preset("dense-27b"), preset("hybrid-27b")
    per_slot = MP.gdn_state_bytes_per_slot(hyb)
    assert MP.gdn_state_bytes_per_slot(dense) == 0
    assert per_slot == 2 * 48 * (48 * 128 * 128 * 4 + (2 * 16 * 128 + 48 * 128) * 3 * 4)
    # only the 16 attention layers hold KV pages
    assert MP.kv_bytes_per_page(hyb, "bf16") * 4 == MP.kv_bytes_per_page(dense, "bf16")
    a, b = MP.plan(hyb, 1, 4096), MP.plan(hyb, 8, 4096)
    assert b.total - a.total >= 7 * per_slot
    assert MP.weight_bytes(hyb) > MP.weight_bytes(dense)


def test_attention_split_rule_and_quantiser_slots():
    from b200serve.models.decoder import attn_splits
    from b200serve.ops.lib import quant_slots
    assert attn_splits(8, 4096) == 37            # 8 KV heads x 37 splits = one wave of 2 x 148 CTAs
    assert attn_splits(8, 1024) == 16            # never fewer than 64 keys per split
    assert attn_splits(8, 100) == 4
    assert attn_splits(1, 32768) == 64           # the partial buffers hold at most 64 splits
    assert attn_splits(4, 262144) == 64
    assert [quant_slots(m) for m in (1, 8, 9, 16, 17, 33, 64)] == [8, 8, 16, 16, 32, 64, 64]


def test_quant_x_refuses_buffers_that_are_too_small():
    """The binding checks the sizes before the kernel runs: 3 rows still need 8 token slots per 64-k group."""
    import pytest
    import torch
    from b200serve.ops import lib as K
    m, k = 3, 1024
    x = torch.zeros(m, k, dtype=torch.bfloat16)
    xq = torch.zeros(m * (k // 64) * 128, dtype=torch.uint8)
    with pytest.raises(ValueError):
        K.quant_x(x, m, k, xq, torch.zeros(m * (k // 64) * 2, dtype=torch.int32))
    with pytest.raises(ValueError):
        K.quant_x(x, m, k, xq[:-1], torch.zeros(8 * (k // 64) * 2, dtype=torch.int32))
    with pytest.raises(ValueError):
        K.quant_x(torch.zeros(65, k, dtype=torch.bfloat16), 65, k, torch.zeros(65 * (k // 64) * 128, dtype=torch.uint8),
                  torch.zeros(64 * (k // 64) * 2, dtype=torch.int32))


@pytest.mark.parametrize("name", ["tiny-dense", "small-dense", "small-moe", "small-hybrid", "dense-27b"])
def test_every_step_buffer_is_known_to_the_planner(name):
    """The allocator and the planner agree: every tensor of StepBuffers / KVCache has a registry entry, and each
    group holds no more than the planner budgets (the reference enforces this at compile time)."""
    import torch
    from b200serve.models.config import preset
    from b200serve.models.decoder import KVCache, StepBuffers, attn_splits
    from b200serve.ops import lib as K
    from b200serve.runtime import buffer_registry as R
    cfg = preset(name)
    rows = 8 if name == "dense-27b" else 64
    buf = StepBuffers(cfg, rows, attn_splits(cfg.n_kv_heads, 4096), "cpu")
    for lin in cfg.linears():                   # the split-K partial sums a step allocates on first use
        buf.part(lin.name, K.gemv_splits(lin.n, lin.k), lin.n)
    kv = KVCache(cfg, cfg.n_layers, 9, "cpu", "bf16", n_slots=2)
    groups = R.audit(buf, kv, cfg, "bf16", max_seqs=2)
    assert groups["step"] > 0 and groups["kv"] > 0
    buf.surprise = torch.zeros(4)               # a buffer nobody told the planner about
    with pytest.raises(AssertionError, match="surprise"):
        R.audit(buf, kv, cfg, "bf16", max_seqs=2)
