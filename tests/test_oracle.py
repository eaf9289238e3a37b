"""fp32 oracle self-consistency: incremental decode == full forward, tie rules, routing."""
import torch

from b200serve.models.config import tiny_dense, tiny_moe
from b200serve.models.oracle import OracleModel, OracleKV, argmax_low_tie, moe_route, apply_rope
from b200serve.models.weights import random_weights, interleave16, deinterleave16


def test_argmax_ties_to_lower_id():
    x = torch.tensor([[1.0, 3.0, 3.0, 2.0], [5.0, 5.0, 5.0, 5.0]])
    assert argmax_low_tie(x).tolist() == [1, 0]


def test_moe_route_ties_and_renorm():
    logits = torch.tensor([[0.0, 1.0, 1.0, 1.0, -1.0]])
    idx, w = moe_route(logits, 2)
    assert idx.tolist() == [[1, 2]]
    assert abs(float(w.sum()) - 1.0) < 1e-6


def test_interleave16_roundtrip():
    g, u = torch.randn(32, 8), torch.randn(32, 8)
    f = interleave16(g, u)
    assert torch.equal(f[:16], g[:16]) and torch.equal(f[16:32], u[:16])
    x = torch.randn(3, 64)
    a, b = deinterleave16(x)
    assert torch.equal(a[:, :16], x[:, :16]) and torch.equal(b[:, :16], x[:, 16:32])


def test_rope_preserves_norm_and_is_relative():
    x = torch.randn(4, 2, 64)
    pos = torch.tensor([0, 1, 5, 100])
    y = apply_rope(x, pos, 1e6)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)
    assert torch.allclose(y[0], x[0])


def _consistency(cfg):
    w = random_weights(cfg)
    m = OracleModel(w)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (24,), generator=g)
    toks, logits = m.generate(ids, 6)
    full = m.forward(torch.cat([ids, toks]))
    assert (full[23:29] - logits).abs().max() < 1e-4
    # chunked ingest equals one pass
    kv = OracleKV(cfg)
    a = m.forward(ids[:10], kv, 0)
    b = m.forward(ids[10:], kv, 10)
    assert (torch.cat([a, b]) - full[:24]).abs().max() < 1e-4


def test_dense_incremental_equals_full():
    _consistency(tiny_dense())


def test_moe_incremental_equals_full():
    _consistency(tiny_moe())


def test_sliding_window_layers_and_config_round_trip():
    import dataclasses
    from b200serve.models.config import ModelConfig
    cfg = dataclasses.replace(tiny_dense(), n_layers=4, sliding_window=8, full_attn_every=2)
    assert [cfg.window_of(i) for i in range(4)] == [8, 0, 8, 0]
    assert dataclasses.replace(cfg, full_attn_every=0).window_of(1) == 8
    back = ModelConfig.from_hf_config(cfg.to_hf_config())
    assert back.sliding_window == 8 and back.full_attn_every == 2
    assert ModelConfig.from_hf_config(tiny_dense().to_hf_config()).sliding_window == 0
    _consistency(cfg)       # incremental and chunked passes see the same windows as one pass
    # the window changes the result once the context is longer than it, and not before
    w = random_weights(cfg)
    full = dataclasses.replace(cfg, sliding_window=0)
    w_full = dataclasses.replace(w, cfg=full) if dataclasses.is_dataclass(w) else None
    if w_full is not None:
        g = torch.Generator().manual_seed(1)
        ids = torch.randint(0, cfg.vocab, (20,), generator=g)
        a, b = OracleModel(w).forward(ids), OracleModel(w_full).forward(ids)
        assert (a[:8] - b[:8]).abs().max() < 1e-5
        assert (a[12:] - b[12:]).abs().max() > 1e-4


def test_hybrid_gdn_incremental_equals_full():
    """Gated delta-net layers: token-by-token and chunked passes carry the recurrent state and the convolution
    window, so they equal one pass over the whole sequence."""
    from b200serve.models.config import ModelConfig, preset
    cfg = preset("small-hybrid")
    assert [cfg.is_gdn_layer(i) for i in range(4)] == [True, False, True, False]
    assert cfg.n_gdn_layers == 2 and cfg.gdn_index(2) == 1 and cfg.gdn_proj_dim == 2 * 256 + 2 * 512 + 8
    back = ModelConfig.from_hf_config(cfg.to_hf_config())
    assert (back.gdn_k_heads, back.gdn_v_heads, back.full_attn_every) == (2, 4, 2)
    _consistency(cfg)
