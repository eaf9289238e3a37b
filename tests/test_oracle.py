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
