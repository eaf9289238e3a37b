"""Mixture of experts on the GPU: routing against the oracle's rule, the row path and the grouped
tensor-core prompt path against the fp32 oracle."""
import pytest
import torch

from b200serve.models.config import small_moe, tiny_moe
from b200serve.models.oracle import OracleKV, OracleModel, argmax_low_tie, moe_route
from b200serve.models.weights import random_weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("t,e,k", [(5, 8, 2), (300, 256, 8), (64, 16, 4)])
def test_route_matches_oracle_rule(t, e, k):
    from b200serve.ops import moe as M
    torch.manual_seed(e)
    ld = e + 8
    logits = torch.randn(t, ld)
    logits[0, :e] = 0.0                                   # all equal: ties go to the lowest ids
    logits[1, 3] = logits[1, 1] = 5.0                     # a two-way tie at the top
    idx = torch.zeros(t * k, dtype=torch.int32, device="cuda")
    w = torch.zeros(t * k, dtype=torch.float32, device="cuda")
    M.route(logits.cuda(), ld, t, e, k, idx, w)
    torch.cuda.synchronize()
    ref_idx, ref_w = moe_route(logits[:, :e], k)
    got_idx = idx.cpu().reshape(t, k).long()
    assert got_idx[0].tolist() == list(range(k))
    assert got_idx[1, :2].tolist() == [1, 3]
    # rows whose k-th and (k+1)-th probabilities are not within rounding of each other must agree exactly
    p = torch.softmax(logits[:, :e], -1).sort(descending=True).values
    clear = (p[:, k - 1] - p[:, k]) > 1e-6 if e > k else torch.ones(t, dtype=torch.bool)
    assert torch.equal(got_idx[clear].sort(-1).values, ref_idx[clear].sort(-1).values)
    assert torch.equal(got_idx[clear], ref_idx[clear])
    assert (w.cpu().reshape(t, k)[clear] - ref_w[clear]).abs().max() < 1e-5


def _teacher_forced(oracle, prompt, toks, margin):
    kv = OracleKV(oracle.cfg)
    logits = oracle.forward(prompt, kv, 0)[-1]
    for i, t in enumerate(toks):
        want = int(argmax_low_tie(logits[None])[0])
        if t != want:
            assert float(logits[want] - logits[t]) < margin, (i, t, want)
        logits = oracle.forward(torch.tensor([t]), kv, len(prompt) + i)[0]


def test_tiny_moe_rows_path_matches_oracle():
    from b200serve.ops import lib as K
    from b200serve.runtime.engine import Engine, Row
    cfg = tiny_moe()
    w = random_weights(cfg, seed=1)
    oracle = OracleModel(w)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, cfg.vocab, (70,), generator=g)
    eng = Engine(random_weights(cfg, device="cuda", seed=1), max_seqs=1, max_len=256, nsplit_attn=4)
    eng.forward_rows([Row(0, i, int(t)) for i, t in enumerate(prompt[:40])])
    got = eng.logits(40).float().cpu()
    ref = oracle.forward(prompt[:40])
    K.check_status()
    # a near-tie between the k-th and (k+1)-th expert may flip under bf16 activations and moves that
    # row's logits by a whole expert: most rows must be tight, none may be far off
    err = (got - ref).abs().amax(dim=1) / ref.abs().max()
    assert (err < 0.04).float().mean() >= 0.85 and err.max() < 0.25, err
    toks = eng.generate(prompt.tolist(), 12)
    K.check_status()
    _teacher_forced(oracle, prompt, toks, 0.03)


@pytest.mark.parametrize("backend", ["bf16", "bf16-resident"])
def test_small_moe_prompt_path_matches_oracle(backend):
    from b200serve.ops import lib as K
    from b200serve.runtime.engine import Engine
    cfg = small_moe()
    w = random_weights(cfg, seed=4)
    oracle = OracleModel(w)
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, cfg.vocab, (400,), generator=g)
    eng = Engine(random_weights(cfg, device="cuda", seed=4), max_seqs=1, max_len=1024, prefill_backend=backend,
                 nsplit_attn=4)
    first = eng.prefill(0, prompt.tolist(), chunk=256)
    K.check_status()
    assert eng._prefill is not None
    ref = oracle.forward(prompt)[-1]
    got = eng.logits(1)[0].float().cpu()
    assert (got - ref).abs().max() < 0.04 * ref.abs().max()
    eng.decode_begin([0], [first])
    toks = [first] + [eng.decode_step()[0] for _ in range(5)]
    K.check_status()
    _teacher_forced(oracle, prompt, toks, 0.04)
