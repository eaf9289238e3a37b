"""Device sampler (ops/csrc/sampler.cu) against the host sampler (native spec.h: filter_probs + draw), whose rule
and random number it mirrors: the same seed gives the same token."""
import numpy as np
import pytest
import torch


def _run(logits, temps, topks, topps, seeds, penalty=None, hist=None):
    from b200serve.ops import lib as K
    m, v = logits.shape
    dev = "cuda"
    lg = torch.from_numpy(logits).to(dev)
    t = torch.tensor(temps, dtype=torch.float32, device=dev)
    k = torch.tensor(topks, dtype=torch.int32, device=dev)
    p = torch.tensor(topps, dtype=torch.float32, device=dev)
    s = torch.tensor([x - (1 << 64) if x >= (1 << 63) else x for x in seeds], dtype=torch.int64, device=dev)
    tok = torch.full((m,), -7, dtype=torch.int32, device=dev)
    st = torch.full((m,), -7, dtype=torch.int32, device=dev)
    kept = torch.zeros(m, dtype=torch.int32, device=dev)
    kw = {}
    if hist is not None:
        cap = max(len(h) for h in hist)
        hh = torch.zeros(m, cap, dtype=torch.int32)
        for i, h in enumerate(hist):
            hh[i, :len(h)] = torch.tensor(h, dtype=torch.int32)
        kw = dict(penalty=torch.tensor(penalty, dtype=torch.float32, device=dev), hist=hh.to(dev),
                  hist_len=torch.tensor([len(h) for h in hist], dtype=torch.int32, device=dev))
    K.sample_rows(lg, m, v, t, k, p, s, tok, st, kept=kept, **kw)
    torch.cuda.synchronize()
    K.check_status()
    return tok.tolist(), st.tolist(), kept.tolist()


@pytest.mark.gpu
@pytest.mark.parametrize("vocab", [1000, 50257, 151936])
def test_sampler_draws_the_host_samplers_token(vocab):
    from b200serve.native import host as H
    rng = np.random.default_rng(vocab)
    m = 24
    logits = (rng.standard_normal((m, vocab)) * 3.0).astype(np.float32)
    logits[3, 17] = logits[3, 900] = logits[3].max() + 1.0         # a tie at the top: the lower id comes first
    temps = [float(rng.choice([0.0, 0.3, 0.7, 1.0, 1.5])) for _ in range(m)]
    topks = [int(rng.choice([0, 1, 5, 40, 64, 1024])) for _ in range(m)]
    topps = [float(rng.choice([1.0, 0.95, 0.9, 0.5, 0.1])) for _ in range(m)]
    seeds = [int(rng.integers(0, 2 ** 63)) * 2 + int(rng.integers(0, 2)) for _ in range(m)]
    temps[3], topks[3] = 0.0, 0
    tok, st, kept = _run(logits, temps, topks, topps, seeds)
    n_dev = 0
    for i in range(m):
        if temps[i] <= 0:
            want = int(H.argmax_low_tie(logits[i], vocab))
            assert st[i] == 0 and tok[i] == want, (i, tok[i], want)
            continue
        ids, probs, mass = H.filter_probs(logits[i], vocab, temps[i], topks[i], topps[i])
        if st[i] == 1:      # left to the host: only when the filtered set is wider than the kernel's candidates
            assert (topks[i] == 0 or topks[i] > 1024) and len(ids) > 1024, (i, topks[i], len(ids))
            continue
        n_dev += 1
        if topps[i] < 1.0:
            assert kept[i] == len(ids), (i, kept[i], len(ids))
        want = int(H.sample(logits[i], vocab, temps[i], topks[i], topps[i], seeds[i]))
        assert tok[i] == want, (i, tok[i], want, temps[i], topks[i], topps[i])
    assert n_dev >= m // 2
    assert tok[3] == 17


@pytest.mark.gpu
def test_sampler_repetition_penalty_and_host_fallbacks():
    from b200serve.native import host as H
    rng = np.random.default_rng(5)
    vocab, m = 4096, 6
    logits = (rng.standard_normal((m, vocab)) * 2.0).astype(np.float32)
    hist = [[int(x) for x in rng.integers(0, vocab, 50)] + [int(np.argmax(logits[i]))] * 3 for i in range(m)]
    pen = [1.3, 1.0, 2.0, 1.1, 1.7, 1.3]
    temps = [0.0, 0.8, 0.8, 1.0, 0.0, 0.6]
    topks = [0, 20, 50, 100, 0, 8]
    topps = [1.0, 0.9, 0.95, 1.0, 1.0, 0.8]
    seeds = [int(x) for x in rng.integers(0, 2 ** 62, m)]
    tok, st, _ = _run(logits, temps, topks, topps, seeds, penalty=pen, hist=hist)
    for i in range(m):
        lg = logits[i].copy()
        H.apply_repetition_penalty(lg, vocab, hist[i], pen[i])
        want = int(H.argmax_low_tie(lg, vocab)) if temps[i] <= 0 else int(H.sample(lg, vocab, temps[i], topks[i], topps[i], seeds[i]))
        assert st[i] == 0 and tok[i] == want, (i, tok[i], want)
    # a flat row with top_p < 1 and no top-k needs more than 1024 candidates; so does top_k = 2000: both go to the host
    flat = np.zeros((2, 8192), dtype=np.float32)
    flat[1] = rng.standard_normal(8192).astype(np.float32)
    tok, st, _ = _run(flat, [1.0, 1.0], [0, 2000], [0.9, 1.0], [1, 2])
    assert st == [1, 1] and tok == [-1, -1]


@pytest.mark.gpu
def test_adapter_sample_matches_host_path():
    import dataclasses
    from b200serve.models.config import preset
    from b200serve.models.weights import random_weights
    from b200serve.native import host as H
    from b200serve.runtime.engine import Engine
    from b200serve.server.adapter import EngineAdapter
    cfg = dataclasses.replace(preset("tiny-dense"), n_layers=2)
    eng = Engine(random_weights(cfg, device="cuda", seed=3), max_seqs=2, max_len=256)
    ad = EngineAdapter(eng)
    ad.prefill(0, list(range(5, 25)))
    lg = np.array(ad.logits(0, 0), dtype=np.float32)
    for seed, (t, k, p) in enumerate([(0.7, 40, 0.9), (1.0, 0, 1.0), (0.0, 0, 1.0), (1.3, 5, 0.5)]):
        got = ad.sample(0, 0, t, k, p, seed + 11)
        want = int(H.argmax_low_tie(lg, cfg.vocab)) if t <= 0 else int(H.sample(lg, cfg.vocab, t, k, p, seed + 11))
        assert got == want, (t, k, p, got, want)
    hist = list(range(5, 25))
    lg2 = lg.copy()
    H.apply_repetition_penalty(lg2, cfg.vocab, hist, 1.5)
    assert ad.sample(0, 0, 0.9, 30, 0.95, 99, 1.5, hist) == int(H.sample(lg2, cfg.vocab, 0.9, 30, 0.95, 99))
    res = ad.step({0: [7, 8, 9]})
    lg3 = np.array(ad.logits(0, 2), dtype=np.float32)
    assert ad.sample(0, 2, 0.5, 10, 1.0, 5) == int(H.sample(lg3, cfg.vocab, 0.5, 10, 1.0, 5))
    assert len(res[0]) == 3
