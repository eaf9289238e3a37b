"""Draft heads on the GPU: the MTP head against the fp32 oracle, and lossless verify-accept loops."""
import pytest
import torch

from b200serve.models.config import preset
from b200serve.models.weights import random_weights

pytestmark = pytest.mark.gpu


def _mtp_cfg():
    import dataclasses
    return dataclasses.replace(preset("small-dense"), mtp_layers=1, name="small-dense-mtp")


def test_mtp_head_rows_match_oracle():
    from b200serve.models.oracle import OracleKV, OracleModel
    from b200serve.runtime.engine import Engine
    from b200serve.runtime.spec import SpecAdapter
    from b200serve.server.adapter import EngineAdapter
    cfg = _mtp_cfg()
    w = random_weights(cfg, device="cuda", seed=2)
    eng = Engine(w, max_seqs=1, max_len=256, use_graphs=False, extra_kv_layers=1)
    ad = SpecAdapter(EngineAdapter(eng), "mtp", 3)
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, cfg.vocab, (24,), generator=g)
    first = ad.prefill(0, prompt.tolist())
    drafts = ad.draft(0, first, 3)
    assert len(drafts) == 3
    # oracle: trunk hidden states of the prompt, MTP over the shifted pairs, then the chain
    wc = random_weights(cfg, device="cpu", seed=2)
    om = OracleModel(wc)
    kv = OracleKV(cfg)
    hidden = om.forward(prompt, kv, 0, return_hidden=True)[1]
    mkv = OracleKV(cfg)
    # the head's entry of position p pairs (h_{p-1}, x_p); position 0 pairs a zero state with x_0
    hid = torch.cat([torch.zeros(1, cfg.hidden), hidden])
    nxt = torch.cat([prompt, torch.tensor([first])])
    logits, h = om.mtp_forward(hid, nxt, mkv, 0)
    want = int(torch.argmax(logits[-1]))
    top2 = torch.topk(logits[-1], 2).values
    if float(top2[0] - top2[1]) > 0.05:          # only a clear arg-max is compared
        assert drafts[0] == want


@pytest.mark.parametrize("kind,dv", [("mtp", 0), ("dflash", 0), ("mtp", 512), ("mtp-hybrid", 0), ("dflash", 512),
                                     ("dflash-int8", 512)])
def test_speculative_loop_is_lossless(kind, dv):
    """Greedy output with drafts + verify + accept equals plain greedy decoding, token for token.  The hybrid
    variant has gated delta-net layers: rejected rows rewind the recurrent state through the engine's copy from
    before the verify step and a replay of the kept rows."""
    from b200serve.native import host as H
    from b200serve.runtime.engine import Engine
    from b200serve.runtime.spec import SpecAdapter
    from b200serve.server.adapter import EngineAdapter
    cfg = _mtp_cfg()
    int8_cand = kind == "dflash-int8"      # candidates from an int8 copy of the reduced head, re-scored exactly
    kind = "dflash" if int8_cand else kind
    if kind == "mtp-hybrid":
        import dataclasses
        from b200serve.models.config import preset
        cfg, kind = dataclasses.replace(preset("small-hybrid"), mtp_layers=1), "mtp"
    w = random_weights(cfg, device="cuda", seed=5)
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, cfg.vocab, (100,), generator=g).tolist()
    plain = Engine(w, max_seqs=1, max_len=512, use_graphs=False)
    # the speculating engine cuts a row's keys into fixed spans, so that a row's bits do not depend on its company in
    # the step; the plain engine has to sum in the same order for a token-for-token comparison through near-ties
    plain.model.attn_fixed_spans = True
    want = plain.generate(prompt, 24)
    eng = Engine(w, max_seqs=1, max_len=512, use_graphs=False, extra_kv_layers=2)
    ad = SpecAdapter(EngineAdapter(eng), kind, 3, draft_vocab=dv,      # dv: drafts from a reduced vocabulary
                     candidate_head_int8=int8_cand)
    pending = ad.prefill(0, prompt)
    got = [pending]
    iters = 0
    while len(got) < 24:
        drafts = ad.draft(0, pending, 3)
        out = ad.step({0: [pending] + drafts})[0]
        acc, nxt = H.accept_greedy(out, drafts)
        if acc < len(drafts):
            ad.truncate(0, ad.length(0) - (len(drafts) - acc))
        got += drafts[:acc] + [nxt]
        pending = nxt
        iters += 1
    assert got[:24] == want[:24]
    assert ad.stats["drafted"] >= iters


def test_block_drafter_batches_slots_and_samples_from_its_candidates():
    """The block drafter serves two slots in one pass with the same drafts as slot by slot; at a temperature each
    draft is a keyed draw from the row's 16 candidates (same seed, same drafts), the candidates come back as the q of
    the sparse accept rule, and the served loop with that rule runs."""
    import numpy as np
    from b200serve.native import host as H
    from b200serve.runtime.engine import Engine
    from b200serve.runtime.spec import SpecAdapter
    from b200serve.server.adapter import EngineAdapter
    cfg = _mtp_cfg()
    w = random_weights(cfg, device="cuda", seed=5)
    g = torch.Generator().manual_seed(10)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (60, 85)]
    eng = Engine(w, max_seqs=2, max_len=512, use_graphs=False, extra_kv_layers=2)
    ad = SpecAdapter(EngineAdapter(eng), "dflash", 4)
    pend = {s: ad.prefill(s, prompts[s]) for s in (0, 1)}
    one = {s: ad.draft(s, pend[s], 4) for s in (0, 1)}
    both = ad.draft_many({s: (pend[s], 4) for s in (0, 1)})
    assert both == one and all(len(v) == 4 for v in both.values())
    # sampled drafts
    a = ad.draft_many({0: (pend[0], 4, 0.9, 77), 1: (pend[1], 4, 0.0, 0)})
    q0 = ad.draft_q(0)
    b = ad.draft_many({0: (pend[0], 4, 0.9, 77), 1: (pend[1], 4, 0.0, 0)})
    assert a == b and a[1] == one[1]
    assert ad.draft_q(1) is None and q0 is not None
    cand, score = q0
    assert cand.shape == (4, 16) and score.shape == (4, 16)
    for i, t in enumerate(a[0]):
        assert t in cand[i].tolist()
        assert np.all(np.diff(score[i][np.isfinite(score[i])]) <= 0)        # best first
    assert cand[0].tolist()[0] == one[0][0]                                # the greedy draft is the best candidate
    # the verify step and the sparse rule
    out = ad.step({0: [pend[0]] + a[0], 1: [pend[1]] + a[1]})
    p_rows = np.stack([ad.logits(0, i) for i in range(5)])
    acc, nxt = H.accept_sparse(p_rows, cand, score, a[0], cfg.vocab, 0.9, 0, 1.0, 123)
    assert 0 <= acc <= 4 and 0 <= nxt < cfg.vocab
    assert len(out[1]) == 5
