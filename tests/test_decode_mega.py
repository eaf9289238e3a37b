"""The whole-step decode kernel (one cooperative launch for embedding + all dense layers) against the fp32 CPU
oracle and against the launch-per-kernel path of the same engine: phase by phase (the kernel can stop after any
phase), for 1, 4 and 8 rows, through CUDA graphs, and replayed twice for bitwise equality.

The schedule arithmetic (which CTA streams which ring stages) is checked on the CPU for the benchmark shapes.
"""
import pytest
import torch

from b200serve.models.config import small_dense, dense_27b
from b200serve.ops import lib as K


def test_schedule_covers_every_stage_once():
    # pure host arithmetic inside the library: every ring stage of every linear belongs to exactly one CTA's run
    for n_cta in (148, 132, 8):
        for m in (1, 3, 8):
            for cfg in (small_dense(), dense_27b()):
                if cfg.n_kv_heads > n_cta:
                    continue
                plan = K.decode_mega_plan(n_cta, m, cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads, cfg.ffn)
                assert plan is not None and plan["rows"] >= m and plan["stages"] >= 4
                assert plan["nsplit"] * cfg.n_kv_heads <= n_cta
    assert K.decode_mega_plan(148, 9, 512, 8, 2, 1408) is None         # more rows than the kernel serves
    assert K.decode_mega_plan(148, 1, 500, 8, 2, 1408) is None         # hidden size not a multiple of 128


def _setup(m_rows, prompt_len=200, graphs=False):
    from test_engine_tiny import _to_cuda
    from b200serve.models.oracle import OracleModel, OracleKV
    from b200serve.models.weights import random_weights
    from b200serve.runtime.engine import Engine, Row
    cfg = small_dense()
    w = random_weights(cfg, seed=0)
    wc = _to_cuda(w)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (prompt_len,), generator=g)
    mega = Engine(wc, max_seqs=1, max_len=1024, use_graphs=graphs)
    plain = Engine(wc, max_seqs=1, max_len=1024, use_graphs=graphs)
    mega.model.use_mega = True       # off by default
    plain.model.use_mega = False
    return cfg, w, wc, prompt, mega, plain, g


@pytest.mark.gpu
@pytest.mark.parametrize("m_rows", [1, 4, 8])
def test_hidden_states_match_the_oracle_after_every_layer(m_rows):
    from b200serve.models.oracle import OracleModel, OracleKV, rmsnorm
    from b200serve.runtime.engine import Row
    cfg, w, wc, prompt, mega, plain, g = _setup(m_rows)
    oracle = OracleModel(w)
    P = len(prompt)
    first = mega.prefill(0, prompt.tolist())
    toks = [first] + torch.randint(0, cfg.vocab, (m_rows - 1,), generator=g).tolist()
    rows = [Row(0, P + i, t) for i, t in enumerate(toks)]
    kv = OracleKV(cfg)
    oracle.forward(prompt, kv, 0)
    h = w.embed.float()[torch.tensor(toks)]
    pos = torch.arange(P, P + m_rows)
    refs = [h.clone()]
    for li, lw in enumerate(w.layers):
        h = h + oracle.attention(lw, rmsnorm(h, lw.input_norm, cfg.rms_eps), pos, kv, li)
        refs.append(h.clone())
        h = h + oracle.swiglu(lw.gate_up, lw.down, rmsnorm(h, lw.post_norm, cfg.rms_eps))
        refs.append(h.clone())
    plan = mega.model.mega_plan(wc.layers, m_rows, mega.kv)
    assert plan is not None
    for r in rows:
        mega._ensure_pages(r.slot, r.pos + 1)
    mega._write_rows(rows)
    # phases: 0 embedding; per layer qkv, attention, o (residual folded), gate||up, down (residual folded)
    cuts = [(1, 0)] + [(1 + 5 * li + 3, 1 + 2 * li) for li in range(cfg.n_layers)] + \
           [(1 + 5 * li + 5, 2 + 2 * li) for li in range(cfg.n_layers)]
    for n_phases, ref_i in sorted(cuts):
        mega.model.mega_layers(wc.layers, m_rows, mega.ctrl, mega.block_table, mega.max_blocks, mega.kv, plan, 0,
                               n_phases=n_phases)
        torch.cuda.synchronize()
        K.check_status()
        got = mega.model.buf.resid[:m_rows].float().cpu()
        ref = refs[ref_i]
        # the stream is bf16: half an ulp of the largest value per fold, and the activations' own rounding
        tol = 0.02 * float(ref.abs().max())
        assert float((got - ref).abs().max()) < tol, (n_phases, float((got - ref).abs().max()), tol)
        cos = torch.nn.functional.cosine_similarity(got, ref, dim=1)
        assert float(cos.min()) > 0.999, (n_phases, cos)


@pytest.mark.gpu
@pytest.mark.parametrize("m_rows", [1, 4, 8])
def test_step_matches_the_launch_per_kernel_path(m_rows):
    from b200serve.runtime.engine import Row
    cfg, w, wc, prompt, mega, plain, g = _setup(m_rows)
    P = len(prompt)
    fa, fb = mega.prefill(0, prompt.tolist()), plain.prefill(0, prompt.tolist())
    assert fa == fb
    toks = [fa] + torch.randint(0, cfg.vocab, (m_rows - 1,), generator=g).tolist()
    rows = [Row(0, P + i, t) for i, t in enumerate(toks)]
    oa, ob = mega.forward_rows(rows), plain.forward_rows(rows)
    K.check_status()
    la, lb = mega.logits(m_rows).float(), plain.logits(m_rows).float()
    scale = float(lb.abs().max())
    assert float((la - lb).abs().max()) < 0.03 * scale
    for i in range(m_rows):     # the arg-max may differ only where the two paths' top logits are within their noise
        if oa[i] != ob[i]:
            assert float(lb[i, ob[i]] - lb[i, oa[i]]) < 0.03 * scale
    # every kernel of the step is ours: 1 whole-step launch + final norm + head + arg-max
    assert mega.model.mega_plan(wc.layers, m_rows, mega.kv) is not None


@pytest.mark.gpu
def test_graph_decode_loop_and_replay_twice_bitwise():
    from b200serve.models.oracle import OracleModel, OracleKV, argmax_low_tie
    cfg, w, wc, prompt, mega, plain, g = _setup(1, graphs=True)
    oracle = OracleModel(w)
    toks = mega.generate(prompt.tolist(), 24)
    K.check_status()
    assert mega.launches(1, True) <= 4                      # whole-step kernel, final norm, head, arg-max
    # the oracle, teacher-forced with the engine's tokens: a different token only on a near-tie
    kv = OracleKV(cfg)
    logits = oracle.forward(prompt, kv, 0)[-1]
    for i, t in enumerate(toks):
        want = int(argmax_low_tie(logits[None])[0])
        if t != want:
            assert float(logits[want] - logits[t]) < 0.05, (i, t, want)
        logits = oracle.forward(torch.tensor([t]), kv, len(prompt) + i)[0]
    # replay twice from the same state: the same bits (fixed summation order everywhere, no atomics on data)
    again = mega.generate(prompt.tolist(), 24)
    assert again == toks
    r1 = mega.model.buf.resid[:1].clone()
    l1 = mega.logits(1).clone()
    mega.generate(prompt.tolist(), 24)
    assert torch.equal(r1, mega.model.buf.resid[:1]) and torch.equal(l1, mega.logits(1))
