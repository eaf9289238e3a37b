"""The tensor-parallel kernels driven as a group of one rank on one GPU.

With a single rank every "peer" store lands in the GPU's own buffers and every counter is complete
before the kernel that waits on it starts (stream order), so the whole fused prompt pass -- GEMM ->
reduce-scatter push, owner fold + norm + all-gather push, all-gather -> GEMM wait -- and the decode
wires run without a second GPU and must reproduce the plain one-GPU engine.
"""
import pytest
import torch

from b200serve.models.config import preset
from b200serve.models.weights import random_weights

pytestmark = pytest.mark.gpu


def _engine(**kw):
    from b200serve.runtime.engine import Engine
    cfg = preset("small-dense")
    w = random_weights(cfg, device="cuda", seed=3)
    return cfg, Engine(w, max_seqs=1, max_len=1024, use_graphs=False, **kw)


def test_fused_prompt_pass_single_rank_matches_plain():
    from b200serve.ops import lib as K
    from b200serve.parallel.tp_prefill import TpPrefillRunner
    from b200serve.runtime.prefill import PrefillRunner
    cfg, eng = _engine()
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, cfg.vocab, (300,), generator=g).tolist()
    plain = PrefillRunner(eng, max_chunk=512)
    t_ref = plain.run(0, ids)
    ref_logits = eng.model.buf.logits[0].clone()
    eng.reset(0)
    fused = TpPrefillRunner(eng, max_chunk=512)
    t = fused.run(0, ids)
    K.check_status()
    logits = eng.model.buf.logits[0]
    err = float((logits - ref_logits).abs().max())
    assert err < 0.02 * float(ref_logits.abs().max()), err
    assert t == t_ref
    # two chunks, the second one ragged
    eng.reset(0)
    t2 = fused.run(0, ids, chunk=256)
    K.check_status()
    assert float((eng.model.buf.logits[0] - ref_logits).abs().max()) < 0.03 * float(ref_logits.abs().max())
    fused.close()


def test_small_allreduce_and_argmax_wire_single_rank():
    from b200serve.ops import lib as K
    from b200serve.parallel.symm import TpWires
    wires = TpWires(hidden=512, mcap=8)
    x = torch.randn(3, 512, device="cuda")
    out = torch.zeros_like(x)
    for _ in range(3):          # epochs advance, slots alternate
        K.allreduce_rows(x, out, 3, 512, wires.sum, wires.mcap)
    assert torch.equal(out, x)
    ncand = 16
    val = torch.randn(2 * ncand, device="cuda")
    idx = torch.arange(2 * ncand, device="cuda", dtype=torch.int32) % ncand
    ctrl = torch.zeros(K.CTRL_WORDS, dtype=torch.int32, device="cuda")
    K.argmax_finish_tp(val, idx, ncand, 2, 100, ctrl, False, wires.head, wires.mcap)
    K.check_status()
    want = val.view(2, ncand).argmax(dim=1) + 100
    assert ctrl[K.CTRL_OUT_TOKEN: K.CTRL_OUT_TOKEN + 2].tolist() == want.tolist()
    wires.close()


def test_expert_parallel_block_single_rank_matches_plain():
    """Dispatch -> grouped GEMMs -> return -> weighted sum as a group of one rank, against the one-GPU MoE pass."""
    from b200serve.ops import lib as K
    from b200serve.parallel.ep import EpMoe
    from b200serve.runtime.engine import Engine
    from b200serve.runtime.prefill import PrefillRunner
    cfg = preset("small-moe")
    w = random_weights(cfg, device="cuda", seed=4)
    eng = Engine(w, max_seqs=1, max_len=1024, use_graphs=False)
    g = torch.Generator().manual_seed(12)
    ids = torch.randint(0, cfg.vocab, (300,), generator=g).tolist()
    plain = PrefillRunner(eng, max_chunk=512)
    t_ref = plain.run(0, ids)
    ref_logits = eng.model.buf.logits[0].clone()
    for mode in ("fused", "nccl"):
        eng.reset(0)
        runner = PrefillRunner(eng, max_chunk=512)
        runner.ep = EpMoe(cfg, 512, mode=mode)
        t = runner.run(0, ids)
        K.check_status()
        err = float((eng.model.buf.logits[0] - ref_logits).abs().max())
        assert err < 0.02 * float(ref_logits.abs().max()), (mode, err)
        assert t == t_ref
        runner.ep.close()


def test_expert_parallel_decode_rows_single_rank_match_plain():
    """Decode / verify rows through the exchange's row form (dispatch -> gather on the owner -> batched int4 GEMVs ->
    return -> slot-order sum) as a group of one rank, against the plain MoE row path of the same engine weights."""
    from b200serve.ops import lib as K
    from b200serve.parallel.ep import attach_rows
    from b200serve.runtime.engine import Engine
    cfg = preset("small-moe")
    w = random_weights(cfg, device="cuda", seed=4)
    g = torch.Generator().manual_seed(12)
    ids = torch.randint(0, cfg.vocab, (70,), generator=g).tolist()
    from b200serve.runtime.engine import Row
    plain = Engine(w, max_seqs=1, max_len=256, use_graphs=False, prefill_backend="rows")
    eng = Engine(w, max_seqs=1, max_len=256, use_graphs=False, prefill_backend="rows")
    ep = attach_rows(eng, eng.max_rows)      # the prompt goes through row steps of up to max_rows positions as well
    tok, tok2 = plain.prefill(0, ids), eng.prefill(0, ids)
    scale = float(plain.model.buf.logits[plain.last_prefill_row].abs().max())
    err = float((eng.model.buf.logits[eng.last_prefill_row] - plain.model.buf.logits[plain.last_prefill_row]).abs().max())
    agree = int(tok == tok2)
    for _ in range(7):     # teacher-forced: each step's logits are comparable
        r = plain.forward_rows([Row(0, plain.seq_len[0], tok)])[0]
        g2 = eng.forward_rows([Row(0, eng.seq_len[0], tok)])[0]
        err = max(err, float((eng.model.buf.logits[0] - plain.model.buf.logits[0]).abs().max()))
        agree += int(r == g2)
        tok = r
    K.check_status()
    assert err < 0.02 * scale, err        # the returned rows are bf16 where the plain path folds fp32 slices
    assert agree >= 7, agree
    ep.close()
