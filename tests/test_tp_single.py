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


def test_reduce_scatter_fold_error_with_eight_sources():
    """The owner's fold adds bf16 partial tiles from every source rank to the residual row in fp32 and rounds once.
    One rank, eight landing slots filled by hand: the result against the fp32 sum of the UNROUNDED partials stays
    inside the rounding of the eight bf16 partials plus the final rounding, and equals the fp32 sum of the rounded
    partials to the last bit (fixed source order)."""
    from b200serve.ops import lib as K
    from b200serve.parallel.symm import Wire
    torch.manual_seed(21)
    nsrc, h, tpr, c = 8, 1024, 1, 100
    rows_cap = tpr * 128
    rs = Wire(nsrc * rows_cap * h * 2, nsrc * tpr, 0, None, torch.device("cuda"))
    xw = Wire(rows_cap * h * 2, tpr, 0, None, torch.device("cuda"))
    part32 = torch.randn(nsrc, rows_cap, h, device="cuda") * 0.7          # what the GEMMs would hold in fp32
    part16 = part32.to(torch.bfloat16)
    rs.buf.view(torch.bfloat16, 0, nsrc * rows_cap * h).copy_(part16.view(-1))
    rs.flags.fill_(5)                                                       # every tile of every source has arrived
    resid0 = (torch.randn(rows_cap, h, device="cuda") * 2.0).to(torch.bfloat16)
    resid = resid0.clone()
    norm_w = torch.ones(h, device="cuda")
    done = torch.zeros(tpr, dtype=torch.int32, device="cuda")
    K.rs_fold(rs, 5, nsrc, done, resid, norm_w, 1e-6, xw, h, tpr, c)
    torch.cuda.synchronize()
    K.check_status()
    exact_rounded = resid0[:c].float()
    for s_ in range(nsrc):                                                  # the kernel's order: residual, then sources 0..7
        exact_rounded = exact_rounded + part16[s_, :c].float()
    assert torch.equal(resid[:c], exact_rounded.to(torch.bfloat16))
    true = resid0[:c].float() + part32[:, :c].sum(0)
    err = (resid[:c].float() - true).abs()
    # bf16 keeps 8 significant bits: unit roundoff 2^-8 for each partial and for the stored result
    bound = part32[:, :c].abs().sum(0) * 2.0 ** -8 + (true.abs() + 0.1) * 2.0 ** -8 + 1e-6
    assert (err <= bound).all()
    rel = float(err.max() / true.abs().max())
    assert rel < 4e-3, rel          # bf16 transport of 8 partials costs a few 1e-3 of the row's scale
    rs.close()
    xw.close()
