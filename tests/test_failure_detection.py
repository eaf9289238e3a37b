"""Failure detection without faulting a GPU: the wire's host mirror under injected losses (CPU threads), and a
device wait that runs out because nothing sets its flag (GPU, bounded, context stays usable)."""
import numpy as np
import pytest

from b200serve.parallel.protocol import STALE, TIMEOUT, HostWire, run_ranks


def _parts(rank, i):
    rng = np.random.default_rng(1000 * rank + i)
    return rng.standard_normal(64).astype(np.float32)


def test_host_mirror_all_ranks_hold_identical_bits():
    w = HostWire(4, 64)
    out = run_ranks(w, 6, _parts)
    for i in range(6):
        want = np.zeros(64, dtype=np.float32)
        for r in range(4):
            want = want + _parts(r, i)
        for r in range(4):
            assert out[r][i] is not None and np.array_equal(out[r][i], out[0][i])
            assert np.array_equal(out[r][i], want)
    assert all(s is None for s in w.status)


def test_dropped_flag_times_out_once_and_latches():
    w = HostWire(2, 64, bound_s=0.2)
    w.drop_next(writer=1, reader=0)            # rank 0 never sees rank 1's first flag
    out = run_ranks(w, 3, _parts)
    assert out[0][0] is None and w.status[0] == (TIMEOUT, 1, 1)
    assert w.bounds_paid[0] == 1               # later waits do not spin again: one bound per dead peer
    assert out[1][0] is not None               # the other direction was delivered
    w.reset(0)
    assert w.status[0] is None


def test_flag_before_data_is_reported_as_stale():
    w = HostWire(2, 64, bound_s=0.2)
    w.skip_data(writer=0, reader=1)
    out = run_ranks(w, 1, _parts)
    assert out[1][0] is None and w.status[1][0] == STALE


def test_rank_that_leaves_between_calls_costs_one_bound():
    w = HostWire(3, 64, bound_s=0.2)
    first = run_ranks(w, 1, _parts)
    assert all(o[0] is not None for o in first)
    w.kill(2)                                   # leaves between steps, nothing in flight
    out = run_ranks(w, 2, _parts)
    assert out[0][0] is None and out[1][0] is None
    assert w.status[0][0] == TIMEOUT and w.status[0][1] == 2
    assert w.bounds_paid[0] == 1 and w.bounds_paid[1] == 1


@pytest.mark.gpu
def test_device_wait_runs_out_and_reports_status():
    """A counter that nothing increments: the kernel gives up after its bound, the status word names the wait,
    the context stays usable and the status can be cleared."""
    import time
    import torch
    from b200serve.ops import lib as K
    K.status_clear()
    cnt = torch.zeros(4, dtype=torch.int32, device="cuda")
    t0 = time.time()
    K.wire_wait(cnt, 1)
    torch.cuda.synchronize()
    dt = time.time() - t0
    st = K.status()
    assert "comm" in st and st["comm"]["code"] == hex(0x501)
    assert 0.2 < dt < 10.0
    with pytest.raises(K.KernelError):
        K.check_status()
    K.status_clear()
    assert K.status() == {}
    x = torch.ones(8, device="cuda")           # the context is still usable
    assert float(x.sum()) == 8.0
    cnt.fill_(1)
    K.wire_wait(cnt, 1)                          # a satisfied wait returns at once
    torch.cuda.synchronize()
    assert K.status() == {}


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_plan_is_consistent_across_ranks(world):
    """Every rank derives the layout from the same counts: rows of different sources never overlap in a
    destination's buffer, every expert's rows are contiguous, and the owner's block table covers exactly them."""
    from b200serve.parallel.protocol import ep_plan_mirror
    rng = np.random.default_rng(world)
    e_total, el = 32, 32 // world
    cnt = rng.integers(0, 300, size=(world, e_total)).tolist()
    for s in range(world):
        cnt[s][rng.integers(0, e_total)] = 0          # some experts get nothing from some sources
    plans = [ep_plan_mirror(cnt, r, world) for r in range(world)]
    for dest in range(world):
        _, blocks, total_rows = plans[dest]
        taken = np.zeros(total_rows, dtype=np.int32)
        owner_of = np.full(total_rows, -1, dtype=np.int32)
        for src in range(world):
            base = plans[src][0]
            for e in range(dest * el, (dest + 1) * el):
                lo, n = base[e], cnt[src][e]
                assert lo + n <= total_rows
                taken[lo: lo + n] += 1
                owner_of[lo: lo + n] = e - dest * el
        assert taken.max() <= 1                        # no two (source, expert) ranges overlap
        covered = np.zeros(total_rows, dtype=bool)
        for el_id, row0, rows in blocks:
            assert row0 % 128 == 0 and 0 < rows <= 128
            assert (taken[row0: row0 + rows] == 1).all() and (owner_of[row0: row0 + rows] == el_id).all()
            assert (taken[row0 + rows: row0 + 128] == 0).all()      # padding rows belong to nobody
            covered[row0: row0 + rows] = True
        assert (covered == (taken == 1)).all()         # the blocks cover exactly the rows that arrive


@pytest.mark.gpu
def test_engine_latches_on_a_wait_that_ran_out_and_recovers_bitwise():
    """The serving path reads the failure word after every step: a bounded wait that ran out while a step was in
    flight (here: a stream-ordered wait on a counter nothing increments) raises an error that names the unit and the
    code, the engine refuses further steps until reset_failure(), and after it the same step gives the same bits."""
    import torch
    from b200serve.models.config import small_dense
    from b200serve.models.weights import random_weights
    from b200serve.ops import lib as K
    from b200serve.runtime.engine import Engine, Row
    K.status_clear()
    cfg = small_dense()
    eng = Engine(random_weights(cfg, device="cuda", seed=0), max_seqs=1, max_len=256, use_graphs=False)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    first = eng.prefill(0, prompt)
    want = eng.forward_rows([Row(0, 40, first)])
    want_logits = eng.logits(1).clone()
    eng.truncate(0, 40)
    cnt = torch.zeros(4, dtype=torch.int32, device="cuda")
    K.wire_wait(cnt, 1)                       # gives up after its bound and records 0x501 in the comm unit
    with pytest.raises(K.KernelError, match="comm: code 0x501"):
        eng.forward_rows([Row(0, 40, first)])
    assert eng.broken is not None
    with pytest.raises(K.KernelError, match="latched"):
        eng.forward_rows([Row(0, 40, first)])
    eng.reset_failure()
    assert eng.broken is None and K.status() == {}
    eng.truncate(0, 40)
    got = eng.forward_rows([Row(0, 40, first)])
    assert got == want and torch.equal(eng.logits(1), want_logits)
