"""Control plane and routing of multi-GPU serving, exercised with mock engines on gloo CPU ranks, plus the
host-side arithmetic of the parallel layouts."""
import os
import sys

import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _init(rank, world, port):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)


def _lockstep(rank, world, port, q):
    sys.path.insert(0, ROOT)
    from b200serve.parallel import launch as L
    from b200serve.server.iface import MockEngine
    _init(rank, world, port)
    plane = L.ControlPlane()
    eng = MockEngine(vocab_size=259, max_seqs=2)
    if rank == 0:
        lead = L.LockstepLeader(eng, plane)
        first = lead.prefill(0, [5, 6, 7])
        out = lead.step({0: [first]})
        lead.truncate(0, 3)
        lead.shutdown()
        q.put(("leader", first, out[0], eng.length(0)))
    else:
        n = L.follow_lockstep(eng, plane)
        q.put(("follower", n, eng.length(0), list(eng.seqs[0])))


def _sharded(rank, world, port, q):
    """A tensor-parallel mock: every rank holds its slice of the vocabulary, as the GPU engines do."""
    sys.path.insert(0, ROOT)
    import numpy as np
    from b200serve.parallel import launch as L
    from b200serve.server.iface import MockEngine
    _init(rank, world, port)
    plane = L.ControlPlane()

    class Sharded(MockEngine):
        def logits_shard(self, slot, row=0):
            full = np.asarray(MockEngine.logits(self, slot, row), dtype=np.float32)
            per = (self.vocab_size + world - 1) // world
            return rank * per, full[rank * per: (rank + 1) * per]

        def logits(self, slot, row=0):           # what a shard-holding engine returns by itself: its slice only
            return self.logits_shard(slot, row)[1]

    eng = Sharded(vocab_size=259, max_seqs=2)
    if rank == 0:
        lead = L.LockstepLeader(eng, plane)
        first = lead.prefill(0, [5, 6, 7])
        row = lead.logits(0, 0)
        want = np.asarray(MockEngine.logits(eng, 0, 0), dtype=np.float32)
        lead.shutdown()
        q.put(("leader", len(row), bool(np.array_equal(row, want)), int(row.argmax()), first))
    else:
        n = L.follow_lockstep(eng, plane)
        q.put(("follower", n))


def _lockstep_spec(rank, world, port, q):
    """An engine with a draft head behind the lock-step leader: drafts are made on every rank."""
    sys.path.insert(0, ROOT)
    from b200serve.parallel import launch as L
    from b200serve.server.iface import MockEngine
    _init(rank, world, port)
    plane = L.ControlPlane()

    class Drafting(MockEngine):
        def __init__(self, **kw):
            super().__init__(**kw)
            self.draft_calls = []
            self.stats = {"drafted": 0}

        def draft_many(self, reqs):
            self.draft_calls.append(dict(reqs))
            out = {s: [(r[0] + 1 + j) % self.vocab_size for j in range(r[1])] for s, r in reqs.items()}
            self.stats["drafted"] += sum(len(v) for v in out.values())
            return out

        def draft(self, slot, pending, k, temperature=0.0, seed=0):
            return self.draft_many({slot: (pending, k, temperature, seed)})[slot]

        def draft_q(self, slot):
            return None

    eng = Drafting(vocab_size=259, max_seqs=2)
    if rank == 0:
        lead = L.lockstep_leader(eng, plane)
        assert isinstance(lead, L.LockstepSpecLeader)
        plain = L.lockstep_leader(MockEngine(vocab_size=259, max_seqs=2), plane)
        first = lead.prefill(0, [5, 6, 7])
        d1 = lead.draft(0, first, 3)
        d2 = lead.draft_many({0: (first, 2, 0.5, 9)})
        lead.shutdown()
        q.put(("leader", d1, d2, not hasattr(plain, "draft_many"), lead.stats["drafted"], lead.draft_q(0)))
    else:
        n = L.follow_lockstep(eng, plane)
        q.put(("follower", n, eng.draft_calls, eng.stats["drafted"]))


def _replica(rank, world, port, q):
    sys.path.insert(0, ROOT)
    from b200serve.parallel import launch as L
    from b200serve.server.iface import MockEngine
    _init(rank, world, port)
    plane = L.ControlPlane()
    eng = MockEngine(vocab_size=259, max_seqs=2)
    if rank == 0:
        r = L.ReplicaRouter(eng, plane)
        assert r.max_seqs == 4
        t0 = r.prefill(0, [10, 11])      # rank 0, local slot 0
        t3 = r.prefill(3, [10, 11])      # rank 1, local slot 1
        out = r.step({0: [t0], 3: [t3]})
        lens = (r.length(0), r.length(3))
        lg = r.logits(3, 0)
        eng.fail_slots = set()
        r.shutdown()
        q.put(("router", t0, t3, out, lens, int(lg.argmax()), r.calls))
    else:
        n = L.serve_replica_worker(eng, plane)
        q.put(("worker", n, eng.length(1)))


def _spawn(fn, world=2, port=29701):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=fn, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in ps]
    res = [q.get(timeout=120) for _ in range(world)]
    [p.join(timeout=60) for p in ps]
    assert all(p.exitcode == 0 for p in ps)
    return {r[0]: r for r in res}


def test_lockstep_followers_execute_every_leader_call():
    res = _spawn(_lockstep, port=29701)
    _, first, out, length = res["leader"]
    _, n, flen, fseq = res["follower"]
    assert n == 3 and flen == length == 3          # prefill, step, truncate reached the follower
    assert fseq == [5, 6, 7]


def test_lockstep_leader_with_a_draft_head_drafts_on_every_rank():
    res = _spawn(_lockstep_spec, port=29704)
    _, d1, d2, plain_has_none, drafted, q0 = res["leader"]
    _, n, calls, fdrafted = res["follower"]
    assert len(d1) == 3 and list(d2) == [0] and len(d2[0]) == 2
    assert plain_has_none and q0 is None            # an engine without a head gets the plain leader
    assert n == 3 and len(calls) == 2               # prefill + two draft calls reached the follower
    assert calls[0][0][1] == 3 and calls[1][0][1:] == (2, 0.5, 9)
    assert drafted == fdrafted == 5


def test_lockstep_leader_assembles_full_vocabulary_row_from_shards():
    # a sampled request under tensor parallelism must see vocab_size logits, not rank 0's slice
    res = _spawn(_sharded, port=29703)
    _, n, equal, top, first = res["leader"]
    assert n == 259 and equal and top == first
    assert res["follower"][1] == 2                  # prefill and the shard request reached the follower


def test_native_samplers_refuse_a_short_row():
    import numpy as np
    from b200serve.native import host as H
    row = np.zeros(100, dtype=np.float32)
    for call in (lambda: H.sample(row, 259, 1.0, 0, 1.0, 1), lambda: H.argmax_low_tie(row, 259),
                 lambda: H.apply_repetition_penalty(row, 259, [1, 2], 1.1)):
        with pytest.raises(ValueError):
            call()


def test_replica_router_routes_slots_to_ranks():
    res = _spawn(_replica, port=29702)
    _, t0, t3, out, lens, top, calls = res["router"]
    assert t0 == t3                                   # same prompt, same mock continuation on either rank
    assert set(out) == {0, 3} and out[0] == out[3]
    assert lens == (3, 3) and top == out[3][0]
    assert calls[1] >= 3
    _, n, wlen = res["worker"]
    assert wlen == 3 and n >= 4


def test_split_layers_and_shard_arithmetic():
    from b200serve.models.config import preset
    from b200serve.parallel.launch import parse_parallel
    from b200serve.parallel.pp import split_layers
    parts = split_layers(64, 2)
    assert parts[0][0] == 0 and parts[-1][1] == 64 and parts[0][1] == parts[1][0]
    assert parts[0][1] - parts[0][0] > parts[1][1] - parts[1][0]       # the head counts on the last stage
    assert [b - a for a, b in split_layers(40, 4)] and sum(b - a for a, b in split_layers(40, 4)) == 40
    cfg = preset("dense-27b").tp_shard(8)
    assert (cfg.n_q_heads, cfg.n_kv_heads, cfg.ffn) == (5, 1, 2176) and cfg.hidden == 5120
    with pytest.raises(ValueError):
        preset("dense-27b").tp_shard(16)
    assert parse_parallel("tp4") == ("tp", 4) and parse_parallel("replica") == ("replica", None)
