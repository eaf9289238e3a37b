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
