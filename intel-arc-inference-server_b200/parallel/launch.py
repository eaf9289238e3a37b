"""Multi-GPU serving: process launch and the control plane between the HTTP process and the ranks.

``--parallel replica``  every GPU holds the whole model; rank 0 runs the HTTP server and routes each
                        request's slot to a rank (prefix affinity first, then the rank with most free slots);
                        the other ranks run a worker loop.  The reference's replica mode does this with one
                        thread per card inside one process (src/cli/replica_engine.h:1-40).
``--parallel tpN / ppN / epN``  one model over N GPUs: every engine call of the leader is first broadcast to
                        the followers, then every rank executes it -- the ranks meet inside the kernels
                        (fused wires) or in NCCL calls (pipeline hand-off).

The control plane is a gloo group (host objects only), separate from the NCCL group the engines use, so a
command never queues behind GPU work.  Everything here runs with mock engines on CPU ranks (tests).
"""
from __future__ import annotations

import os
import sys
from typing import Dict, List, Optional, Sequence

import numpy as np

from ..server.iface import EngineIface

SHUTDOWN = "__shutdown__"


class ControlPlane:
    """Commands from the leader (rank 0 of ``group``) to follower ranks over gloo."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    # leader side ---------------------------------------------------------
    def broadcast(self, msg):
        box = [msg]
        self.dist.broadcast_object_list(box, src=self._global(0), group=self.group)

    def send(self, rank: int, msg):
        self.dist.send_object_list([msg], dst=self._global(rank), group=self.group)

    def recv(self, rank: int):
        box = [None]
        self.dist.recv_object_list(box, src=self._global(rank), group=self.group)
        return box[0]

    # follower side -------------------------------------------------------
    def next_broadcast(self):
        box = [None]
        self.dist.broadcast_object_list(box, src=self._global(0), group=self.group)
        return box[0]

    def _global(self, r: int) -> int:
        return self.dist.get_global_rank(self.group, r) if self.group is not None else r


def _apply(engine: EngineIface, msg):
    name, args = msg
    return getattr(engine, name)(*args)


# ---------------------------------------------------------------------- one model over all ranks
class LockstepLeader(EngineIface):
    """The leader of a tensor / pipeline / expert parallel group: each call is broadcast, then run locally."""

    def __init__(self, engine: EngineIface, plane: ControlPlane):
        self.e, self.plane = engine, plane
        self.vocab_size, self.max_len, self.max_seqs, self.eos_ids = engine.vocab_size, engine.max_len, engine.max_seqs, engine.eos_ids

    def _all(self, name, *args):
        self.plane.broadcast((name, args))
        return getattr(self.e, name)(*args)

    def reset(self, slot): return self._all("reset", slot)
    def truncate(self, slot, length): return self._all("truncate", slot, length)
    def prefill(self, slot, ids): return self._all("prefill", slot, list(ids))
    def step(self, rows): return self._all("step", {int(k): list(v) for k, v in rows.items()})
    def length(self, slot): return self.e.length(slot)

    def reset_failure(self):
        if hasattr(self.e, "reset_failure"):
            self._all("reset_failure")
    def kv_form(self): return self.e.kv_form()

    def logits(self, slot, row=0):
        """The row's logits over the WHOLE vocabulary.  Under tensor parallelism every rank holds a slice of the
        vocabulary, under pipeline parallelism only the last stage holds the row: every rank reports its part
        (first id, values) over the control plane and the leader puts the row together, so the host sampler never
        sees a shard (the reference gathers both halves of a sampled row on the host: src/runtime/tp_engine.h:240-243)."""
        if not hasattr(self.e, "logits_shard"):
            return self.e.logits(slot, row)
        self.plane.broadcast(("logits_shard", (slot, row)))
        parts = [self.e.logits_shard(slot, row)] + [self.plane.recv(r) for r in range(1, self.plane.world)]
        full = np.full(self.vocab_size, -np.inf, dtype=np.float32)
        for off, vals in parts:
            vals = np.asarray(vals, dtype=np.float32)
            full[off: off + len(vals)] = vals[: max(0, self.vocab_size - off)]
        return full

    def shutdown(self):
        self.plane.broadcast((SHUTDOWN, ()))


class LockstepSpecLeader(LockstepLeader):
    """The leader of a group whose engines carry a draft head: every rank drafts (the head's layers are sliced like the
    trunk's and its chained rows meet in the same kernels); the drafts the leader returns reach the followers again as
    the verify step's rows."""

    def draft(self, slot, pending, k, temperature=0.0, seed=0):
        return self._all("draft", int(slot), int(pending), int(k), float(temperature), int(seed))

    def draft_many(self, reqs):
        return self._all("draft_many", {int(s): tuple(r) for s, r in reqs.items()})

    def draft_q(self, slot):
        return self.e.draft_q(slot)

    @property
    def stats(self):
        return self.e.stats


def lockstep_leader(engine: EngineIface, plane: ControlPlane) -> LockstepLeader:
    return LockstepSpecLeader(engine, plane) if hasattr(engine, "draft_many") else LockstepLeader(engine, plane)


def follow_lockstep(engine: EngineIface, plane: ControlPlane) -> int:
    """Follower loop of a lock-step group; returns the number of commands executed."""
    n = 0
    while True:
        msg = plane.next_broadcast()
        if msg[0] == SHUTDOWN:
            return n
        try:
            res = _apply(engine, msg)
        except Exception as e:  # noqa: BLE001   a failed step latches this rank's engine; the leader's own copy of
            res = e             # the step fails too (the ranks meet inside it) and sends reset_failure next
            sys.stderr.write(f"[rank {plane.rank}] {msg[0]} failed: {e}\n")
        if msg[0] == "logits_shard":     # the one call whose result the leader needs from every rank
            plane.send(0, res if not isinstance(res, Exception) else (0, np.zeros(0, dtype=np.float32)))
        n += 1


# ---------------------------------------------------------------------- replicas
class ReplicaRouter(EngineIface):
    """Slots of all replicas behind one EngineIface.  Global slot ``g`` lives on rank ``g // per`` as local slot
    ``g % per``; rank 0's own engine is called directly, the others through the control plane."""

    def __init__(self, local: EngineIface, plane: ControlPlane):
        self.local, self.plane = local, plane
        self.per = local.max_seqs
        self.world = plane.world
        self.vocab_size, self.max_len, self.eos_ids = local.vocab_size, local.max_len, local.eos_ids
        self.max_seqs = self.per * self.world
        self.calls = [0] * self.world

    def _where(self, slot: int):
        return slot // self.per, slot % self.per

    def _call(self, rank: int, name: str, *args):
        self.calls[rank] += 1
        if rank == 0:
            return getattr(self.local, name)(*args)
        self.plane.send(rank, (name, args))
        return self.plane.recv(rank)

    def reset(self, slot):
        r, s = self._where(slot)
        return self._call(r, "reset", s)

    def length(self, slot):
        r, s = self._where(slot)
        return self._call(r, "length", s)

    def truncate(self, slot, length):
        r, s = self._where(slot)
        return self._call(r, "truncate", s, length)

    def prefill(self, slot, ids):
        r, s = self._where(slot)
        return self._call(r, "prefill", s, list(ids))

    def logits(self, slot, row=0):
        r, s = self._where(slot)
        return np.asarray(self._call(r, "logits", s, row))

    def step(self, rows: Dict[int, List[int]]):
        by_rank: Dict[int, Dict[int, List[int]]] = {}
        for g, toks in rows.items():
            r, s = self._where(int(g))
            by_rank.setdefault(r, {})[s] = list(toks)
        # remote ranks first (they start working while rank 0 runs its own rows), then collect
        for r, part in by_rank.items():
            if r != 0:
                self.calls[r] += 1
                self.plane.send(r, ("step", (part,)))
        out: Dict[int, List[int]] = {}
        if 0 in by_rank:
            self.calls[0] += 1
            for s, v in self.local.step(by_rank[0]).items():
                out[s] = v
        for r, part in by_rank.items():
            if r != 0:
                res = self.plane.recv(r)
                if isinstance(res, Exception):
                    raise res
                for s, v in res.items():
                    out[r * self.per + int(s)] = v
        return out

    def shutdown(self):
        for r in range(1, self.world):
            self.plane.send(r, (SHUTDOWN, ()))


def serve_replica_worker(engine: EngineIface, plane: ControlPlane) -> int:
    """Worker loop of a replica rank: executes the router's calls on the local engine and returns the results."""
    n = 0
    while True:
        msg = plane.recv(0)
        if msg[0] == SHUTDOWN:
            return n
        try:
            res = _apply(engine, msg)
        except Exception as e:  # noqa: BLE001   (the request fails on the leader, the worker lives on)
            res = RuntimeError(f"replica rank {plane.rank}: {e}")
        plane.send(0, res)
        n += 1


# ---------------------------------------------------------------------- process launch
def parse_parallel(text: str):
    """``replica`` | ``tp4`` | ``pp2`` | ``ep8`` -> (kind, degree or None)."""
    t = (text or "").strip().lower()
    for kind in ("replica", "tp", "pp", "ep"):
        if t.startswith(kind):
            rest = t[len(kind):]
            return kind, (int(rest) if rest else None)
    raise ValueError(f"unknown --parallel value {text!r}")


def serve_parallel(flags, par: str, world: int) -> int:
    """Entry of ``serve --parallel ...``: under a launcher (RANK set) this is one rank; otherwise the ranks are
    started with the torch launcher on 127.0.0.1 and this process waits for them."""
    if "RANK" not in os.environ:
        import subprocess
        kind, deg = parse_parallel(par)
        n = deg or world
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29571"),
               "-m", "b200serve.cli.serve"] + sys.argv[1:]
        return subprocess.call(cmd)
    from ..cli.common import build_rank_engine
    return build_rank_engine(flags, par)
