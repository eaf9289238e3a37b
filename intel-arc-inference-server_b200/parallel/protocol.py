"""Host mirror of the cross-GPU wire: the same slots, epochs, flags and fold order, run by CPU threads.

The device kernels (``ops/csrc/wire.cuh``, the fold epilogue of ``gemv_w4.cu``) cannot be made to fail on
a shared GPU, so the protocol's failure behaviour is pinned here, as the reference pins its own with a host
mirror run by threads (src/runtime/tp_protocol.h:1-157, injection hooks :82-84):

  * call ``n`` uses slot ``n & 1``; a writer stores its part into every reader's landing buffer, then the
    flag ``= n`` (flags only grow);
  * a reader waits, bounded, for every peer's flag of that slot in ITS OWN memory, then adds the parts in
    rank order, so all ranks compute identical bits;
  * the first wait that runs out records (code, peer, call) once in the rank's status; later waits do not
    spin again, so a dead peer costs one bound; the rank stays "broken" until ``reset``.

Injection: ``drop_next(writer, reader)`` loses one flag, ``skip_data(writer, reader)`` delivers the flag
without the data (the stamp check catches it), ``kill(rank)`` stops a rank between calls.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional, Tuple

import numpy as np

TIMEOUT, STALE = 1, 2


class HostWire:
    def __init__(self, world: int, width: int, bound_s: float = 0.2):
        self.world, self.width, self.bound = world, width, bound_s
        # landing[reader][slot][writer] = (stamp, data); flags[reader][slot][writer] = call number
        self.data = np.zeros((world, 2, world, width), dtype=np.float32)
        self.stamp = np.zeros((world, 2, world), dtype=np.int64)
        self.flags = np.zeros((world, 2, world), dtype=np.int64)
        self.calls = [0] * world
        self.status: List[Optional[Tuple[int, int, int]]] = [None] * world      # (code, peer, call)
        self.waits_spun = [0] * world
        self.bounds_paid = [0] * world      # waits that ran their whole bound
        self._drop: Dict[Tuple[int, int], int] = {}
        self._skip: Dict[Tuple[int, int], int] = {}
        self._dead = set()
        self._lock = threading.Lock()

    # ---- injection
    def drop_next(self, writer: int, reader: int):
        self._drop[(writer, reader)] = self._drop.get((writer, reader), 0) + 1

    def skip_data(self, writer: int, reader: int):
        self._skip[(writer, reader)] = self._skip.get((writer, reader), 0) + 1

    def kill(self, rank: int):
        self._dead.add(rank)

    def reset(self, rank: int):
        self.status[rank] = None

    # ---- one all-reduce call of `rank`
    def all_reduce(self, rank: int, part: np.ndarray) -> Optional[np.ndarray]:
        """Returns the folded sum, or None when a wait ran out (the rank's status says why)."""
        if rank in self._dead:
            return None
        self.calls[rank] += 1
        n = self.calls[rank]
        slot = n & 1
        if self.status[rank] is not None:
            # Failure latch: a rank whose wait ran out takes no further part until it is reset.  Without it the
            # rank's next push would reuse the slot of the epoch its peer may still be waiting for, and the peer
            # would report that late flag as stale data instead of its own time-out.
            return None
        for reader in range(self.world):
            key = (rank, reader)
            with self._lock:
                skip = self._skip.get(key, 0) > 0
                drop = self._drop.get(key, 0) > 0
                if skip:
                    self._skip[key] -= 1
                if drop:
                    self._drop[key] -= 1
            if not skip:
                self.data[reader, slot, rank] = part
                self.stamp[reader, slot, rank] = n              # written with the data, before the flag
            if not drop:
                self.flags[reader, slot, rank] = n              # release: after data and stamp
        ok = True
        for peer in range(self.world):
            if peer == rank:
                continue
            if not self._wait(rank, slot, peer, n):
                ok = False
                break
            if self.stamp[rank, slot, peer] != n:               # flag arrived before the data
                self._fail(rank, STALE, peer, n)
                ok = False
                break
        if not ok:
            return None
        acc = np.zeros(self.width, dtype=np.float32)
        for src in range(self.world):                            # rank order: identical bits on every rank
            acc = acc + self.data[rank, slot, src]
        return acc

    def _wait(self, rank: int, slot: int, peer: int, n: int) -> bool:
        if self.flags[rank, slot, peer] >= n:
            return True
        if self.status[rank] is not None:                         # an earlier wait already ran out
            return False
        self.waits_spun[rank] += 1
        t0 = time.monotonic()
        while self.flags[rank, slot, peer] < n:
            if time.monotonic() - t0 > self.bound:
                self.bounds_paid[rank] += 1
                self._fail(rank, TIMEOUT, peer, n)
                return False
            time.sleep(0.0005)
        return True

    def _fail(self, rank: int, code: int, peer: int, n: int):
        if self.status[rank] is None:
            self.status[rank] = (code, peer, n)


def run_ranks(wire: HostWire, rounds: int, parts) -> List[List[Optional[np.ndarray]]]:
    """Runs ``rounds`` all-reduce calls on one thread per rank; ``parts(rank, round)`` gives each input."""
    out: List[List[Optional[np.ndarray]]] = [[] for _ in range(wire.world)]

    def body(r):
        for i in range(rounds):
            out[r].append(wire.all_reduce(r, parts(r, i)))

    ts = [threading.Thread(target=body, args=(r,)) for r in range(wire.world)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    return out


def ep_plan_mirror(cnt_all, rank: int, world: int, max_blk: int = 1 << 30):
    """Host mirror of ``ep_plan_kernel`` (ops/csrc/ep.cu): from every source's per-expert counts
    (``cnt_all[source][expert]``) the layout one rank derives -- where ITS rows of every expert start in the
    owner's receive buffer (``send_base``) and, for its own experts, the 128-row block table.  Every rank runs the
    same arithmetic on the same counts, which is why nothing but the counts is exchanged."""
    e_total = len(cnt_all[0])
    el = e_total // world
    tot = [sum(cnt_all[s][e] for s in range(world)) for e in range(e_total)]
    pad = [(t + 127) // 128 * 128 for t in tot]
    send_base, blocks = [0] * e_total, []
    total_rows = 0
    for e in range(e_total):
        owner = e // el
        base = sum(pad[e2] for e2 in range(owner * el, e))
        before = sum(cnt_all[s][e] for s in range(rank))
        send_base[e] = base + before
        if owner == rank:
            for j in range(pad[e] // 128):
                if base // 128 + j < max_blk:
                    blocks.append((e - owner * el, base + 128 * j, min(128, tot[e] - 128 * j)))
            if e - owner * el == el - 1:
                total_rows = base + pad[e]
    return send_base, blocks, total_rows
