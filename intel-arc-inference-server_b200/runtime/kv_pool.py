"""Paged-KV page pool: free list, reference counts, per-sequence page tables.

Same contract as the reference's ``KvPool`` (src/runtime/kv_pool.h:24-85): pages
are handed out from a host free list, a page shared by several sequences (a
cached prefix) is reference counted and returns to the free list when the last
holder lets go.  Page 0 is never handed out: unused table entries point at it,
so a kernel that reads a stale entry reads zeros, not another sequence.

The native implementation (``native/kv_pool.cc``) is used when the host library
is built; this Python class is the same algorithm and is what the CPU tests
compare it against.
"""
from __future__ import annotations

from typing import List


class KvPoolPy:
    def __init__(self, num_pages: int, max_seqs: int, max_blocks: int):
        self.num_pages, self.max_seqs, self.max_blocks = num_pages, max_seqs, max_blocks
        self.free: List[int] = list(range(num_pages - 1, 0, -1))   # pop() hands out 1, 2, 3, ...
        self.ref = [0] * num_pages
        self.tables: List[List[int]] = [[] for _ in range(max_seqs)]

    def free_pages(self) -> int:
        return len(self.free)

    def table(self, seq: int) -> List[int]:
        return self.tables[seq]

    def ensure(self, seq: int, n_blocks: int) -> bool:
        """Grow ``seq``'s table to ``n_blocks`` pages. Returns True if the table changed."""
        t = self.tables[seq]
        if n_blocks > self.max_blocks:
            raise MemoryError(f"sequence needs {n_blocks} pages, table holds {self.max_blocks}")
        if len(t) >= n_blocks:
            return False
        need = n_blocks - len(t)
        if need > len(self.free):
            raise MemoryError(f"KV pool exhausted: need {need} pages, {len(self.free)} free")
        for _ in range(need):
            p = self.free.pop()
            self.ref[p] = 1
            t.append(p)
        return True

    def truncate(self, seq: int, n_blocks: int):
        t = self.tables[seq]
        while len(t) > n_blocks:
            self._unref(t.pop())

    def release(self, seq: int):
        self.truncate(seq, 0)

    def share(self, src_seq: int, dst_seq: int, n_blocks: int):
        """Make ``dst_seq`` start with the first ``n_blocks`` pages of ``src_seq`` (prefix reuse)."""
        self.release(dst_seq)
        for p in self.tables[src_seq][:n_blocks]:
            self.ref[p] += 1
            self.tables[dst_seq].append(p)

    def adopt(self, seq: int, pages: List[int]):
        """Append already-referenced pages (from the prefix cache) to ``seq``'s table."""
        for p in pages:
            self.ref[p] += 1
            self.tables[seq].append(p)

    def pin(self, page: int):
        self.ref[page] += 1

    def unpin(self, page: int):
        self._unref(page)

    def _unref(self, p: int):
        self.ref[p] -= 1
        assert self.ref[p] >= 0
        if self.ref[p] == 0:
            self.free.append(p)


def KvPool(num_pages: int, max_seqs: int, max_blocks: int):
    """The native pool when the host library is available, else the Python one."""
    try:
        from ..native import host
        if host.available():
            return host.KvPool(num_pages, max_seqs, max_blocks)
    except Exception:
        pass
    return KvPoolPy(num_pages, max_seqs, max_blocks)
