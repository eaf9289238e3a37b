"""Prefix cache: KV of token blocks kept past the request that computed them.

Two tiers under the native index (``native/src/prefix_cache.h``): a block's KV pages may stay in
the device page pool (a hit adopts the pages into the new sequence's block table -- no copy, the
pages are shared by reference count) and / or in a slot of a pinned host store (a hit costs one
host-to-device copy of the block).  When the device tier is over its budget the least recently
used blocks are spilled to the host store; when the host store is full its oldest leaves go.

The reference's store is host-only with 2048-position blocks plus recurrent-state snapshots
(src/server/prefix_cache.h:1-205, prefix_cache.cc:158-478, docs/04-architecture.md:421-426);
its plans -- Cold, Continue on the slot's own resident prefix, Restore from the store -- and
``--prefix-split-last`` (keep the last position out of the match so a fully cached prompt still
runs one row) are the same here.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np

PAGE = 16


def auto_host_gb() -> float:
    """The host store's size when none is given: min(16 GiB, half the RAM, what is available minus 8 GiB), the
    reference's rule (src/cli/prefix_cache_size.h)."""
    try:
        import psutil
        vm = psutil.virtual_memory()
        return max(0.0, min(16.0, vm.total / 2**31, vm.available / 2**30 - 8.0))   # 16, not 32: the store is pinned at start
    except Exception:
        return 4.0


def parse_gb(text, default_gb=None) -> float:
    if text in (None, "", "auto"):
        return auto_host_gb() if default_gb is None else default_gb
    return float(text)


class EngineKV:
    """What the store needs from an engine: page tables, pins and page copies."""

    def __init__(self, engine):
        import torch
        self.e = engine
        self.torch = torch
        kv = engine.kv
        self.tensors = [kv.k, kv.v] + ([kv.k_scale, kv.v_scale] if kv.kv_int8 else [])
        self.page_bytes = sum(int(t[:, 0].numel()) * t.element_size() for t in self.tensors)
        self.form = f"{engine.kv_dtype}/{engine.cfg.name}"

    def free_pages(self) -> int:
        return self.e.pool.free_pages()

    def total_pages(self) -> int:
        return self.e.kv.num_pages

    def slot_pages(self, slot: int) -> List[int]:
        return list(self.e.pool.table(slot))

    def slot_length(self, slot: int) -> int:
        """Positions of the slot whose KV has been written."""
        return int(self.e.seq_len[slot])

    def pin(self, pages: Sequence[int]):
        for p in pages:
            self.e.pool.pin(p)

    def unpin(self, pages: Sequence[int]):
        for p in pages:
            self.e.pool.unpin(p)

    def set_slot(self, slot: int, pages: Sequence[int], length: int):
        """The slot's sequence becomes ``pages`` (shared) holding ``length`` positions."""
        e = self.e
        pages = list(pages)
        for pg in pages:            # hold the pages across the release: the slot may be their only owner
            e.pool.pin(pg)
        e.pool.release(slot)
        e.pool.adopt(slot, pages)
        for pg in pages:
            e.pool.unpin(pg)
        e.seq_len[slot] = length
        self._sync_table(slot)

    def grow(self, slot: int, n_pages: int) -> List[int]:
        e = self.e
        before = len(e.pool.table(slot))
        e.pool.ensure(slot, before + n_pages)
        self._sync_table(slot)
        return list(e.pool.table(slot))[before:]

    def _sync_table(self, slot: int):
        e, torch = self.e, self.torch
        row = list(e.pool.table(slot))
        if not row:
            return
        host = e.table_stage.begin()
        host[: len(row)] = torch.from_numpy(np.asarray(row, dtype=np.int32))
        e.table_stage.push(e.block_table[slot, : len(row)], host[: len(row)])

    def new_host_store(self, n_slots: int, pages_per_block: int):
        torch = self.torch
        return [torch.empty((n_slots, t.shape[0], pages_per_block) + tuple(t.shape[2:]), dtype=t.dtype).pin_memory()
                for t in self.tensors]

    def to_host(self, store, slot_idx: int, pages: Sequence[int]):
        idx = self.torch.as_tensor(list(pages), device=self.tensors[0].device)
        for t, h in zip(self.tensors, store):
            h[slot_idx].copy_(t.index_select(1, idx), non_blocking=True)
        self.torch.cuda.current_stream().synchronize()

    def from_host(self, store, slot_idx: int, pages: Sequence[int]):
        idx = self.torch.as_tensor(list(pages), device=self.tensors[0].device)
        for t, h in zip(self.tensors, store):
            t.index_copy_(1, idx, h[slot_idx].to(t.device, non_blocking=True))


class PrefixStore:
    def __init__(self, engine_or_kv, host_gb="auto", block_tokens: int = 256, device_fraction: float = 0.5, index=None):
        self.kv = engine_or_kv if hasattr(engine_or_kv, "slot_pages") else EngineKV(engine_or_kv)
        if block_tokens % PAGE:
            raise ValueError("block_tokens must be a multiple of the page size")
        self.block = block_tokens
        self.ppb = block_tokens // PAGE
        if index is None:
            from ..native import host as H
            index = H.PrefixCache(block_tokens)
        self.ix = index
        self.root = self.ix.root(self.kv.form)
        self.device_budget = int(self.kv.total_pages() * device_fraction)
        self.device_pages = 0
        gb = parse_gb(host_gb)
        block_bytes = self.kv.page_bytes * self.ppb
        self.host_slots = max(0, int(gb * (1 << 30) // max(block_bytes, 1)))
        self.host_slots = min(self.host_slots, 4096)
        self.store = self.kv.new_host_store(self.host_slots, self.ppb) if self.host_slots else None
        self.host_free = list(range(self.host_slots - 1, -1, -1))
        self.host_owner: Dict[int, int] = {}        # host slot -> node
        self.resident: Dict[int, List[int]] = {}     # engine slot -> ids whose KV the slot still holds
        self.stats = {"hits": 0, "restored_blocks": 0, "continued": 0, "spilled": 0, "evicted": 0, "inserted": 0}
        self._ended: Dict[int, int] = {}      # slot -> when its request ended (idle sessions, for make_room)
        self._clock = 0
        eng = getattr(self.kv, "e", None)
        if eng is not None:
            eng.on_pool_pressure = self.make_room     # a request that needs pages the pool lacks asks here first

    # ------------------------------------------------------------------ scheduling hint
    def preferred_slot(self, ids: Sequence[int]) -> int:
        """The slot whose resident ids share the longest prefix with ``ids`` (at least one block), else -1."""
        best, best_n = -1, self.block - 1
        for slot, res in self.resident.items():
            n = 0
            lim = min(len(res), len(ids) - 1)
            while n < lim and res[n] == ids[n]:
                n += 1
            if n > best_n:
                best, best_n = slot, n
        return best

    # ------------------------------------------------------------------ request start
    def begin(self, slot: int, prompt: Sequence[int], split_last: bool = False) -> int:
        """Leaves ``slot`` holding the longest cached prefix of ``prompt``; returns its length in tokens."""
        prompt = [int(t) for t in prompt]
        res = self.resident.pop(slot, [])
        self._ended.pop(slot, None)
        plan = self.ix.plan(self.root, prompt, res, split_last)
        kind, matched = plan["kind"], plan["matched_tokens"]
        if kind == "continue":
            keep_pages = (matched + PAGE - 1) // PAGE
            pages = self.kv.slot_pages(slot)[:keep_pages]
            # a partly filled last page would be written by two sequences if it were shared: keep whole pages
            matched = min(matched, len(pages) * PAGE)
            matched -= matched % PAGE
            self.kv.set_slot(slot, pages[: matched // PAGE], matched)
            self.stats["continued"] += 1
            if matched:
                self.stats["hits"] += 1
            return matched
        if kind == "restore":
            pages: List[int] = []
            got = 0
            self.kv.set_slot(slot, [], 0)
            for node in plan["path"]:
                dp = self.ix.device_pages(node)
                if dp:
                    self.kv.set_slot(slot, pages + list(dp), got + self.block)
                    pages += list(dp)
                else:
                    hs = self.ix.host_slot(node)
                    if hs < 0:
                        break
                    self._make_room(self.ppb)
                    self.kv.set_slot(slot, pages, got)
                    try:
                        new = self.kv.grow(slot, self.ppb)
                    except MemoryError:
                        break
                    self.kv.from_host(self.store, hs, new)
                    pages += new
                    self.stats["restored_blocks"] += 1
                    # the block is on the device again: let later requests share these pages
                    self.kv.pin(new)
                    self.ix.set_device_pages(node, new)
                    self.device_pages += len(new)
                got += self.block
            self.kv.set_slot(slot, pages, got)
            if got:
                self.stats["hits"] += 1
            return got
        self.kv.set_slot(slot, [], 0)
        return 0

    # ------------------------------------------------------------------ after the prompt pass / at the end
    def _held(self, slot: int, ids: Sequence[int]) -> List[int]:
        """The ids whose KV the slot really holds: a token that was emitted but never fed (the last one of a request
        that ended by length or by a stop string), or the rest of a prompt whose pass was cancelled, has no KV."""
        n = self.kv.slot_length(slot)
        return [int(t) for t in ids[: max(0, n)]]

    def after_prefill(self, slot: int, prompt: Sequence[int]):
        self._insert_blocks(slot, self._held(slot, prompt))

    def end(self, slot: int, ids: Sequence[int]):
        ids = self._held(slot, ids)
        self._insert_blocks(slot, ids)
        self.resident[slot] = ids
        self._clock += 1
        self._ended[slot] = self._clock          # an idle session from now on: its pages may be taken back

    def make_room(self, slot: int, n_pages: int) -> bool:
        """Called when the page pool cannot give ``slot`` the ``n_pages`` more it needs (the role of the reference
        scheduler's make_room / evict, src/server/scheduler.cc:940-1010).  First cached blocks leave the device tier
        (to the host tier when there is one), least recently used first; then the sessions of finished requests
        that still sit in their slots leave, oldest first: their whole blocks stay in the index (a later turn restores
        them), the partly filled last block is dropped.  True when the pages are free afterwards."""
        self._make_room(n_pages)
        while self.kv.free_pages() < n_pages and self._ended:
            victim = min((s for s in self._ended if s != slot), key=lambda s: self._ended[s], default=None)
            if victim is None:
                break
            del self._ended[victim]
            self.resident.pop(victim, None)
            self.kv.set_slot(victim, [], 0)
            self.stats["idle_evicted"] = self.stats.get("idle_evicted", 0) + 1
            self._make_room(n_pages)          # the session's shared blocks are unreferenced now and may spill
        return self.kv.free_pages() >= n_pages

    def _insert_blocks(self, slot: int, ids: List[int]):
        pages = self.kv.slot_pages(slot)
        # whole blocks of WRITTEN positions only: a block whose last position has no KV yet is not shared
        n_blocks = min(len(ids) // self.block, len(pages) // self.ppb, max(0, self.kv.slot_length(slot)) // self.block)
        parent = self.root
        for b in range(n_blocks):
            blk_ids = ids[b * self.block: (b + 1) * self.block]
            blk_pages = pages[b * self.ppb: (b + 1) * self.ppb]
            node, created = self.ix.insert(parent, blk_ids, blk_pages)
            if created:
                self.kv.pin(blk_pages)
                self.device_pages += len(blk_pages)
                self.stats["inserted"] += 1
            parent = node
        self._trim_device()

    # ------------------------------------------------------------------ tiers
    def _trim_device(self):
        while self.device_pages > self.device_budget:
            if not self._spill_one():
                break

    def _make_room(self, n_pages: int):
        while self.kv.free_pages() < n_pages:
            if not self._spill_one():
                break

    def _spill_one(self) -> bool:
        """Moves the least recently used device block to the host store (or drops it when there is none)."""
        node = self.ix.device_victim()
        if node < 0:
            return False
        pages = list(self.ix.device_pages(node))
        if self.store is not None and self.ix.host_slot(node) < 0:
            hs = self._host_slot()
            if hs >= 0:
                self.kv.to_host(self.store, hs, pages)
                self.ix.set_host_slot(node, hs)
                self.host_owner[hs] = node
                self.stats["spilled"] += 1
        self.ix.set_device_pages(node, [])
        self.kv.unpin(pages)
        self.device_pages -= len(pages)
        if self.ix.host_slot(node) < 0:
            hs = self._drop(node)
            if hs >= 0:
                self.host_free.append(hs)
        return True

    def _host_slot(self) -> int:
        if self.host_free:
            return self.host_free.pop()
        for _ in range(64):
            victim = self.ix.leaf_victim()      # oldest unpinned leaf
            if victim < 0:
                return -1
            hs = self._drop(victim)
            if hs >= 0:
                return hs
        return -1

    def _drop(self, node: int) -> int:
        """Removes a leaf from the index and releases what it held; returns its host slot (or -1)."""
        try:
            pages, hs = self.ix.remove(node)
        except Exception:
            return -1          # an inner node: it stays as a bare link of the chain
        if pages:
            self.kv.unpin(list(pages))
            self.device_pages -= len(pages)
        if hs >= 0:
            self.host_owner.pop(hs, None)
        self.stats["evicted"] += 1
        return hs
