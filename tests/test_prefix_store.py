"""Prefix store policy on a fake page pool: hits adopt pages, misses compute, spills and restores keep the data."""
import pytest

from b200serve.runtime.kv_pool import KvPoolPy
from b200serve.server.prefix import PAGE, PrefixStore

H = pytest.importorskip("b200serve.native.host")


class FakeKV:
    """Pages hold the token ids 'computed' into them, so a restore can be checked position by position."""
    form = "fake"
    page_bytes = 64

    def __init__(self, num_pages=64, slots=4):
        self.pool = KvPoolPy(num_pages, slots, 64)
        self.data = {}
        self.num_pages = num_pages
        self.seq_len = [0] * slots

    def free_pages(self): return self.pool.free_pages()
    def total_pages(self): return self.num_pages
    def slot_pages(self, slot): return list(self.pool.table(slot))
    def slot_length(self, slot): return self.seq_len[slot]
    def pin(self, pages): [self.pool.pin(p) for p in pages]
    def unpin(self, pages): [self.pool.unpin(p) for p in pages]

    def set_slot(self, slot, pages, length):
        pages = list(pages)
        [self.pool.pin(p) for p in pages]
        self.pool.release(slot)
        self.pool.adopt(slot, pages)
        [self.pool.unpin(p) for p in pages]
        self.seq_len[slot] = length

    def grow(self, slot, n):
        before = len(self.pool.table(slot))
        self.pool.ensure(slot, before + n)
        return list(self.pool.table(slot))[before:]

    def new_host_store(self, n_slots, ppb): return [dict() for _ in range(1)]
    def to_host(self, store, idx, pages): store[0][idx] = [self.data.get(p) for p in pages]
    def from_host(self, store, idx, pages):
        for p, d in zip(pages, store[0][idx]):
            self.data[p] = d

    # the "engine": computes positions [have, len(ids)) into the slot's pages
    def prefill(self, slot, ids):
        have = self.seq_len[slot]
        self.pool.ensure(slot, (len(ids) + PAGE - 1) // PAGE)
        t = self.pool.table(slot)
        for pos in range(have - have % PAGE, len(ids), PAGE):
            self.data[t[pos // PAGE]] = tuple(ids[pos: pos + PAGE])
        self.seq_len[slot] = len(ids)
        return len(ids) - have

    def check(self, slot, ids, upto):
        t = self.pool.table(slot)
        for pos in range(0, upto, PAGE):
            assert self.data[t[pos // PAGE]][: min(PAGE, upto - pos)] == tuple(ids[pos: pos + min(PAGE, upto - pos)])


def _store(kv, **kw):
    return PrefixStore(kv, host_gb=kw.pop("host_gb", 1e-6 * 40), block_tokens=32, **kw)


def run(store, kv, slot, ids):
    cached = store.begin(slot, ids)
    assert kv.seq_len[slot] == cached
    kv.check(slot, ids, cached)
    computed = kv.prefill(slot, ids)
    store.after_prefill(slot, ids)
    store.end(slot, ids)
    return cached, computed


def test_cold_then_restore_on_another_slot_shares_pages():
    kv = FakeKV()
    st = _store(kv)
    a = list(range(100, 200))                 # 100 tokens: 3 whole blocks of 32
    assert run(st, kv, 0, a) == (0, 100)
    b = a[:70] + [9, 9, 9, 9]                 # shares 70 tokens: 2 whole blocks
    cached, computed = run(st, kv, 1, b)
    assert cached == 64 and computed == len(b) - 64
    assert kv.slot_pages(1)[:4] == kv.slot_pages(0)[:4]          # the same device pages, by reference
    assert st.stats["hits"] == 1


def test_continue_on_the_same_slot_uses_resident_prefix():
    kv = FakeKV()
    st = _store(kv)
    a = list(range(50))
    run(st, kv, 0, a)
    assert st.preferred_slot(a + [1, 2, 3]) == 0
    cached, _ = run(st, kv, 0, a + [1, 2, 3])
    assert cached == 48                       # whole pages of the 50 resident positions
    assert st.stats["continued"] == 1


def test_split_last_and_full_hit_still_runs_a_row():
    kv = FakeKV()
    st = _store(kv)
    a = list(range(64))
    run(st, kv, 0, a)
    cached = st.begin(1, a, True)
    assert cached <= 63 and cached == 32      # the last position is never served from the cache


def test_spill_to_host_and_restore_keeps_data():
    kv = FakeKV(num_pages=24)
    st = _store(kv, device_fraction=0.2, host_gb=1e-5)    # device budget: 4 pages = 2 blocks
    assert st.host_slots >= 4
    a = list(range(1000, 1128))               # 4 blocks
    run(st, kv, 0, a)
    assert st.stats["spilled"] >= 2 and st.device_pages <= st.device_budget
    st.resident.clear()
    kv.set_slot(0, [], 0)
    for p in list(kv.data):                   # wipe what no longer belongs to a pinned page
        if kv.pool.ref[p] == 0:
            kv.data[p] = None
    cached, computed = run(st, kv, 2, a + [5])
    assert cached == 128 and computed == 1
    assert st.stats["restored_blocks"] >= 2


def _boundary_store(block=32):
    kv = FakeKV()
    return kv, PrefixStore(kv, host_gb=0, block_tokens=block, device_fraction=0.9)


@pytest.mark.parametrize("n_prompt,n_out", [(60, 4), (28, 4), (16, 16), (30, 3)])
def test_end_records_only_positions_whose_kv_was_written(n_prompt, n_out):
    # a request that ends by length: its last emitted token was never fed, so the slot holds P + n - 1 positions.
    # Total lengths on a page boundary (16), on a block boundary (32, 64) and in between.
    kv, st = _boundary_store()
    prompt = list(range(100, 100 + n_prompt))
    out = list(range(500, 500 + n_out))
    st.begin(0, prompt)
    kv.prefill(0, prompt)
    st.after_prefill(0, prompt)
    kv.prefill(0, prompt + out[:-1])                       # decode steps feed every token but the last one
    st.end(0, prompt + out)
    held = n_prompt + n_out - 1
    assert len(st.resident[0]) == held
    nxt = prompt + out + [7, 8, 9]
    got = st.begin(0, nxt)
    assert got <= held and got % PAGE == 0
    kv.check(0, nxt, got)
    # blocks in the index cover written positions only
    assert st.stats["inserted"] == held // 32


def test_cancel_in_the_middle_of_the_prompt_pass_keeps_the_written_part_only():
    kv, st = _boundary_store()
    prompt = list(range(200, 300))
    st.begin(1, prompt)
    kv.prefill(1, prompt[:40])                              # the pass was cancelled after 40 positions
    st.end(1, prompt)
    assert len(st.resident[1]) == 40
    got = st.begin(1, prompt)
    assert got <= 40 and got % PAGE == 0
    kv.check(1, prompt, got)


def test_split_last_keeps_one_more_position_out():
    ix = H.PrefixCache(16)
    root = ix.root("bf16")
    ids = list(range(33))
    ix.insert(root, ids[0:16], [1])
    node = ix.match(root, ids, 32)[0]
    ix.insert(node, ids[16:32], [2])
    # 33-token prompt: positions 0..31 may come from the cache, the last token is run
    assert ix.plan(root, ids, [], False)["matched_tokens"] == 32
    # split_last: the match must end before position n - 2 as well, so the second block no longer fits
    assert ix.plan(root, ids, [], True)["matched_tokens"] == 16


def test_pool_pressure_spills_cached_blocks_then_evicts_idle_sessions():
    """A request that needs more pages than the pool has free: cached blocks leave the device tier first, then the
    sessions of finished requests leave their slots, least recently ended first; the running request itself and the
    requesting slot are never touched, and a later turn of an evicted session finds its whole blocks in the index."""
    kv = FakeKV(num_pages=24, slots=4)
    st = PrefixStore(kv, host_gb=1e-6 * 40, block_tokens=32, device_fraction=0.9)
    a, b = list(range(1000, 1100)), list(range(2000, 2100))        # 100 tokens each: 7 pages, 3 whole blocks
    run(st, kv, 0, a)
    run(st, kv, 1, b)
    free0 = kv.free_pages()
    assert 0 < free0 <= 24 - 14
    # slot 2 is a running request that grows past what is free
    c = list(range(3000, 3000 + 16 * free0))
    st.begin(2, c)
    kv.prefill(2, c)                                               # takes every free page
    assert kv.free_pages() == 0
    assert st.make_room(2, 4)
    assert kv.free_pages() >= 4
    assert st.stats["spilled"] + st.stats.get("idle_evicted", 0) > 0
    assert kv.slot_pages(2) and kv.seq_len[2] == len(c)            # the running request kept everything
    # everything idle may go when more is asked for; what cannot be covered is reported
    assert st.make_room(2, 12)
    assert not st.make_room(2, 100)
    assert 0 not in st.resident and 1 not in st.resident           # both idle sessions left their slots
    # the first session's whole blocks are still known: its next turn restores them (from the host tier here)
    cached = st.begin(3, a + [7, 7, 7])
    assert cached in (0, 32, 64, 96)
    kv.check(3, a, cached)
