"""Native host library: KV pool, prompt lookup (against brute force), acceptance rules, K policies,
prefix cache index, scheduler.  CPU only."""
import random

import numpy as np
import pytest

from b200serve.native import host as H
from b200serve.runtime.kv_pool import KvPoolPy


# ----------------------------------------------------------------------------- KV pool
def test_kv_pool_native_equals_python_model():
    rnd = random.Random(0)
    a, b = H.KvPool(40, 4, 16), KvPoolPy(40, 4, 16)
    for _ in range(500):
        op = rnd.choice(["ensure", "truncate", "release", "share"])
        s = rnd.randrange(4)
        try:
            if op == "ensure":
                n = rnd.randrange(0, 12)
                ra = a.ensure(s, n)
            elif op == "truncate":
                n = rnd.randrange(0, 12)
                ra = a.truncate(s, n)
            elif op == "release":
                ra = a.release(s)
            else:
                d = rnd.randrange(4)
                if d == s:
                    continue
                n = rnd.randrange(0, 6)
                ra = a.share(s, d, n)
        except RuntimeError:
            ra = "oom"
        try:
            if op == "ensure":
                rb = b.ensure(s, n)
            elif op == "truncate":
                rb = b.truncate(s, n)
            elif op == "release":
                rb = b.release(s)
            else:
                rb = b.share(s, d, n)
        except MemoryError:
            rb = "oom"
        assert ra == rb
        assert a.free_pages() == b.free_pages()
        for q in range(4):
            assert list(a.table(q)) == b.table(q)
    assert 0 not in [p for q in range(4) for p in a.table(q)]     # page 0 is never handed out


def test_kv_pool_shared_pages_are_freed_once():
    p = H.KvPool(10, 2, 8)
    p.ensure(0, 3)
    p.share(0, 1, 2)
    assert p.free_pages() == 6 and p.refcount(p.table(0)[0]) == 2
    p.release(0)
    assert p.free_pages() == 7          # only the unshared third page came back
    p.release(1)
    assert p.free_pages() == 9


# ----------------------------------------------------------------------------- prompt lookup
def brute_match(ids, min_n, max_match=64):
    t = len(ids)
    best_e, best_m = -1, 0
    for e in range(t - 1):
        m = 0
        while m < max_match and m <= e and ids[e - m] == ids[t - 1 - m]:
            m += 1
        if m >= min_n and (m > best_m or (m == best_m and e > best_e)):
            best_e, best_m = e, m
    return best_e, best_m


@pytest.mark.parametrize("alphabet,n", [(3, 400), (8, 2000), (50, 3000)])
def test_prompt_lookup_equals_brute_force(alphabet, n):
    rnd = random.Random(alphabet)
    lk = H.PromptLookup(64, 1 << 30, 1 << 30)      # caps out of the way: the answer must be exact
    ids = []
    for i in range(n):
        if ids and rnd.random() < 0.3:              # copy a stretch from earlier: long matches exist
            src = rnd.randrange(len(ids))
            ext = ids[src: src + rnd.randrange(1, 40)]
        else:
            ext = [rnd.randrange(alphabet)]
        for t in ext:
            ids.append(t)
            lk.append(t)
        if i % 7 == 0 and len(ids) > 2:
            for min_n in (2, 3, 5, 16):
                e, m, _, trunc = lk.match(min_n)
                be, bm = brute_match(ids, min_n)
                assert not trunc
                assert (e, m if e >= 0 else 0) == (be, bm if be >= 0 else 0), (len(ids), min_n)


def test_prompt_lookup_overlapping_copy_boundary_truncate():
    lk = H.PromptLookup()
    lk.extend([5, 6, 7, 7, 7, 7])
    assert lk.propose(6, 2) == [7, 7, 7, 7, 7, 7]            # a run drafts the run on (LZ77 overlap)
    lk.clear()
    lk.extend([1, 2, 3, 4])
    lk.boundary()
    lk.extend([9, 1, 2, 3])
    assert lk.propose(5, 3) == [4]                             # the continuation stops at the boundary
    lk.truncate(8)                                             # ... 9, 1, 2
    assert lk.size() == 8
    assert lk.propose(5, 2) == [3, 4]
    with pytest.raises(ValueError):
        lk.append(0xFFF00001)


def test_lookup_policy_enter_stay_escalate():
    p = H.LookupPolicy()
    assert p.decide(5) == 0 and not p.active()
    assert p.decide(8) == 16
    p.observe(16, 16)
    assert p.decide(4) == 32
    p.observe(32, 32)
    assert p.decide(3) == 64
    p.observe(64, 10)
    assert p.decide(3) == 16
    assert p.decide(2) == 0 and not p.active()


# ----------------------------------------------------------------------------- acceptance
def test_filter_probs_topk_topp():
    logits = np.array([1.0, 3.0, 2.0, 0.0, -5.0], dtype=np.float32)
    ids, probs, mass = H.filter_probs(logits, 5, 1.0, 3, 1.0)
    assert ids == [1, 2, 0] and abs(mass - 1.0) < 1e-12
    ids, probs, mass = H.filter_probs(logits, 5, 1.0, 0, 0.6)
    assert ids == [1]                                        # the first prefix reaching 0.6
    ids, _, _ = H.filter_probs(logits, 2, 1.0, 0, 1.0)       # vocabulary mask: ids >= vocab_used never appear
    assert set(ids) == {0, 1}


def test_repetition_penalty_hf_rule():
    l = np.array([2.0, -2.0, 1.0], dtype=np.float32)
    H.apply_repetition_penalty(l, 3, [0, 1, 1, 7], 2.0)
    assert l.tolist() == [1.0, -4.0, 1.0]


def test_accept_greedy():
    assert H.accept_greedy([4, 5, 6, 7], [4, 5, 9]) == (2, 6)
    assert H.accept_greedy([4, 5, 6, 7], [4, 5, 6]) == (3, 7)
    assert H.accept_greedy([4], []) == (0, 4)


def test_accept_sampled_is_lossless():
    """The emitted first token is distributed as p whatever q is (Leviathan et al.)."""
    rng = np.random.default_rng(0)
    v = 6
    p_rows = rng.normal(size=(2, v)).astype(np.float32)
    q_rows = rng.normal(size=(1, v)).astype(np.float32)
    p = np.exp(p_rows[0] - p_rows[0].max()); p /= p.sum()
    q = np.exp(q_rows[0] - q_rows[0].max()); q /= q.sum()
    counts = np.zeros(v)
    n = 20000
    draft_rng = np.random.default_rng(1)
    for i in range(n):
        d = int(draft_rng.choice(v, p=q))
        acc, nxt = H.accept_sampled(p_rows, q_rows, [d], v, 1.0, 0, 1.0, 1000 + i)
        counts[d if acc == 1 else nxt] += 1
    assert np.abs(counts / n - p).max() < 0.015


def test_accept_point_mass_is_lossless():
    rng = np.random.default_rng(3)
    v = 5
    p_rows = rng.normal(size=(2, v)).astype(np.float32)
    p = np.exp(p_rows[0] - p_rows[0].max()); p /= p.sum()
    counts = np.zeros(v)
    n = 20000
    for i in range(n):
        acc, nxt = H.accept_point_mass(p_rows, [2], v, 1.0, 0, 1.0, 5000 + i)
        counts[2 if acc == 1 else nxt] += 1
    assert np.abs(counts / n - p).max() < 0.015


def test_accept_sparse_is_lossless():
    rng = np.random.default_rng(4)
    v = 8
    p_rows = rng.normal(size=(2, v)).astype(np.float32)
    p = np.exp(p_rows[0] - p_rows[0].max()); p /= p.sum()
    cand = np.array([[1, 4, 6]], dtype=np.uint32)
    scores = np.array([[0.5, 1.5, -0.3]], dtype=np.float32)
    q = np.exp(scores[0] - scores[0].max()); q /= q.sum()
    counts = np.zeros(v)
    n = 20000
    drng = np.random.default_rng(9)
    for i in range(n):
        d = int(cand[0][drng.choice(3, p=q)])
        acc, nxt = H.accept_sparse(p_rows, cand, scores, [d], v, 1.0, 0, 1.0, 77 + i)
        counts[d if acc == 1 else nxt] += 1
    assert np.abs(counts / n - p).max() < 0.015


# ----------------------------------------------------------------------------- K policies
def test_draft_length_policy_follows_acceptance():
    k = H.DraftLengthPolicy()
    assert k.next() == 3                                   # settles at the deepest depth first
    for _ in range(30):
        kk = k.next()
        k.observe(kk, kk)                                  # everything accepted
    assert k.current() == 3 and k.acceptance(0) > 0.9 and k.acceptance(2) > 0.9
    assert k.expected_tokens(3) > 3.5
    for _ in range(60):
        kk = k.next()
        k.observe(kk, 0)                                   # nothing accepted
    assert k.current() == 0 and k.acceptance(0) < 0.1
    probes = 0
    for _ in range(60):
        kk = k.next()
        probes += kk > 0
        k.observe(kk, 0)
    assert 1 <= probes <= 8                                # at depth 0 a probe now and then, the gap growing
    for _ in range(200):                                   # the text becomes predictable again: probes bring depth back
        kk = k.next()
        k.observe(kk, kk)
    assert k.current() == 3


def test_draft_length_policy_is_per_position():
    # a head whose first draft is reliable and whose later drafts are not: depth 1 pays, depth 3 does not
    k = H.DraftLengthPolicy()
    for _ in range(80):
        kk = k.next()
        k.observe(kk, min(kk, 1))
    assert k.acceptance(0) > 0.9 and k.acceptance(1) < 0.3
    assert k.current() == 1 and k.best_depth() == 1


def test_step_costs_table():
    c = H.StepCosts([1.0, 1.1, 1.2, 1.3], [0.2, 0.4, 0.6])
    assert c.deepest() == 3 and abs(c.iteration(2) - 1.6) < 1e-12 and c.iteration(0) == 1.0
    f = c.free_drafts()
    assert abs(f.iteration(3) - 1.3) < 1e-12


def test_confidence_stop_drops_unsure_draft():
    model = H.ConfidenceModel()
    s = H.ConfidenceStop(H.StepCosts(), 3, model)
    assert s.begin() == 3
    assert s.after_draft(1, 0.99) == -1                     # confident: draft another
    r = s.after_draft(2, 0.02)                              # unsure: verify only the first
    assert r == 1
    s.observe(1)
    assert s.verified() == 1


def test_confidence_model_learns_overconfidence():
    model = H.ConfidenceModel()
    assert abs(model.accept_prob(1, 0.9) - 0.9) < 1e-9      # starts by believing the head
    rnd = random.Random(3)
    for _ in range(3000):                                   # position 1 says 0.9 but is right half of the time
        model.learn(1, 0.9, rnd.random() < 0.5)
    assert 0.35 < model.accept_prob(1, 0.9) < 0.65         # near one half, up to the noise of single-sample steps
    assert abs(model.accept_prob(0, 0.9) - 0.9) < 1e-9      # other positions are untouched


# ----------------------------------------------------------------------------- prefix cache
def test_prefix_cache_match_plan_evict():
    c = H.PrefixCache(16)
    root = c.root("bf16")
    ids = list(range(100))
    n0, created = c.insert(root, ids[0:16], [3])
    assert created
    n1, _ = c.insert(n0, ids[16:32], [4])
    n1b, created = c.insert(n0, ids[16:32], [9])
    assert n1b == n1 and not created                       # an equal block is not stored twice
    assert c.match(root, ids, 100) == [n0, n1]
    assert c.match(root, ids, 31) == [n0]                  # only whole blocks below the limit
    assert c.match(c.root("int8"), ids, 100) == []         # forms do not mix
    other = ids[:20] + [999] + ids[21:]
    assert c.match(root, other, 100) == [n0]
    p = c.plan(root, ids[:40], [], False)
    assert p["kind"] == "restore" and p["matched_tokens"] == 32 and p["path"] == [n0, n1]
    p = c.plan(root, ids[:32], [], False)                  # the last prompt token is always run
    assert p["matched_tokens"] == 16
    p = c.plan(root, ids[:40], ids[:36], False)
    assert p["kind"] == "continue" and p["matched_tokens"] == 36
    p = c.plan(root, [7] * 40, [], False)
    assert p["kind"] == "cold"
    # eviction: device pages go leaf first, pinned nodes stay
    assert c.device_victim() == n1
    c.pin(n1)
    assert c.device_victim() == -1                         # n0 still has a child holding device pages
    c.unpin(n1)
    c.set_device_pages(n1, [])
    assert c.device_victim() == n0
    assert c.leaf_victim() == n1
    pages, slot = c.remove(n1)
    assert pages == [] and slot == -1 and c.num_nodes() == 1


# ----------------------------------------------------------------------------- scheduler
def test_scheduler_tick_order_and_row_budget():
    o = H.SchedOptions()
    o.max_slots, o.max_queue, o.prefill_chunk, o.row_budget = 2, 2, 100, 5
    s = H.Scheduler(o)
    assert s.submit(1, 250, 10) and s.submit(2, 50, 10)
    assert not s.submit(3, 10, 10)                          # queue full -> 503
    plan = s.tick()
    assert [a["kind"] for a in plan] == ["grant", "grant", "prefill"]
    assert plan[2]["slot"] == 0 and (plan[2]["begin"], plan[2]["end"], plan[2]["last"]) == (0, 100, False)
    s.prefill_done(0, 100)
    assert s.submit(3, 10, 10)
    plan = s.tick()
    assert [a["kind"] for a in plan] == ["prefill"] and plan[0]["begin"] == 100
    s.prefill_done(0, 200)
    s.tick(); s.prefill_done(0, 250)                        # request 1 now decodes
    plan = s.tick()
    kinds = [a["kind"] for a in plan]
    assert kinds == ["prefill", "decode"]                  # one chunk of request 2 and a decode step of request 1
    assert plan[1]["slots"] == [0] and plan[1]["rows"] == [1]
    s.prefill_done(1, 50)
    s.set_rows(0, 4); s.set_rows(1, 4)
    plan = s.tick()
    assert plan[-1]["kind"] == "decode" and plan[-1]["slots"] == [0, 1]
    assert plan[-1]["rows"] == [4, 1]                       # budget 5: both get a row, the older gets the drafts
    s.tokens(0, 20, False)                                  # reaches max_new -> released next tick, request 3 granted
    plan = s.tick()
    assert [a["kind"] for a in plan][:2] == ["release", "grant"]
    s.cancel(2)
    plan = s.tick()
    assert plan[0]["kind"] == "release" and plan[0]["req"] == 2
