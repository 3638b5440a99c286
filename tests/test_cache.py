"""Host bookkeeping of the cache: slots and pages are never lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from spissa_b200.cache import CacheFull, CacheManager, CacheMisuse, IndexPool
from spissa_b200.parts.base import KVCacheRequest, StateRequest


def manager(max_tokens=640, max_seqs=4, window=None, extra=None):
    req = {0: KVCacheRequest(2, 16, None), 1: KVCacheRequest(2, 16, None)}
    if window:
        req[2] = KVCacheRequest(2, 16, window)
    if extra:
        req.update(extra)
    return CacheManager(req, max_tokens, max_seqs, 64, torch.float32, "cpu", allocate=False)


def test_index_pool_basic():
    p = IndexPool(3, "slot")
    a, b, c = p.acquire(), p.acquire(), p.acquire()
    assert sorted([a, b, c]) == [0, 1, 2]
    with pytest.raises(CacheFull):
        p.acquire()
    p.release(b)
    with pytest.raises(CacheMisuse, match="not held"):
        p.release(b)
    with pytest.raises(CacheMisuse, match="does not exist"):
        p.release(7)
    assert p.acquire() == b            # the slot given back is used again
    p.check()


def test_groups_by_need():
    m = manager(window=100, extra={3: StateRequest((4, 2)), 4: None})
    assert len(m.kv_groups) == 2 and len(m.state_groups) == 1
    names = {m.cache_group[c] for c in (0, 1)}
    assert len(names) == 1 and m.cache_group[2] not in names
    assert 4 not in m.cache_group


def test_reserve_commit_release_accounts_pages():
    m = manager(max_tokens=640)                       # 10 pages per group
    s0, s1 = m.acquire(), m.acquire()
    t = m.reserve([(s0, 65), (s1, 1)])
    (g,) = m.kv_groups
    assert [len(r) for r in t[g]] == [2, 1]
    m.commit(t)
    assert m.length(s0) == 65 and m.length(s1) == 1
    m.check()
    t = m.reserve([(s0, 63), (s1, 63)])               # 128 and 64 tokens: still 2 and 1 pages
    assert [len(r) for r in t[g]] == [2, 1]
    m.commit(t)
    t = m.reserve([(s1, 1)])
    assert len(t[g][0]) == 2
    m.commit(t)
    assert m.kv_groups[g].pages.held_count == 4
    m.release(s0)
    assert m.kv_groups[g].pages.held_count == 2
    with pytest.raises(CacheMisuse):
        m.release(s0)
    with pytest.raises(CacheMisuse):
        m.length(s0)
    m.release(s1)
    m.check()
    assert m.kv_groups[g].pages.free_count == 10 and m.slots.free_count == 4


def test_refused_step_changes_nothing():
    m = manager(max_tokens=256)                       # 4 pages
    s0, s1 = m.acquire(), m.acquire()
    m.commit(m.reserve([(s0, 100)]))
    (g,) = m.kv_groups
    before = (m.kv_groups[g].pages.free_count, m.length(s0), m.length(s1))
    with pytest.raises(CacheFull, match="needs 4 more pages"):
        m.reserve([(s0, 29), (s1, 129)])
    assert (m.kv_groups[g].pages.free_count, m.length(s0), m.length(s1)) == before
    with pytest.raises(CacheMisuse, match="twice"):
        m.reserve([(s0, 1), (s0, 1)])
    with pytest.raises(ValueError):
        m.reserve([(s0, 0)])
    m.check()


def test_exact_budget_of_rounded_lengths():
    # three live requests of 1, 64 and 65 tokens need 64 + 64 + 128 tokens and not one more
    m = manager(max_tokens=256, max_seqs=3)
    s = [m.acquire() for _ in range(3)]
    m.commit(m.reserve([(s[0], 1), (s[1], 64), (s[2], 65)]))
    assert m.free_tokens() == 0
    with pytest.raises(CacheFull):
        m.reserve([(s[1], 1)])
    m.commit(m.reserve([(s[0], 63)]))                           # room inside the page it already holds
    m.release(s[2])
    assert m.free_tokens() == 128
    m.check()


def test_window_group_returns_pages_out_of_reach():
    m = manager(max_tokens=64 * 20, window=100)
    s = m.acquire()
    wname = m.cache_group[2]
    m.commit(m.reserve([(s, 300)]))
    # next query at 300 sees keys >= 201: pages 0..2 (positions 0..191) are returned
    assert m.seqs[s].pages[wname][:3] == [None, None, None] and m.seqs[s].pages[wname][3] is not None
    assert m.kv_groups[wname].pages.held_count == 2
    assert m.kv_groups[m.cache_group[0]].pages.held_count == 5
    t = m.reserve([(s, 1)])
    assert len(t[wname][0]) == 5 and t[wname][0][:3] == [0, 0, 0]
    m.commit(t)
    m.check()
    m.release(s)
    m.check()
    assert m.kv_groups[wname].pages.free_count == 20


def test_random_traffic_keeps_the_books():
    """Steps in flight (advanced, not yet confirmed), confirmed oldest first or rolled back newest first, with slots
    released in between: lengths follow the confirmed and pending steps, no page is lost or owned twice."""
    rng = random.Random(0)
    m = manager(max_tokens=64 * 12, max_seqs=5, window=70)
    live = {}                      # slot -> length counting confirmed and pending steps
    pending = []                   # [(reservation, step)] oldest first
    rolled = confirmed = 0
    for _ in range(3000):
        r = rng.random()
        if r < 0.2 and m.slots.free_count:
            live[m.acquire()] = 0
        elif r < 0.3 and live:
            s = rng.choice(list(live))
            m.release(s)           # its pending steps stay in the list: confirm and rollback skip a released sequence
            del live[s]
        elif r < 0.65 and live and len(pending) < 3:
            k = rng.randint(1, len(live))
            step = [(s, rng.choice([1, 1, 1, 5, 64, 130])) for s in rng.sample(list(live), k)]
            try:
                res = m.reserve(step)
            except CacheFull:
                continue
            m.advance(res)
            pending.append((res, step, {s: m.seqs[s] for s, _ in step}))
            for s, n in step:
                live[s] += n
        elif r < 0.9 and pending:
            res, _, _ = pending.pop(0)
            m.confirm(res)
            confirmed += 1
        elif pending:
            while pending:         # a fault: everything in flight is undone, newest first
                res, step, seqs = pending.pop()
                m.rollback(res)
                rolled += 1
                for s, n in step:
                    if s in live and m.seqs.get(s) is seqs[s]:
                        live[s] -= n
        m.check()
        assert {s: m.length(s) for s in live} == live
    while pending:
        m.confirm(pending.pop(0)[0])
    assert rolled > 20 and confirmed > 100
    for s in list(live):
        m.release(s)
    m.check()
    assert all(g.pages.free_count == g.n_pages for g in m.kv_groups.values())


def test_rollback_returns_pages_and_lengths():
    m = manager(max_tokens=640)
    s0, s1 = m.acquire(), m.acquire()
    m.commit(m.reserve([(s0, 60), (s1, 3)]))
    (g,) = m.kv_groups
    free = m.kv_groups[g].pages.free_count
    a = m.reserve([(s0, 10), (s1, 1)])                # s0 takes a second page
    m.advance(a)
    b = m.reserve([(s0, 70)])                         # and a third
    m.advance(b)
    assert m.length(s0) == 140 and m.kv_groups[g].pages.free_count == free - 2
    with pytest.raises(CacheMisuse):
        m.confirm(m.reserve([(s1, 1)]))               # confirming what never advanced
    m.rollback(b)
    assert m.length(s0) == 70 and m.kv_groups[g].pages.free_count == free - 1
    m.rollback(a)
    assert (m.length(s0), m.length(s1)) == (60, 3) and m.kv_groups[g].pages.free_count == free
    with pytest.raises(CacheMisuse):
        m.rollback(a)                                 # once only
    m.check()
