"""Graph registry (csrc/dist/graph_registry.cpp): LRU pools keyed by geometry, capture at the
threshold-th use, all-rank probe-then-recapture, stale commits, sticky failure.  Ranks are
threads here; no GPU and no real graph is involved (handles are integers)."""
import threading

import pytest

from orinfer_b200.parallel.graph_registry import (CAPTURE, E_STALE, E_TIMEOUT, REPLAY, RUN_DIRECT,
                                                  GraphPool, GraphRegistry, GraphRegistryError,
                                                  key_of)


def test_capture_at_second_use_then_replay():
    reg = GraphRegistry(1, capacity=4, threshold=2)
    k = key_of(((512,), 1, False))
    assert not reg.probe(k)
    d, g, rel, ep = reg.decide(k, False)
    assert (d, g, rel) == (RUN_DIRECT, -1, -1)
    d, g, rel, ep = reg.decide(k, reg.probe(k))
    assert d == CAPTURE
    assert reg.commit(k, 7, ep)
    assert reg.probe(k)
    d, g, rel, ep = reg.decide(k, True)
    assert (d, g) == (REPLAY, 7)
    assert reg.stats()["hits"] == 1 and reg.stats()["captures"] == 1


def test_lru_eviction_hands_the_graph_back():
    reg = GraphRegistry(1, capacity=2, threshold=1)
    keys = [key_of((n,)) for n in (1, 2, 3)]
    for i, k in enumerate(keys[:2]):
        d, _, _, ep = reg.decide(k, False)
        assert d == CAPTURE and reg.commit(k, 10 + i, ep)
    assert reg.decide(keys[0], True)[0] == REPLAY          # key 0 is now the most recent
    d, g, rel, ep = reg.decide(keys[2], False)             # evicts key 1
    assert rel == 11 and d == CAPTURE
    assert not reg.probe(keys[1]) and reg.probe(keys[0])
    assert reg.stats()["evictions"] == 1


def test_a_miss_anywhere_forces_recapture_everywhere():
    reg = GraphRegistry(2, capacity=4, threshold=1)
    k = key_of(("decode", 8))
    for rank in (0, 1):
        d, _, _, ep = reg.decide(k, False, rank)
        assert d == CAPTURE and reg.commit(k, 100 + rank, ep, rank)
    assert reg.probe(k, 0) and reg.probe(k, 1)
    assert reg.evict(k, 1) == 101                           # rank 1 lost its graph
    all_hit = reg.probe(k, 0) and reg.probe(k, 1)
    assert not all_hit
    d0, g0, rel0, ep0 = reg.decide(k, all_hit, 0)
    d1, g1, rel1, ep1 = reg.decide(k, all_hit, 1)
    assert rel0 == 100 and d0 == CAPTURE                    # the hit is invalidated and redone
    assert d1 == CAPTURE and rel1 == -1
    assert reg.stats()["recaptures"] == 1
    # a capture that was started before the invalidation cannot be committed any more
    assert not reg.commit(k, 555, ep0 - 1, 0)
    assert reg.commit(k, 200, ep0, 0) and reg.commit(k, 201, ep1, 1)
    assert reg.decide(k, True, 0)[:2] == (REPLAY, 200)


def test_replay_vote_that_contradicts_a_pool_is_a_sticky_failure():
    reg = GraphRegistry(2, capacity=4, threshold=1)
    k = key_of((1, 2, 3))
    with pytest.raises(GraphRegistryError) as err:
        reg.decide(k, True, 1)                              # "all hit", but rank 1 holds nothing
    assert err.value.code == E_STALE and err.value.rank == 1
    assert reg.status() == E_STALE
    with pytest.raises(GraphRegistryError):
        reg.probe(k, 0)                                     # sticky for everybody


def test_follower_falls_back_and_reports_the_miss():
    lead, follow = GraphPool(4, 1), GraphPool(4, 1)
    geo = ((300,), 1, True)
    d, key, obj, ep = lead.plan(geo)
    assert d == CAPTURE and lead.commit(key, ep, "leader graph")
    fd, fkey, fobj, fep, missed = follow.follow(geo, d)
    assert fd == CAPTURE and not missed and follow.commit(fkey, fep, "follower graph")
    # both replay
    assert lead.plan(geo)[0] == REPLAY
    assert follow.follow(geo, REPLAY)[2] == "follower graph"
    # the follower loses its graph: it runs directly and says so; the leader evicts and the
    # next use goes through trial and capture on both
    follow.evict(fkey)
    d, _, obj, _ = lead.plan(geo)
    assert d == REPLAY and obj == "leader graph"
    fd, _, fobj, fep, missed = follow.follow(geo, d)
    assert fd == RUN_DIRECT and missed and fobj is None
    lead.evict(key)
    assert len(lead) == 0
    d, key, _, ep = lead.plan(geo)
    assert d == CAPTURE                                      # threshold 1: captured again at once
    fd, fkey, _, fep, missed = follow.follow(geo, d)
    assert fd == CAPTURE and not missed


def test_threads_vote_and_a_missing_rank_times_out():
    reg = GraphRegistry(3, capacity=4, threshold=1)
    k = key_of(("v",))
    out = [None] * 3

    def rank(i, hit):
        out[i] = reg.vote(k, hit, i, timeout_ms=5000)
    ts = [threading.Thread(target=rank, args=(i, i != 1)) for i in range(3)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert out == [False, False, False]                     # rank 1 missed
    ts = [threading.Thread(target=rank, args=(i, True)) for i in range(3)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert out == [True, True, True]
    # only two of three ranks arrive: the vote fails closed for both
    errs = []

    def lonely(i):
        try:
            reg.vote(k, True, i, timeout_ms=200)
        except GraphRegistryError as e:
            errs.append(e.code)
    ts = [threading.Thread(target=lonely, args=(i,)) for i in range(2)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert len(errs) == 2 and E_TIMEOUT in errs
    assert reg.status() == E_TIMEOUT


def test_pool_keeps_objects_only_while_the_registry_does():
    pool = GraphPool(capacity=2, threshold=1)
    held = []
    for n in range(3):
        d, key, _, ep = pool.plan((n,))
        assert d == CAPTURE and pool.commit(key, ep, f"g{n}")
        held.append(key)
    assert len(pool) == 2 and set(pool.objects.values()) == {"g1", "g2"}
    pool.clear()
    assert len(pool) == 0 and pool.registry.stats()["entries"] == 0
