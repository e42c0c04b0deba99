"""Radix prefix cache (C++ core, CPU)."""
from orinfer_b200.core.prefix import RadixPrefixCache


def _toks(*blocks, p=4):
    out = []
    for b in blocks:
        out += [b * 100 + i for i in range(p)]
    return out


def test_match_insert_share():
    c = RadixPrefixCache(page_tokens=4)
    assert c.match(_toks(1, 2, 3)) == ([], [])
    adopted, ids = c.insert(_toks(1, 2, 3) + [7], [10, 11, 12])
    assert adopted == [True, True, True] and len(ids) == 3
    # an equal prefix is found; a prompt must keep at least one token to run
    n, pages = c.match(_toks(1, 2, 3), limit_tokens=11)
    assert pages == [10, 11]
    n2, pages2 = c.match(_toks(1, 2, 9, 9))
    assert pages2 == [10, 11]
    # inserting an existing prefix adopts nothing new
    adopted, _ = c.insert(_toks(1, 2, 4), [20, 21, 22])
    assert adopted == [False, False, True]
    st = c.statistics()
    assert st.device_pages == 4 and st.nodes == 4 and st.lookups == 3 and st.hit_rate > 0


def test_eviction_respects_users_and_leaves():
    c = RadixPrefixCache(page_tokens=4)
    c.insert(_toks(1, 2), [1, 2])
    c.insert(_toks(1, 3), [1, 3])
    ids, pages = c.match(_toks(1, 2))            # acquires nodes of path 1-2
    victims = c.evict(10)
    assert [p for _, p in victims] == [3]        # only the unused leaf goes
    c.release(ids)
    victims = c.evict(10)
    assert [p for _, p in victims] == [2, 1]     # leaf first, then its parent
    assert c.statistics().nodes == 0


def test_utility_prefers_popular_and_recent():
    c = RadixPrefixCache(page_tokens=4)
    c.insert(_toks(1), [1])
    c.insert(_toks(2), [2])
    for _ in range(5):
        ids, _ = c.match(_toks(2))
        c.release(ids)
    assert c.evict(1) == [(1, 1)]


def test_abandoned_matches_do_not_count_as_hits():
    # a request that waits for pages matches on every admission attempt; those matches must
    # not make its prefix look more popular than one that was really used
    c = RadixPrefixCache(page_tokens=4)
    c.insert(_toks(1), [1])
    c.insert(_toks(2), [2])
    c.insert(_toks(3), [3])
    for _ in range(3):
        ids, _ = c.match(_toks(1))
        c.release(ids)                           # prefix 1: three real uses
    for _ in range(6):
        ids, _ = c.match(_toks(2))
        c.abandon(ids)                           # prefix 2: six retries, never used
    held, _ = c.match(_toks(3))                  # prefix 3 stays in use: not evictable
    for _ in range(90):                          # time passes, so that age no longer decides
        c.match(_toks(3), acquire=False)
    assert c.evict(1) == [(2, 2)]                # with the retries counted, 1 would go first
    assert c.evict(1) == [(1, 1)]                # abandon dropped the users as well
    assert c.evict(1) == []
    c.release(held)


def test_host_tier_roundtrip():
    c = RadixPrefixCache(page_tokens=4)
    c.insert(_toks(1, 2), [5, 6])
    victims = c.evict(2, to_host=True)
    assert [p for _, p in victims] == [6, 5]
    # until the host copy is registered, the nodes are not matchable
    assert c.match(_toks(1, 2)) == ([], [])
    for i, (nid, _) in enumerate(victims):
        c.set_host(nid, 100 + i)
    ids, pages = c.match(_toks(1, 2), acquire=False)
    assert pages == [-1, -1] and c.host_handle(ids[0]) == 101
    assert c.restore(ids[0], 9)
    assert c.match(_toks(1, 2), acquire=False)[1] == [9, -1]
    assert c.drop_host(5) == [100]
    st = c.statistics()
    assert st.offloaded == 2 and st.restored == 1


def test_media_hash_separates_equal_tokens():
    c = RadixPrefixCache(page_tokens=4)
    c.insert(_toks(1), [1], media=[111])
    assert c.match(_toks(1), media=[222]) == ([], [])
    assert c.match(_toks(1), media=[111])[1] == [1]
