"""Conditional-memory host side: n-gram addressing, shards, gather plans, row stores."""
import numpy as np
import pytest

from orinfer_b200.core.host_rows import (ConditionalMemory, HashLayer, HostRowError, Int8RowStore,
                                         NgramHasher, RowPlan, dequant_rows, row_shard,
                                         write_int8_table)


def hasher(heads=1, primes=(5, 7, 9), rows=21):
    return NgramHasher(list(range(16)), 0, [14, 15], heads,
                       [HashLayer(1, rows, [1, 3, 5, 7], list(primes))])


def test_addresses_depend_only_on_committed_history():
    h = hasher()
    seq = [1, 2, 3, 4, 5, 6]
    whole, _ = h.hash([], seq)
    a, _ = h.hash([], seq[:2])
    b, _ = h.hash(seq[:2], seq[2:])
    assert np.array_equal(np.concatenate([a, b]), whole)          # chunked prefill
    h.hash([1, 2], [9, 10, 11])                                    # a rejected branch
    assert np.array_equal(h.hash([1, 2], [3, 4])[0], whole[2:4])   # leaves no trace
    assert np.array_equal(h.hash([99 % 16, 1, 2, 3], [4])[0], h.hash([1, 2, 3], [4])[0])


def test_barriers_and_bucket_offsets():
    h = hasher()
    ids, valid = h.hash([], [1, 2, 14, 3])
    assert valid.tolist() == [True, True, False, True]
    flat = ids.reshape(4, -1)
    # values worked by hand from the layout: window (1, pad, pad, pad) with pad id 0
    assert flat[0].tolist() == [1, 6, 13]
    assert flat[1].tolist() == [1, 6, 13]            # 2 xor 3*1 == 1
    assert flat[2].tolist() == [0, 0, 0]
    assert np.array_equal(flat[3], h.hash([], [3])[0].reshape(-1))   # nothing crosses the barrier
    # python restatement of the rolling hash, with negative products and floor modulo
    h2 = NgramHasher([7, 3, 9, 11], 0, [], 2,
                     [HashLayer(0, 5 + 7 + 11 + 13 + 17 + 19, [3, 5, 7, 9], [5, 7, 11, 13, 17, 19]),
                      HashLayer(4, 12, [1, 1, 1, 1], [2, 2, 2, 2, 2, 2])])
    ids, _ = h2.hash([1], [2, 3])
    tm = [7, 3, 9, 11]
    window = [tm[3], tm[2], tm[1], tm[0]]             # token 3, then 2, then history 1, then pad
    rolling = window[0] * 3
    expect, offset = [], 0
    primes = [5, 7, 11, 13, 17, 19]
    for shift in (1, 2, 3):
        rolling ^= window[shift] * (5, 7, 9)[shift - 1]
        for head in range(2):
            p = primes[(shift - 1) * 2 + head]
            expect.append(rolling % p + sum(primes[:(shift - 1) * 2 + head]))
    assert ids[1, 0].reshape(-1).tolist() == expect
    assert ids.shape == (2, 2, 3, 2)


def test_malformed_layouts_and_tokens_are_refused():
    with pytest.raises(HostRowError):
        hasher(rows=22)                                # buckets do not sum to the rows
    with pytest.raises(HostRowError):
        NgramHasher(list(range(4)), 0, [], 1, [HashLayer(0, 21, [1, 2, 5, 7], [5, 7, 9])])  # even
    with pytest.raises(HostRowError):
        NgramHasher(list(range(4)), 9, [], 1, [HashLayer(0, 21, [1, 3, 5, 7], [5, 7, 9])])
    with pytest.raises(HostRowError):
        hasher().hash([], [16])
    with pytest.raises(HostRowError):
        hasher().hash([77], [1])


def test_shards_cover_the_table_once():
    for rows, ranks in ((10, 4), (8, 8), (3, 8), (1000003, 8)):
        spans = [row_shard(rows, ranks, r) for r in range(ranks)]
        assert sum(c for _, c in spans) == rows
        for (f0, c0), (f1, _) in zip(spans, spans[1:]):
            assert f0 + c0 == f1 or c0 == 0 or f1 == rows
    assert row_shard(10, 4, 3) == (9, 1) and row_shard(3, 8, 5) == (3, 0)
    with pytest.raises(HostRowError):
        row_shard(10, 4, 4)


def test_plan_groups_unique_rows_by_owner_and_restores_order():
    ids = [17, 3, 17, 9, 0, 3, 19]
    plan = RowPlan.build(ids, table_rows=20, ranks=4)              # span 5
    assert plan.starts.tolist() == [0, 2, 3, 3, 5]
    assert plan.for_rank(0).tolist() == [3, 0] and plan.for_rank(1).tolist() == [9]
    assert plan.for_rank(2).tolist() == [] and plan.for_rank(3).tolist() == [17, 19]
    assert plan.rows[plan.restore].tolist() == ids
    with pytest.raises(HostRowError):
        RowPlan.build([20], 20, 4)
    with pytest.raises(HostRowError):
        RowPlan.build([-1], 20, 4)
    with pytest.raises(HostRowError):
        RowPlan.build([1, 2, 3], 20, 4, max_queries=2)
    assert RowPlan.build([], 20, 4).rows.size == 0


def test_row_store_cache_resident_and_bounds(tmp_path):
    rng = np.random.default_rng(0)
    table = rng.standard_normal((257, 48)).astype(np.float32)
    path = tmp_path / "rows.bin"
    row_bytes = write_int8_table(path, table)
    assert row_bytes == 50
    raw = np.fromfile(path, dtype=np.uint8).reshape(257, row_bytes)
    plain = Int8RowStore(path, row_bytes, 257)
    ids = [5, 200, 5, 256, 0]
    assert np.array_equal(plain.gather(ids), raw[ids])
    assert np.abs(dequant_rows(plain.gather(ids)) - table[ids]).max() < 0.03
    cached = Int8RowStore(path, row_bytes, 257, cache_bytes=4096 + 66 * 64)
    assert cached.cache_slots == 64
    for _ in range(3):
        assert np.array_equal(cached.gather(ids), raw[ids])
    st = cached.stats()
    assert st["misses"] == 4 and st["hits"] == 11 and st["gathered_rows"] == 15
    sweep = np.arange(257)
    assert np.array_equal(cached.gather(sweep), raw)                # evictions keep bytes right
    assert np.array_equal(cached.gather(sweep[::-1]), raw[::-1])
    assert Int8RowStore(path, row_bytes, 257, cache_bytes=100).cache_slots == 0
    res = Int8RowStore(path, row_bytes, 257, resident_budget=1 << 20)
    assert res.resident and np.array_equal(res.gather(ids), raw[ids])
    assert res.stats()["resident_bytes"] == 257 * row_bytes
    res.close()
    with pytest.raises(HostRowError, match="budget"):
        Int8RowStore(path, row_bytes, 257, resident_budget=100)
    with pytest.raises(HostRowError, match="shorter"):
        Int8RowStore(path, row_bytes, 258)
    shard = Int8RowStore(path, row_bytes, 57, first_row=200, data_offset=200 * row_bytes)
    assert np.array_equal(shard.gather([200, 256]), raw[[200, 256]])
    with pytest.raises(HostRowError, match="outside"):
        shard.gather([199])
    with pytest.raises(HostRowError, match="byte budget"):
        plain.gather(ids, max_bytes=100)


def test_sharded_lookup_equals_whole_table_lookup(tmp_path):
    rng = np.random.default_rng(1)
    primes = [11, 13, 17, 19, 23, 29]
    rows = sum(primes)
    table = rng.standard_normal((rows, 16)).astype(np.float32)
    whole = tmp_path / "t.bin"
    rb = write_int8_table(whole, table)
    h = NgramHasher(list(range(32)), 0, [31], 2, [HashLayer(2, rows, [3, 5, 7, 9], primes)])
    one = ConditionalMemory(h, [[Int8RowStore(whole, rb, rows)]])
    stores = []
    for r in range(4):
        first, count = row_shard(rows, 4, r)
        stores.append(Int8RowStore(whole, rb, count, first_row=first, data_offset=first * rb,
                                   cache_bytes=1 << 16))
    four = ConditionalMemory(h, [stores])
    tokens = [4, 9, 31, 9, 4, 9, 4, 9]
    a, va = one.lookup([1, 2, 3], tokens)
    b, vb = four.lookup([1, 2, 3], tokens)
    assert a.shape == (8, 1, 6, 16) and np.array_equal(a, b) and np.array_equal(va, vb)
    assert not va[2] and np.all(a[2] == 0) and np.any(a[3] != 0)
