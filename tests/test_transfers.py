"""Staging ring and input packing (host bookkeeping of uploads)."""
import numpy as np
import pytest

from orinfer_b200.core.transfers import StagingRing, pack_inputs


def test_ring_is_fifo_bounded_and_never_overlaps_live_regions():
    ring = StagingRing(1024, 64)
    rng = np.random.default_rng(0)
    live = []                                                # (ticket, offset, bytes)
    issued = 0
    for step in range(2000):
        want = int(rng.integers(1, 400))
        got = ring.acquire(want)
        if got is None:
            assert live, "an empty ring must accept anything that fits"
            ticket = live[int(rng.integers(0, len(live)))][0]     # stream passed some copy
            retired = ring.retire_through(ticket)
            assert retired == sum(1 for t in live if t[0] <= ticket)
            live = [t for t in live if t[0] > ticket]
            continue
        ticket, off = got
        issued += 1
        assert ticket == issued and off % 64 == 0 and off + want <= 1024
        for _, o, b in live:
            assert off + want <= o or o + b <= off, "overlaps a region still in flight"
        live.append((ticket, off, want))
        assert ring.stats()["live"] == len(live) and ring.stats()["used"] <= 1024
    st = ring.stats()
    assert st["refused"] > 0 and st["peak"] <= 1024
    with pytest.raises(ValueError, match="never fit"):
        ring.acquire(1025)
    with pytest.raises(ValueError, match="never issued"):
        ring.retire_through(10 ** 9)
    with pytest.raises(ValueError):
        StagingRing(1000, 64)
    assert ring.retire_through(issued) == len(live) and ring.stats()["used"] == 0
    assert ring.acquire(1024) == (issued + 1, 0)            # empty ring starts over at zero


def test_packing_keeps_write_order_and_joins_neighbours():
    stage = np.zeros(64, dtype=np.uint8)
    a = np.arange(8, dtype=np.uint8) + 1
    b = np.full(4, 200, dtype=np.uint8)
    ranges = pack_inputs(stage, [(0, a), (4, b), (40, np.int32([7, 9])), (8, b[:2])])
    assert ranges == [(0, 10), (40, 8)]
    assert stage[:10].tolist() == [1, 2, 3, 4, 200, 200, 200, 200, 200, 200]   # later write wins
    assert stage[40:48].view(np.int32).tolist() == [7, 9]
    again = pack_inputs(stage, [(4, a[:4]), (0, b)])                             # reversed order
    assert again == [(0, 8)] and stage[:8].tolist() == [200, 200, 200, 200, 1, 2, 3, 4]
    assert pack_inputs(stage, [(0, a[:2]), (10, a[:2]), (30, a[:2])], merge_gap=8) == \
        [(0, 12), (30, 2)]
    assert pack_inputs(stage, []) == []
    with pytest.raises(ValueError, match="outside"):
        pack_inputs(stage, [(60, a)])
    with pytest.raises(ValueError, match="uint8"):
        pack_inputs(np.zeros(4, np.int32), [])
