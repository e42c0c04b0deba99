"""Preparation pool: worker and memory budgets, arrival order, cancellation, refusal."""
import asyncio
import threading
import time

import pytest

from orinfer_b200.api.chat_codec import RequestError
from orinfer_b200.api.preparation import (BASE_BYTES, PreparationPool, body_size,
                                           estimate_bytes)


def test_estimate_counts_text_and_inline_media():
    small = estimate_bytes({"messages": [{"role": "user", "content": "hi"}]})
    big = estimate_bytes({"messages": [{"role": "user", "content": "x" * 10000}]})
    assert BASE_BYTES < small < big and big - small > 5 * 9000
    img = "data:image/png;base64," + "A" * 40000
    media = estimate_bytes({"messages": [{"role": "user", "content": [
        {"type": "image_url", "image_url": {"url": img}}]}]})
    assert media > BASE_BYTES + 4 * 29000
    assert body_size(b"not json") == BASE_BYTES + 6 * 8
    assert body_size(b'{"a": "bb"}') == estimate_bytes({"a": "bb"})


def test_workers_bound_concurrency_and_order_is_kept():
    async def main():
        pool = PreparationPool(workers=2, memory_mib=64)
        running, peak, order = 0, 0, []
        lock = threading.Lock()

        def work(i):
            nonlocal running, peak
            with lock:
                running += 1
                peak = max(peak, running)
                order.append(i)
            time.sleep(0.03)
            with lock:
                running -= 1
            return i * i

        out = await asyncio.gather(*[pool.run(lambda i=i: work(i), 1 << 20) for i in range(6)])
        pool.close()
        return out, peak, order, pool.snapshot()

    out, peak, order, snap = asyncio.run(main())
    assert out == [0, 1, 4, 9, 16, 25] and peak == 2
    assert sorted(order[:2]) == [0, 1] and sorted(order[2:4]) == [2, 3]
    assert snap["prepared"] == 6 and snap["running"] == 0 and snap["held_bytes"] == 0
    assert snap["peak_waiting"] >= 4


def test_memory_budget_serialises_large_requests_and_refuses_oversized():
    async def main():
        pool = PreparationPool(workers=4, memory_mib=4)
        active, peak = 0, 0
        lock = threading.Lock()

        def work():
            nonlocal active, peak
            with lock:
                active += 1
                peak = max(peak, active)
            time.sleep(0.02)
            with lock:
                active -= 1

        await asyncio.gather(*[pool.run(work, 3 << 20) for _ in range(3)])
        with pytest.raises(RequestError) as e:
            await pool.run(work, 5 << 20)
        pool.close()
        return peak, e.value.status, pool.snapshot()

    peak, status, snap = asyncio.run(main())
    assert peak == 1 and status == 413
    assert snap["refused"] == 1 and snap["peak_bytes"] == 3 << 20


def test_cancelled_waiter_leaves_the_line_and_errors_release_the_slot():
    async def main():
        pool = PreparationPool(workers=1, memory_mib=8)
        gate = threading.Event()
        first = asyncio.create_task(pool.run(gate.wait, 1 << 20))
        await asyncio.sleep(0.01)
        second = asyncio.create_task(pool.run(lambda: "second", 1 << 20))
        third = asyncio.create_task(pool.run(lambda: "third", 1 << 20))
        await asyncio.sleep(0.01)
        second.cancel()
        await asyncio.sleep(0)
        gate.set()
        assert await third == "third"
        await first
        with pytest.raises(ZeroDivisionError):
            await pool.run(lambda: 1 // 0, 1 << 20)
        assert await pool.run(lambda: 7, 1 << 20) == 7
        flagged = pool.run(lambda: 1, 1 << 20, cancelled=lambda: True)
        with pytest.raises(RequestError):
            await flagged
        pool.close()
        return pool.snapshot()

    snap = asyncio.run(main())
    assert snap["cancelled"] == 2 and snap["running"] == 0 and snap["waiting"] == 0
