"""CPU-side request preparation off the event loop, under a worker and a memory budget.

Rendering the chat template, tokenising, compiling a JSON-schema grammar and decoding inline
media are CPU work that can take milliseconds to seconds; done on the event loop it would stall
every open stream.  ``PreparationPool.run`` executes one preparation on a worker thread after
reserving (a) one of ``workers`` slots and (b) ``estimate(body)`` bytes of ``memory_mib``;
requests wait their turn in arrival order, a cancelled waiter leaves the line, and a request
whose estimate exceeds the whole budget is refused outright (413) instead of waiting forever.
Counterpart of the reference's preparation pool with its memory and worker semaphores and
request-memory estimate (crates/orinfer-api/src/server/preparation.rs:4-180,487-539).
"""

from __future__ import annotations

import asyncio
import json
import time
from collections import deque
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from typing import Any, Callable, Deque, Optional, Tuple

from .chat_codec import RequestError

DEFAULT_WORKERS = 4
DEFAULT_MEMORY_MIB = 1024
# a prepared request holds the body, the rendered prompt and the token ids: a small multiple of
# the JSON size; inline base64 media expands to decoded pixels / samples
TEXT_FACTOR = 6
MEDIA_FACTOR = 4
BASE_BYTES = 64 << 10


def estimate_bytes(body: Any) -> int:
    """Upper estimate of the host memory that preparing ``body`` holds at once."""
    text = media = 0

    def walk(node):
        nonlocal text, media
        if isinstance(node, str):
            if node.startswith("data:") and ";base64," in node[:64]:
                media += len(node) * 3 // 4
            else:
                text += len(node)
        elif isinstance(node, dict):
            for k, v in node.items():
                text += len(k)
                walk(v)
        elif isinstance(node, (list, tuple)):
            for v in node:
                walk(v)
        elif node is not None:
            text += 8

    walk(body)
    return BASE_BYTES + TEXT_FACTOR * text + MEDIA_FACTOR * media


@dataclass
class PreparationStats:
    prepared: int = 0
    refused: int = 0
    cancelled: int = 0
    waited_s: float = 0.0
    busy_s: float = 0.0
    peak_bytes: int = 0
    peak_waiting: int = 0


class PreparationPool:
    def __init__(self, workers: int = DEFAULT_WORKERS, memory_mib: int = DEFAULT_MEMORY_MIB):
        if workers < 1 or memory_mib < 1:
            raise ValueError("preparation pool needs at least one worker and 1 MiB")
        self.workers, self.budget = workers, memory_mib << 20
        self._threads = ThreadPoolExecutor(max_workers=workers, thread_name_prefix="prepare")
        self._line: Deque[Tuple[asyncio.Future, int]] = deque()
        self._running = 0
        self._held = 0
        self.stats = PreparationStats()

    # admission is decided on the event loop only, so no lock is needed
    def _admit(self) -> None:
        while self._line:
            fut, size = self._line[0]
            if fut.cancelled():
                self._line.popleft()
                continue
            if self._running >= self.workers or self._held + size > self.budget:
                return                                  # strict arrival order: no overtaking
            self._line.popleft()
            self._running += 1
            self._held += size
            self.stats.peak_bytes = max(self.stats.peak_bytes, self._held)
            fut.set_result(None)

    async def run(self, fn: Callable[[], Any], size: int,
                  cancelled: Optional[Callable[[], bool]] = None) -> Any:
        """Reserves a worker and ``size`` bytes, runs ``fn()`` on a worker thread, releases."""
        if size > self.budget:
            self.stats.refused += 1
            raise RequestError("request is too large to prepare within the memory budget",
                               status=413, code="request_too_large")
        loop = asyncio.get_running_loop()
        ticket: asyncio.Future = loop.create_future()
        self._line.append((ticket, size))
        self.stats.peak_waiting = max(self.stats.peak_waiting, len(self._line))
        t0 = time.monotonic()
        self._admit()
        try:
            await ticket
        except asyncio.CancelledError:
            if ticket.done() and not ticket.cancelled():   # admitted while being cancelled
                self._release(size)
            else:
                ticket.cancel()
                self._admit()
            self.stats.cancelled += 1
            raise
        t1 = time.monotonic()
        self.stats.waited_s += t1 - t0
        try:
            if cancelled is not None and cancelled():
                self.stats.cancelled += 1
                raise RequestError("request was cancelled", status=499, code="cancelled")
            result = await loop.run_in_executor(self._threads, fn)
            self.stats.prepared += 1
            return result
        finally:
            self.stats.busy_s += time.monotonic() - t1
            self._release(size)

    def _release(self, size: int) -> None:
        self._running -= 1
        self._held -= size
        self._admit()

    def snapshot(self) -> dict:
        s = self.stats
        return {"workers": self.workers, "memory_budget_bytes": self.budget,
                "running": self._running, "waiting": len(self._line), "held_bytes": self._held,
                "prepared": s.prepared, "refused": s.refused, "cancelled": s.cancelled,
                "waited_s": round(s.waited_s, 6), "busy_s": round(s.busy_s, 6),
                "peak_bytes": s.peak_bytes, "peak_waiting": s.peak_waiting}

    def close(self) -> None:
        self._threads.shutdown(wait=False, cancel_futures=True)


def body_size(raw: bytes) -> int:
    """Estimate straight from the wire bytes when the body is not parsed yet."""
    try:
        return estimate_bytes(json.loads(raw))
    except (ValueError, UnicodeDecodeError):
        return BASE_BYTES + TEXT_FACTOR * len(raw)
