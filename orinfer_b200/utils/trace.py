"""Tracing hooks: NVTX ranges, device-timed spans and one-line JSON traces.

Three switches, all off by default and free when off:

* ``ORINFER_NVTX=1`` - ``span(name)`` pushes an NVTX range (visible to Nsight tools), one per
  layer block of the model runner and per engine phase.
* ``ORINFER_SPAN_PROFILE=1`` - the same spans are bracketed by CUDA events on the current
  stream; ``report()`` synchronises once and returns count / total / mean device time per
  span name.  The engine prints it as ``SPANS {json}`` at shutdown.  Do not combine with
  CUDA-graph capture (events recorded during capture cannot be timed): spans opened while a
  stream is capturing are skipped.
* ``ORINFER_TRACE=a,b`` - ``line(topic, **fields)`` prints ``TOPIC {json}`` to stderr for the
  listed topics (``prefill_choose``, ``admit``, ``mtp``, ``layered``; ``all`` for every one).

The reference exposes the same kinds of evidence: scheduler statistics on ``/health`` and as
``SCHEDULER {json}`` at exit (crates/orinfer-api/src/server/continuous.rs:1003-1008), env
traces (``ORINFER_MTP_TRACE``, ``PREFILL_CHOOSE`` lines, runtime/requests.rs:1971-1976),
NVTX ranges per plan operation in its diagnostics build (runtime/requests/profile.rs:49-80)
and CUDA-event timing of the decode graph (backend/cuda/executor/graph_profile.rs:28-60).
"""

from __future__ import annotations

import contextlib
import json
import os
import sys
import threading
from typing import Dict, List, Tuple

_lock = threading.Lock()
_pending: List[Tuple[str, object, object]] = []        # (name, start event, end event)
_totals: Dict[str, List[float]] = {}                    # name -> [count, total ms]


def _flag(name: str) -> bool:
    return os.environ.get(name, "") not in ("", "0")


def nvtx_enabled() -> bool:
    return _flag("ORINFER_NVTX")


def profile_enabled() -> bool:
    return _flag("ORINFER_SPAN_PROFILE")


def topics() -> set:
    return {t.strip() for t in os.environ.get("ORINFER_TRACE", "").split(",") if t.strip()}


def enabled(topic: str) -> bool:
    ts = topics()
    return bool(ts) and ("all" in ts or topic in ts)


def line(topic: str, **fields) -> None:
    """``TOPIC {json}`` on stderr when the topic is traced."""
    if enabled(topic):
        print(f"{topic.upper()} {json.dumps(fields, sort_keys=True, default=str)}",
              file=sys.stderr, flush=True)


_null = contextlib.nullcontext()


def span(name: str):
    """Context manager around a stretch of launches on the current stream."""
    if not (nvtx_enabled() or profile_enabled()):
        return _null
    return _Span(name)


class _Span:
    __slots__ = ("name", "start", "pushed")

    def __init__(self, name: str):
        self.name, self.start, self.pushed = name, None, False

    def __enter__(self):
        import torch
        if not torch.cuda.is_available():
            return self
        if nvtx_enabled():
            torch.cuda.nvtx.range_push(self.name)
            self.pushed = True
        if profile_enabled() and not torch.cuda.is_current_stream_capturing():
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *exc):
        import torch
        if self.start is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            with _lock:
                _pending.append((self.name, self.start, end))
                overflow = len(_pending) > 65536
            if overflow:
                collect()
        if self.pushed:
            torch.cuda.nvtx.range_pop()
        return False


def collect() -> None:
    """Folds finished spans into the totals (synchronises the device once)."""
    with _lock:
        batch, _pending[:] = list(_pending), []
    if not batch:
        return
    import torch
    torch.cuda.synchronize()
    with _lock:
        for name, start, end in batch:
            slot = _totals.setdefault(name, [0, 0.0])
            slot[0] += 1
            slot[1] += start.elapsed_time(end)


def add(name: str, ms: float, count: int = 1) -> None:
    """Adds a host-measured duration to the same table (used off the GPU and in tests)."""
    with _lock:
        slot = _totals.setdefault(name, [0, 0.0])
        slot[0] += count
        slot[1] += ms


def report(reset: bool = False) -> Dict[str, dict]:
    """name -> {count, total_ms, mean_us, share}, ordered by total time."""
    collect()
    with _lock:
        items = sorted(_totals.items(), key=lambda kv: -kv[1][1])
        grand = sum(v[1] for _, v in items) or 1.0
        out = {k: {"count": int(v[0]), "total_ms": round(v[1], 3),
                   "mean_us": round(1e3 * v[1] / max(v[0], 1), 2),
                   "share": round(v[1] / grand, 4)} for k, v in items}
        if reset:
            _totals.clear()
    return out


def dump(prefix: str = "SPANS") -> None:
    rep = report()
    if rep:
        print(f"{prefix} {json.dumps(rep)}", file=sys.stderr, flush=True)
