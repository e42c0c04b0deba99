"""One streaming chat request measured from the client side, plus small statistics helpers.

The reference's bench tools share the same three observations per request
(tools/bench/concurrency.py: first output, completion, usage); ``StreamResult`` holds them.
"""

from __future__ import annotations

import json
import threading
import time
from dataclasses import dataclass, field

import requests


@dataclass
class StreamResult:
    ok: bool = False
    status: int = 0
    error: str = ""
    start: float = 0.0            # time.perf_counter() at send
    first_output: float = 0.0     # first non-empty text / reasoning / tool delta
    first_event: float = 0.0      # first chunk after the role chunk (may be the finish chunk)
    end: float = 0.0
    arrivals: list = field(default_factory=list)   # perf_counter of every content chunk
    text: str = ""
    reasoning: str = ""
    tool_calls: list = field(default_factory=list)
    finish_reason: str = ""
    prompt_tokens: int = 0
    completion_tokens: int = 0
    cached_tokens: int = 0

    @property
    def ttft_s(self):
        """Time to the first non-empty delta; a reply without any visible output (random-init
        weights emitting unprintable tokens) falls back to its first event after the role
        chunk."""
        mark = self.first_output or self.first_event
        return (mark - self.start) if mark else None

    @property
    def latency_s(self):
        return self.end - self.start

    def gaps(self):
        return [b - a for a, b in zip(self.arrivals, self.arrivals[1:])]


def _delta_has_output(delta: dict) -> bool:
    if delta.get("content") or delta.get("reasoning_content") or delta.get("reasoning"):
        return True
    return any((c.get("function") or {}).get("arguments") or (c.get("function") or {}).get("name")
               for c in delta.get("tool_calls") or [])


def stream_chat(base_url: str, body: dict, timeout: float = 600.0, session=None,
                release: threading.Barrier | None = None) -> StreamResult:
    """POST a streaming chat completion and record arrival times.  ``release`` (a barrier) is
    waited on just before the request is sent, so a cohort starts together."""
    body = dict(body, stream=True)
    body.setdefault("stream_options", {"include_usage": True})
    http = session or requests
    res = StreamResult()
    if release is not None:
        release.wait()
    res.start = time.perf_counter()
    try:
        import os
        key = os.environ.get("ORINFER_API_KEY")
        with http.post(base_url.rstrip("/") + "/v1/chat/completions", json=body, stream=True,
                       timeout=timeout,
                       headers={"Authorization": "Bearer " + key} if key else None) as r:
            res.status = r.status_code
            if r.status_code != 200:
                res.error = r.text[:500]
                res.end = time.perf_counter()
                return res
            for raw in r.iter_lines():
                if not raw or not raw.startswith(b"data: "):
                    continue
                now = time.perf_counter()
                payload = raw[6:]
                if payload == b"[DONE]":
                    break
                chunk = json.loads(payload)
                if "error" in chunk:
                    res.error = json.dumps(chunk["error"])[:500]
                    continue
                usage = chunk.get("usage")
                if usage:
                    res.prompt_tokens = usage.get("prompt_tokens", 0)
                    res.completion_tokens = usage.get("completion_tokens", 0)
                    res.cached_tokens = (usage.get("prompt_tokens_details") or {}).get(
                        "cached_tokens", 0)
                for choice in chunk.get("choices") or []:
                    delta = choice.get("delta") or {}
                    if not res.first_event and delta.get("role") is None:
                        res.first_event = now
                    if _delta_has_output(delta):
                        if not res.first_output:
                            res.first_output = now
                        res.arrivals.append(now)
                    res.text += delta.get("content") or ""
                    res.reasoning += delta.get("reasoning_content") or delta.get("reasoning") or ""
                    for call in delta.get("tool_calls") or []:
                        res.tool_calls.append(call)
                    if choice.get("finish_reason"):
                        res.finish_reason = choice["finish_reason"]
            if res.tool_calls:                       # streamed fragments -> whole calls
                from ..api.output_parser import merge_tool_calls
                res.tool_calls = merge_tool_calls([dict(c, index=c.get("index", 0))
                                                   for c in res.tool_calls])
            res.ok = not res.error
    except requests.RequestException as exc:
        res.error = f"{type(exc).__name__}: {exc}"[:500]
    res.end = time.perf_counter()
    return res


def percentile(values, q: float):
    """Nearest-rank percentile (q in 0..100) of a non-empty list; None when empty."""
    vals = sorted(v for v in values if v is not None)
    if not vals:
        return None
    k = max(0, min(len(vals) - 1, int(-(-q * len(vals) // 100)) - 1))
    return vals[k]


class HealthPoller:
    """Samples ``GET /health`` every ``period`` seconds on a thread; each sample keeps the
    time, ``active``, ``queued`` and the scheduler counters."""

    def __init__(self, base_url: str, period: float = 0.1):
        self.url = base_url.rstrip("/") + "/health"
        self.period = period
        self.samples = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        with requests.Session() as s:
            while not self._stop.is_set():
                t = time.perf_counter()
                try:
                    h = s.get(self.url, timeout=5).json()
                    self.samples.append((t, h.get("active", 0), h.get("queued", 0),
                                         h.get("scheduler") or {}))
                except (requests.RequestException, ValueError):
                    pass
                self._stop.wait(max(0.0, self.period - (time.perf_counter() - t)))

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def full_cohort_window(self, n: int, minimum: float = 0.2):
        """Longest run of consecutive samples with ``active == n`` and ``queued == 0``:
        (start, end) or None when shorter than ``minimum`` seconds."""
        best, run_start, prev = None, None, None
        for t, active, queued, _ in self.samples + [(float("inf"), -1, 0, {})]:
            if active == n and queued == 0:
                run_start = t if run_start is None else run_start
                prev = t
            elif run_start is not None:
                if best is None or prev - run_start > best[1] - best[0]:
                    best = (run_start, prev)
                run_start = None
        return best if best and best[1] - best[0] >= minimum else None

    def counter_delta(self):
        """Numeric scheduler counters: last sample minus first."""
        if len(self.samples) < 2:
            return {}
        a, b = self.samples[0][3], self.samples[-1][3]
        return {k: b[k] - a[k] for k in b
                if isinstance(b.get(k), (int, float)) and isinstance(a.get(k), (int, float))}
