"""Prometheus text metrics with the reference's metric names
(crates/orinfer-api/src/server/metrics.rs:23-56,90-204)."""

from __future__ import annotations

import threading
from typing import Dict, List

BUCKETS = [0.005, 0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1, 2.5, 5, 10, 30, 60, 120]
HISTOGRAMS = ["queue", "prefill", "decode", "finalize", "time_to_first_token", "latency",
              "prefix_restore", "prefix_store"]


class Metrics:
    def __init__(self):
        self._lock = threading.Lock()
        self.hist: Dict[str, List[int]] = {h: [0] * (len(BUCKETS) + 1) for h in HISTOGRAMS}
        self.sum: Dict[str, float] = {h: 0.0 for h in HISTOGRAMS}
        self.count: Dict[str, int] = {h: 0 for h in HISTOGRAMS}
        self.counters: Dict[str, float] = {
            "prompt_tokens_total": 0, "completion_tokens_total": 0, "cached_tokens_total": 0,
            "requests_total": 0, "request_errors_total": 0, "compute_seconds_total": 0.0,
            "admission_seconds_total": 0.0,
            # the reference's spellings of the token counters and of its failure, planning,
            # cache and reclaim counters (server/metrics.rs:90-235)
            "generated_tokens_total": 0, "cached_prompt_tokens_total": 0,
            "sampling_request_failures_total": 0, "batch_plan_seconds_total": 0.0,
            "prefix_cache_evictions_total": 0, "prefix_cache_host_evictions_total": 0,
            "prefix_restore_seconds_total": 0.0, "program_reclaims_total": 0}
        self.gauges: Dict[str, float] = {"requests_running": 0, "requests_waiting": 0,
                                         "backend_healthy": 1,
                                         "prefix_cache_device_entries": 0,
                                         "prefix_cache_device_bytes": 0,
                                         "prefix_cache_host_entries": 0,
                                         "prefix_cache_host_bytes": 0}

    def level(self, name: str, value: float) -> None:
        """A counter whose source keeps the running total itself (engine statistics)."""
        with self._lock:
            self.counters[name] = max(self.counters.get(name, 0), value)

    def observe(self, name: str, seconds: float) -> None:
        with self._lock:
            idx = next((i for i, b in enumerate(BUCKETS) if seconds <= b), len(BUCKETS))
            self.hist[name][idx] += 1
            self.sum[name] += seconds
            self.count[name] += 1

    def add(self, name: str, value: float = 1) -> None:
        with self._lock:
            self.counters[name] = self.counters.get(name, 0) + value

    def set(self, name: str, value: float) -> None:
        with self._lock:
            self.gauges[name] = value

    def render(self) -> str:
        out = []
        with self._lock:
            for h in HISTOGRAMS:
                name = f"orinfer_request_{h}_seconds"
                out.append(f"# TYPE {name} histogram")
                acc = 0
                for b, n in zip(BUCKETS, self.hist[h]):
                    acc += n
                    out.append(f'{name}_bucket{{le="{b}"}} {acc}')
                acc += self.hist[h][-1]
                out.append(f'{name}_bucket{{le="+Inf"}} {acc}')
                out.append(f"{name}_sum {self.sum[h]}")
                out.append(f"{name}_count {self.count[h]}")
            for k, v in self.counters.items():
                out.append(f"# TYPE orinfer_{k} counter")
                out.append(f"orinfer_{k} {v}")
            for k, v in self.gauges.items():
                out.append(f"# TYPE orinfer_{k} gauge")
                out.append(f"orinfer_{k} {v}")
        return "\n".join(out) + "\n"
