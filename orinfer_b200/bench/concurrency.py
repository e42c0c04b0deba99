"""Concurrent streaming chat requests released together: committed output throughput, TTFT
percentiles and the full-cohort decode window.

Definitions (tools/bench/concurrency.py of the reference): per level N, ``repetitions`` rounds
of N simultaneous streaming requests released by a barrier;
``committed_output_tps = sum(usage.completion_tokens) / round wall`` (queueing, prefill and
HTTP included); ``/health`` is polled every 100 ms and the full-cohort window is the longest
interval with ``active == N`` and ``queued == 0`` (at least 0.2 s); the report keeps the
median round of each level plus every round's numbers.

    python -m orinfer_b200.bench.concurrency --url http://127.0.0.1:8080 --levels 1,8,128
"""

from __future__ import annotations

import argparse
import json
import statistics
import threading
import time

from .http_client import HealthPoller, percentile, stream_chat

LEVELS = (1, 2, 4, 8, 16, 32, 128)
PROMPT = ("Translate the following sentence into Chinese and explain each clause briefly: "
          "the quick brown fox jumps over the lazy dog near the river bank at dawn. ")


def make_body(index: int, prompt_repeat: int, max_tokens: int, seed: int = 20261002) -> dict:
    # a distinct leading tag per request keeps prefix sharing out of the measurement
    text = f"[request {index:04d}] " + PROMPT * prompt_repeat
    return {"messages": [{"role": "user", "content": text}], "max_tokens": max_tokens,
            "temperature": 0, "seed": seed, "ignore_eos": True, "enable_thinking": False}


def run_round(url: str, n: int, prompt_repeat: int, max_tokens: int, timeout: float,
              tag: int = 0) -> dict:
    barrier = threading.Barrier(n + 1)
    results = [None] * n

    def one(i):
        results[i] = stream_chat(url, make_body(tag * 1000 + i, prompt_repeat, max_tokens),
                                 timeout=timeout, release=barrier)

    threads = [threading.Thread(target=one, args=(i,), daemon=True) for i in range(n)]
    with HealthPoller(url) as poller:
        for t in threads:
            t.start()
        barrier.wait()
        t0 = time.perf_counter()
        for t in threads:
            t.join()
        wall = time.perf_counter() - t0
    done = [r for r in results if r and r.ok]
    out_tokens = sum(r.completion_tokens for r in done)
    window = poller.full_cohort_window(n)
    ttfts = [r.ttft_s for r in done]
    return {"n": n, "completed": len(done), "failed": n - len(done),
            "errors": sorted({r.error for r in results if r and r.error})[:3],
            "wall_s": wall, "output_tokens": out_tokens,
            "prompt_tokens": sum(r.prompt_tokens for r in done),
            "committed_output_tps": out_tokens / wall if wall > 0 else 0.0,
            "ttft_p50_s": percentile(ttfts, 50), "ttft_p95_s": percentile(ttfts, 95),
            "latency_p50_s": percentile([r.latency_s for r in done], 50),
            "latency_p95_s": percentile([r.latency_s for r in done], 95),
            "full_cohort_decode_s": (window[1] - window[0]) if window else None,
            "scheduler_delta": poller.counter_delta()}


def run(url: str, levels=LEVELS, repetitions: int = 3, prompt_repeat: int = 4,
        max_tokens: int = 65, timeout: float = 600.0, warmup: bool = True) -> dict:
    report = {"url": url, "max_tokens": max_tokens, "levels": []}
    if warmup:
        run_round(url, 1, prompt_repeat, min(8, max_tokens), timeout, tag=999)
    for n in levels:
        rounds = [run_round(url, n, prompt_repeat, max_tokens, timeout, tag=rep * 7 + n)
                  for rep in range(repetitions)]
        tps = [r["committed_output_tps"] for r in rounds]
        median = sorted(rounds, key=lambda r: r["committed_output_tps"])[len(rounds) // 2]
        report["levels"].append({"n": n, "median": median, "rounds": rounds,
                                 "committed_output_tps_median": statistics.median(tps)})
    return report


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--url", default="http://127.0.0.1:8080")
    ap.add_argument("--levels", default=",".join(map(str, LEVELS)))
    ap.add_argument("--repetitions", type=int, default=3)
    ap.add_argument("--prompt-repeat", type=int, default=4)
    ap.add_argument("--max-tokens", type=int, default=65)
    ap.add_argument("--timeout", type=float, default=600.0)
    ap.add_argument("--output")
    a = ap.parse_args(argv)
    rep = run(a.url, [int(x) for x in a.levels.split(",")], a.repetitions, a.prompt_repeat,
              a.max_tokens, a.timeout)
    text = json.dumps(rep, indent=1)
    if a.output:
        with open(a.output, "w") as f:
            f.write(text)
    for lv in rep["levels"]:
        m = lv["median"]
        print(f"N={lv['n']:4d}  {lv['committed_output_tps_median']:10.1f} tok/s  "
              f"ttft p50 {m['ttft_p50_s']}  p95 {m['ttft_p95_s']}  failed {m['failed']}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
