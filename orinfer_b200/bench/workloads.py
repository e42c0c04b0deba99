"""Scenario benchmarks over the chat route: cold injection into warm streams, fixed-arrival
replay, bounded acceptance workloads and output stress with a repetition detector.

They restate, against this server, what the reference's tools/bench/mixed.py (arrival gaps of
warm streams while a cold prompt prefills), scheduling.py (requests sent at fixed ``at_s``
offsets whatever the completions do), acceptance.py (heterogeneous bounded workloads with
``expected_words`` checks) and output_stress.py (``contains`` / ``json_equals`` checks and a
long-cycle repetition detector) measure.
"""

from __future__ import annotations

import argparse
import json
import threading
import time

from .http_client import percentile, stream_chat


def _chat(text, max_tokens, **extra):
    return dict({"messages": [{"role": "user", "content": text}], "max_tokens": max_tokens,
                 "temperature": 0, "enable_thinking": False}, **extra)


def mixed(url: str, warm: int = 4, warm_tokens: int = 256, cold_words: int = 1500,
          inject_after_s: float = 0.5, timeout: float = 600.0) -> dict:
    """``warm`` decoding streams, then one cold request with a long prompt.  Reports the
    largest arrival gap each warm stream saw inside the cold request's prefill interval
    (send -> first output) against its gaps outside it."""
    results = [None] * warm
    barrier = threading.Barrier(warm + 1)

    def stream(i):
        results[i] = stream_chat(url, _chat(f"[warm {i}] Count upwards from one in words.",
                                            warm_tokens, ignore_eos=True),
                                 timeout=timeout, release=barrier)

    threads = [threading.Thread(target=stream, args=(i,), daemon=True) for i in range(warm)]
    for t in threads:
        t.start()
    barrier.wait()
    time.sleep(inject_after_s)
    cold = stream_chat(url, _chat("[cold] " + "lorem ipsum dolor sit amet " * (cold_words // 5),
                                  8, ignore_eos=True), timeout=timeout)
    for t in threads:
        t.join()
    lo, hi = cold.start, cold.first_output or cold.end
    inside, outside = [], []
    for r in results:
        if r is None:
            continue
        for a, b in zip(r.arrivals, r.arrivals[1:]):
            (inside if (b >= lo and a <= hi) else outside).append(b - a)
    return {"warm": warm, "cold_prompt_tokens": cold.prompt_tokens, "cold_ttft_s": cold.ttft_s,
            "cold_ok": cold.ok, "warm_ok": sum(1 for r in results if r and r.ok),
            "gap_inside_max_s": max(inside) if inside else None,
            "gap_inside_p50_s": percentile(inside, 50),
            "gap_outside_p50_s": percentile(outside, 50),
            "gap_outside_p95_s": percentile(outside, 95)}


def scheduling(url: str, arrivals, timeout: float = 600.0) -> dict:
    """Replay ``arrivals`` = [{"at_s": t, "prompt": str, "max_tokens": n}, ...]: each request
    is sent at its offset from the start whether or not earlier ones have finished."""
    t0 = time.perf_counter()
    results = [None] * len(arrivals)

    def one(i, item):
        delay = item["at_s"] - (time.perf_counter() - t0)
        if delay > 0:
            time.sleep(delay)
        sent = time.perf_counter() - t0
        r = stream_chat(url, _chat(item["prompt"], item.get("max_tokens", 32), ignore_eos=True),
                        timeout=timeout)
        results[i] = (sent, r)

    threads = [threading.Thread(target=one, args=(i, it), daemon=True)
               for i, it in enumerate(arrivals)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    rows = [{"at_s": it["at_s"], "sent_s": s, "send_lag_s": s - it["at_s"], "ok": r.ok,
             "ttft_s": r.ttft_s, "latency_s": r.latency_s, "completion_tokens": r.completion_tokens}
            for it, (s, r) in zip(arrivals, results)]
    return {"wall_s": wall, "requests": rows,
            "output_tps": sum(x["completion_tokens"] for x in rows) / wall,
            "ttft_p50_s": percentile([x["ttft_s"] for x in rows], 50),
            "ttft_p95_s": percentile([x["ttft_s"] for x in rows], 95)}


def check_output(text: str, spec: dict):
    """Failures of ``text`` against a check spec: ``expected_words`` / ``contains`` (all must
    appear, case-insensitive), ``json_equals`` (text parses to that value), ``max_cycle``
    (no long repeated cycle)."""
    bad = []
    low = text.lower()
    for w in list(spec.get("expected_words") or []) + list(spec.get("contains") or []):
        if w.lower() not in low:
            bad.append(f"missing {w!r}")
    if "json_equals" in spec:
        try:
            if json.loads(text) != spec["json_equals"]:
                bad.append("json differs")
        except ValueError:
            bad.append("not json")
    if spec.get("max_cycle", True):
        cyc = repeated_cycle(text)
        if cyc:
            bad.append(f"repeats a {cyc[0]}-character cycle {cyc[1]} times")
    return bad


def repeated_cycle(text: str, min_period: int = 16, max_period: int = 400, min_repeats: int = 4):
    """Long-cycle repetition detector: the tail of ``text`` consisting of one block of
    ``min_period..max_period`` characters repeated at least ``min_repeats`` times.  Returns
    (period, repeats) or None.  Short periods (counting, punctuation runs) are not flagged."""
    n = len(text)
    for period in range(1, min(max_period, n // min_repeats) + 1):
        block = text[n - period:]
        reps, pos = 1, n - 2 * period
        while pos >= 0 and text[pos:pos + period] == block:
            reps += 1
            pos -= period
        if reps >= min_repeats:     # the smallest period decides: a short one is not a fault
            return (period, reps) if period >= min_period else None
    return None


def acceptance(url: str, workload, timeout: float = 600.0) -> dict:
    """Bounded heterogeneous workload: items ``{"at_s", "prompt", "max_tokens", checks...}``;
    passes when every request completes and every check holds."""
    t0 = time.perf_counter()
    out = [None] * len(workload)

    def one(i, item):
        delay = item.get("at_s", 0.0) - (time.perf_counter() - t0)
        if delay > 0:
            time.sleep(delay)
        body = _chat(item["prompt"], item.get("max_tokens", 64))
        body.update(item.get("body") or {})
        r = stream_chat(url, body, timeout=timeout)
        out[i] = {"ok": r.ok, "error": r.error, "finish_reason": r.finish_reason,
                  "failures": check_output(r.text, item) if r.ok else ["request failed"],
                  "completion_tokens": r.completion_tokens, "ttft_s": r.ttft_s}

    threads = [threading.Thread(target=one, args=(i, it), daemon=True)
               for i, it in enumerate(workload)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    return {"wall_s": time.perf_counter() - t0, "requests": out,
            "passed": all(r["ok"] and not r["failures"] for r in out)}


def output_stress(url: str, items, duration_s: float = 30.0, concurrency: int = 4,
                  timeout: float = 600.0) -> dict:
    """For ``duration_s`` keep ``concurrency`` requests in flight, cycling through ``items``
    (prompt + checks) and letting each run to its natural end of sequence."""
    deadline = time.perf_counter() + duration_s
    lock = threading.Lock()
    state = {"next": 0, "done": 0, "tokens": 0, "failures": []}

    def worker():
        while time.perf_counter() < deadline:
            with lock:
                k = state["next"]
                state["next"] += 1
            item = items[k % len(items)]
            r = stream_chat(url, _chat(item["prompt"], item.get("max_tokens", 512)), timeout=timeout)
            bad = check_output(r.text, item) if r.ok else [r.error or "failed"]
            with lock:
                state["done"] += 1
                state["tokens"] += r.completion_tokens
                if bad:
                    state["failures"].append({"item": k % len(items), "failures": bad})

    t0 = time.perf_counter()
    threads = [threading.Thread(target=worker, daemon=True) for _ in range(concurrency)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    return {"wall_s": wall, "completed": state["done"], "output_tps": state["tokens"] / wall,
            "failures": state["failures"], "passed": not state["failures"]}


def main(argv=None):
    ap = argparse.ArgumentParser(description="scenario benchmarks against a running server")
    ap.add_argument("scenario", choices=["mixed", "scheduling", "acceptance", "output-stress"])
    ap.add_argument("--url", default="http://127.0.0.1:8080")
    ap.add_argument("--workload", help="JSON file: list of items (scheduling / acceptance / stress)")
    ap.add_argument("--warm", type=int, default=4)
    ap.add_argument("--duration", type=float, default=30.0)
    ap.add_argument("--concurrency", type=int, default=4)
    a = ap.parse_args(argv)
    items = json.load(open(a.workload)) if a.workload else None
    if a.scenario == "mixed":
        rep = mixed(a.url, warm=a.warm)
    elif a.scenario == "scheduling":
        rep = scheduling(a.url, items)
    elif a.scenario == "acceptance":
        rep = acceptance(a.url, items)
    else:
        rep = output_stress(a.url, items, a.duration, a.concurrency)
    print(json.dumps(rep, indent=1))
    return 0 if rep.get("passed", True) else 1


if __name__ == "__main__":
    raise SystemExit(main())
