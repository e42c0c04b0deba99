"""Prefill and decode rates over HTTP with exact token counts: token-id prompts through
``POST /v1/completions`` with ``ignore_eos``.

Definitions are the ones of the reference's headline table (docs/performance.md:42-53, harness
crates/orinfer-engine/src/runtime/requests/tests/benchmark.rs:22-170):
``prefill_tps = input_tokens / time_to_first_token`` (request set-up, head and sampling
included) and ``decode_tps = subsequently committed tokens / decode wall``; single-request rows
use 512 or 8192 input tokens and 257 output tokens, multi-request rows 256 in / 65 out per
request; the median of the measured runs after one warm-up is reported.  Prompts are seeded
random ids below ``--vocab`` and differ per request, so the prefix cache cannot help.

    python -m orinfer_b200.bench.token_bench --url http://127.0.0.1:8080 --input 512 --output 257
"""

from __future__ import annotations

import argparse
import json
import random
import statistics
import threading
import time

import requests

SEED = 20261002


def one(url: str, ids, output_tokens: int, timeout: float = 600.0, release=None) -> dict:
    body = {"prompt": ids, "max_tokens": output_tokens, "temperature": 0, "seed": SEED,
            "ignore_eos": True, "stream": True, "stream_options": {"include_usage": True},
            "cache_prompt": False, "return_token_ids": True}
    if release is not None:
        release.wait()
    t0 = time.perf_counter()
    first = last = None
    usage, error = {}, ""
    try:
        with requests.post(url.rstrip("/") + "/v1/completions", json=body, stream=True,
                           timeout=timeout) as r:
            if r.status_code != 200:
                return {"ok": False, "error": r.text[:300]}
            for raw in r.iter_lines():
                if not raw.startswith(b"data: ") or raw == b"data: [DONE]":
                    continue
                now = time.perf_counter()
                ev = json.loads(raw[6:])
                if "error" in ev:
                    error = json.dumps(ev["error"])[:300]
                    continue
                first = first or now            # the first token's own chunk
                last = now
                usage = ev.get("usage") or usage
    except requests.RequestException as e:
        return {"ok": False, "error": str(e)[:300]}
    end = time.perf_counter()
    n_in, n_out = usage.get("prompt_tokens", len(ids)), usage.get("completion_tokens", 0)
    ttft = (first or end) - t0
    decode_wall = end - (first or end)
    return {"ok": not error and n_out > 0, "error": error, "input_tokens": n_in,
            "output_tokens": n_out, "ttft_s": ttft, "latency_s": end - t0,
            "prefill_tps": n_in / ttft if ttft > 0 else None,
            "decode_tps": (n_out - 1) / decode_wall if decode_wall > 0 and n_out > 1 else None}


def prompts(count: int, input_tokens: int, vocab: int, seed: int = SEED):
    rng = random.Random(seed)
    return [[rng.randrange(1, vocab) for _ in range(input_tokens)] for _ in range(count)]


def run(url: str, input_tokens: int = 512, output_tokens: int = 257, concurrency: int = 1,
        runs: int = 3, vocab: int = 256, warmup: int = 1) -> dict:
    rounds = []
    for rnd in range(warmup + runs):
        batch = prompts(concurrency, input_tokens, vocab, SEED + rnd)
        barrier = threading.Barrier(concurrency + 1)
        out = [None] * concurrency

        def go(i):
            out[i] = one(url, batch[i], output_tokens, release=barrier)

        threads = [threading.Thread(target=go, args=(i,), daemon=True) for i in range(concurrency)]
        for t in threads:
            t.start()
        barrier.wait()
        t0 = time.perf_counter()
        for t in threads:
            t.join()
        wall = time.perf_counter() - t0
        if rnd < warmup:
            continue
        ok = [r for r in out if r and r["ok"]]
        first_done = max((r["ttft_s"] for r in ok), default=None)
        total_out = sum(r["output_tokens"] for r in ok)
        rounds.append({
            "wall_s": wall, "failed": concurrency - len(ok),
            "errors": sorted({r["error"] for r in out if r and r.get("error")})[:2],
            "prefill_tps": (sum(r["input_tokens"] for r in ok) / first_done) if first_done else None,
            "decode_tps": ((total_out - len(ok)) / (wall - first_done))
            if first_done and wall > first_done and total_out > len(ok) else None,
            "committed_output_tps": total_out / wall if wall > 0 else None,
            "requests": out})

    def med(key):
        vals = [r[key] for r in rounds if r[key] is not None]
        return statistics.median(vals) if vals else None

    return {"url": url, "input_tokens": input_tokens, "output_tokens": output_tokens,
            "concurrency": concurrency, "runs": runs, "prefill_tps": med("prefill_tps"),
            "decode_tps": med("decode_tps"), "committed_output_tps": med("committed_output_tps"),
            "failed": sum(r["failed"] for r in rounds), "rounds": rounds}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--url", default="http://127.0.0.1:8080")
    ap.add_argument("--input", type=int, default=512)
    ap.add_argument("--output", type=int, default=257)
    ap.add_argument("--concurrency", type=int, default=1)
    ap.add_argument("--runs", type=int, default=3)
    ap.add_argument("--vocab", type=int, default=256, help="prompt ids are drawn below this")
    a = ap.parse_args(argv)
    rep = run(a.url, a.input, a.output, a.concurrency, a.runs, a.vocab)
    rep.pop("rounds")
    print(json.dumps(rep, indent=1))
    return 1 if rep["failed"] else 0


if __name__ == "__main__":
    raise SystemExit(main())
