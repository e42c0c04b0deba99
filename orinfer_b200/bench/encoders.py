"""Embedding and rerank request throughput on a frozen workload.

Counterpart of the reference's tools/bench/encoders.py: a deterministic set of documents and
queries (generated from a seed, so every run sends the same bytes) is sent to
``POST /v1/embeddings`` and ``POST /v1/rerank`` at a fixed concurrency; reported are requests
per second, prompt tokens per second and latency percentiles per route.

    python -m orinfer_b200.bench.encoders --url http://127.0.0.1:8080 --requests 64
"""

from __future__ import annotations

import argparse
import json
import random
import threading
import time

import requests

from .http_client import percentile

WORDS = ("storage engine index query planner cache page buffer log replica shard vector "
         "token kernel stream tensor matrix scale lattice prefix batch graph").split()


def workload(n: int, seed: int = 20261002, doc_words: int = 64, docs_per_query: int = 8):
    rng = random.Random(seed)
    text = lambda k: " ".join(rng.choice(WORDS) for _ in range(k))
    embed = [{"input": [text(doc_words) for _ in range(4)],
              "input_type": "query" if i % 4 == 0 else "document"} for i in range(n)]
    rerank = [{"query": text(8), "documents": [text(doc_words) for _ in range(docs_per_query)],
               "top_n": 3} for _ in range(n)]
    return embed, rerank


def _drive(url: str, path: str, bodies, concurrency: int, timeout: float) -> dict:
    lock = threading.Lock()
    state = {"next": 0}
    lat, tokens, errors = [], [0], []

    def worker():
        with requests.Session() as s:
            while True:
                with lock:
                    k = state["next"]
                    state["next"] += 1
                if k >= len(bodies):
                    return
                t = time.perf_counter()
                try:
                    r = s.post(url.rstrip("/") + path, json=bodies[k], timeout=timeout)
                    body = r.json()
                    if r.status_code != 200:
                        raise ValueError(json.dumps(body)[:200])
                    with lock:
                        lat.append(time.perf_counter() - t)
                        tokens[0] += body.get("usage", {}).get("prompt_tokens", 0)
                except (requests.RequestException, ValueError) as exc:
                    with lock:
                        errors.append(str(exc)[:200])

    t0 = time.perf_counter()
    threads = [threading.Thread(target=worker, daemon=True) for _ in range(concurrency)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    return {"route": path, "requests": len(bodies), "completed": len(lat), "errors": errors[:3],
            "wall_s": wall, "requests_per_s": len(lat) / wall, "prompt_tps": tokens[0] / wall,
            "latency_p50_s": percentile(lat, 50), "latency_p95_s": percentile(lat, 95)}


def run(url: str, n: int = 64, concurrency: int = 4, seed: int = 20261002,
        doc_words: int = 64, timeout: float = 600.0) -> dict:
    embed, rerank = workload(n, seed, doc_words)
    return {"embeddings": _drive(url, "/v1/embeddings", embed, concurrency, timeout),
            "rerank": _drive(url, "/v1/rerank", rerank, concurrency, timeout)}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--url", default="http://127.0.0.1:8080")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--concurrency", type=int, default=4)
    a = ap.parse_args(argv)
    print(json.dumps(run(a.url, a.requests, a.concurrency), indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
