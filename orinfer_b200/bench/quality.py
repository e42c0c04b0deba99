"""Paired next-token probes: how far a candidate scorer (a quantised build, a new kernel, a
different parallel layout) moves the next-token distribution of a baseline on identical
teacher-forced histories.

A *probe* is one position of one case: the context hash, the reference token and its log
probability, the scorer's top-3 and any extra log probabilities that were asked for.  The
candidate must report its probability for each of the baseline's top-3 ids (queried, never
assumed zero).  ``analyze`` pairs the two sides and reports top-1 agreement, top-3 overlap,
mean absolute probability / log-probability error on the baseline's top-3, the change in
target NLL, and disagreement rates on high-confidence (p >= 0.8) and low-margin (gap <= 0.01)
positions.  Definitions follow the reference's tools/eval/quick_quality.py and
crates/orinfer-engine/src/runtime/scoring.rs:1-50 (full-vocabulary normalisation, greedy
selection with lower-id tie breaking, seed 20261002); it is a local probability diagnostic,
not a task benchmark.

    orinfer score-model MODEL --tokens 1,2,3 --jsonl base.jsonl
    orinfer score-model OTHER --tokens 1,2,3 --jsonl cand.jsonl --query-from base.jsonl
    orinfer bench quality --baseline base.jsonl --candidate cand.jsonl
"""

from __future__ import annotations

import argparse
import hashlib
import json
import math
import statistics
from collections import defaultdict
from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np

SEED = 20261002


class ProbeError(ValueError):
    pass


def context_sha256(tokens: Sequence[int]) -> str:
    return hashlib.sha256(np.asarray(tokens, dtype="<u4").tobytes()).hexdigest()


def log_softmax(row: np.ndarray) -> np.ndarray:
    v = np.asarray(row, dtype=np.float64)
    m = v.max()
    return v - (m + math.log(np.exp(v - m).sum()))


def top3_of(logp: np.ndarray) -> List[dict]:
    """Three most likely ids, ties to the lower id."""
    order = np.lexsort((np.arange(logp.size), -logp))[:3]
    return [{"token_id": int(i), "logprob": float(logp[i])} for i in order]


def probes_from_logits(logits: np.ndarray, tokens: Sequence[int], case_id: str,
                       mode: str = "prefill", query: Optional[Dict[int, List[int]]] = None
                       ) -> List[dict]:
    """``logits[i]`` is the distribution after ``tokens[:i + 1]``; one probe per position with
    a next token.  ``query[position]`` lists extra ids whose log probability is reported."""
    out = []
    for i in range(len(tokens) - 1):
        lp = log_softmax(logits[i])
        pos = i + 1
        ids = (query or {}).get(pos, [])
        out.append({"seed": SEED, "case_id": case_id, "execution_mode": mode, "position": pos,
                    "context_sha256": context_sha256(tokens[:pos]),
                    "reference_token_id": int(tokens[pos]),
                    "reference_logprob": float(lp[tokens[pos]]),
                    "top3": top3_of(lp),
                    "logprobs": {str(int(t)): float(lp[t]) for t in ids}})
    return out


def queries_from(probes: Iterable[dict]) -> Dict[int, List[int]]:
    """Ids a candidate must score: the baseline's top-3 at every position."""
    return {p["position"]: [t["token_id"] for t in p["top3"]] for p in probes}


def _check_top3(items) -> List[dict]:
    if len(items) != 3 or len({t["token_id"] for t in items}) != 3:
        raise ProbeError("exactly three distinct top ids are required")
    for t in items:
        if not math.isfinite(t["logprob"]) or t["logprob"] > 1e-9:
            raise ProbeError("top-3 entries need full-vocabulary log probabilities")
    if sum(math.exp(t["logprob"]) for t in items) > 1.00001:
        raise ProbeError("probabilities must use the full-vocabulary normalisation")
    return sorted(items, key=lambda t: (-t["logprob"], t["token_id"]))


def pair(baseline: Iterable[dict], candidate: Iterable[dict]) -> List[dict]:
    cand = {(p["case_id"], p["execution_mode"], p["position"]): p for p in candidate}
    rows, seen = [], set()
    for b in baseline:
        key = (b["case_id"], b["execution_mode"], b["position"])
        if key in seen:
            raise ProbeError("duplicate scoring position")
        seen.add(key)
        c = cand.get(key)
        if c is None:
            raise ProbeError(f"candidate has no probe for {key}")
        if b["seed"] != SEED or c["seed"] != SEED or \
                b["context_sha256"] != c["context_sha256"]:
            raise ProbeError("seed or history mismatch: the probes cannot be paired")
        rows.append({"key": key, "baseline": b, "candidate": c})
    return rows


def analyze(rows: List[dict]) -> dict:
    groups = defaultdict(list)
    for r in rows:
        b, c = r["baseline"], r["candidate"]
        a3, c3 = _check_top3(b["top3"]), _check_top3(c["top3"])
        base_ids = [t["token_id"] for t in a3]
        known = dict(c["logprobs"])
        known.update({str(t["token_id"]): t["logprob"] for t in c3})
        if any(str(i) not in known for i in base_ids):
            raise ProbeError("candidate did not report a baseline top-3 id; query it, never "
                             "fill it with zero")
        vals = [known[str(i)] for i in base_ids]
        if any(not math.isfinite(v) or v > 1e-9 for v in vals) or \
                sum(math.exp(v) for v in vals) > 1.00001:
            raise ProbeError("invalid candidate log probabilities")
        for v in (b["reference_logprob"], c["reference_logprob"]):
            if not math.isfinite(v) or v > 1e-9:
                raise ProbeError("invalid teacher-forced target score")
        selected = c3[0]["token_id"]
        p1, p2 = math.exp(a3[0]["logprob"]), math.exp(a3[1]["logprob"])
        groups[r["key"][:2]].append({
            "top1_agreement": float(selected == base_ids[0]),
            "selected_in_baseline_top3": float(selected in base_ids),
            "top3_overlap": len(set(base_ids) & {t["token_id"] for t in c3}) / 3,
            "mean_abs_probability_error": statistics.mean(
                abs(math.exp(t["logprob"]) - math.exp(v)) for t, v in zip(a3, vals)),
            "mean_abs_logprob_error": statistics.mean(
                abs(t["logprob"] - v) for t, v in zip(a3, vals)),
            "delta_target_nll": b["reference_logprob"] - c["reference_logprob"],
            "high_confidence": p1 >= 0.8, "low_margin": p1 - p2 <= 0.01})
    if not groups:
        raise ProbeError("no scoring records")

    def summarise(values):
        keys = ("top1_agreement", "selected_in_baseline_top3", "top3_overlap",
                "mean_abs_probability_error", "mean_abs_logprob_error", "delta_target_nll")
        sure = [v for v in values if v["high_confidence"]]
        close = [v for v in values if v["low_margin"]]
        return dict(
            positions=len(values), **{k: statistics.mean(v[k] for v in values) for k in keys},
            high_confidence_positions=len(sure),
            high_confidence_top1_disagreement=(
                statistics.mean(1 - v["top1_agreement"] for v in sure) if sure else None),
            low_margin_positions=len(close),
            low_margin_top1_disagreement=(
                statistics.mean(1 - v["top1_agreement"] for v in close) if close else None))

    return {"seed": SEED,
            "aggregate": summarise([v for g in groups.values() for v in g]),
            "by_case_and_mode": [dict(case_id=k[0], execution_mode=k[1], **summarise(v))
                                 for k, v in sorted(groups.items())]}


def read_jsonl(path) -> List[dict]:
    with open(path) as f:
        return [json.loads(line) for line in f if line.strip()]


def write_jsonl(path, probes: Iterable[dict]) -> None:
    with open(path, "w") as f:
        for p in probes:
            f.write(json.dumps(p) + "\n")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--baseline", required=True)
    ap.add_argument("--candidate", required=True)
    ap.add_argument("--min-top1", type=float, default=None,
                    help="exit 1 when aggregate top-1 agreement falls below this")
    a = ap.parse_args(argv)
    rep = analyze(pair(read_jsonl(a.baseline), read_jsonl(a.candidate)))
    print(json.dumps(rep, indent=1))
    if a.min_top1 is not None and rep["aggregate"]["top1_agreement"] < a.min_top1:
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
