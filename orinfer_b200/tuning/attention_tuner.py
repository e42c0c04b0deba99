"""Tunes the key-axis split count of decode attention on the device it runs on.

    python -m orinfer_b200.tuning.attention_tuner --model qwen3.5-4b-class --out table.json
    python -m orinfer_b200.tuning.attention_tuner --qh 32 --kvh 8 --d 128 --rows 1,8 --ctx 512,8192

For every (row bucket, context bucket) it times the heuristic split count of
``ops.functional.attention_splits`` and every candidate (1, 2, 3, 4, 6, 8, 12, 16, 24, 32 that
leaves at least 64 keys per split), launches inside one CUDA graph, and writes an
``attention`` entry when a candidate beats the heuristic by more than ``--margin``.  ``--merge``
keeps the ``gemm`` entries of an existing table.  Every candidate's output is compared with the
unsplit kernel's before it may win.  Counterpart of the reference's auxiliary tuners
(python/orinfer_build/tuning/).
"""

from __future__ import annotations

import argparse
import json
import sys
from typing import List, Tuple

from . import tables
from .tables import AttentionSplit

ROW_BUCKETS = [(1, 1), (2, 2), (3, 4), (5, 8), (9, 16), (17, 32), (33, 64), (65, 128)]
CTX_BUCKETS = [(129, 512), (513, 2048), (2049, 8192), (8193, 32768)]
CANDIDATES = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32)


def candidates(ctx: int) -> List[int]:
    """Split counts worth timing at a context of ``ctx`` keys."""
    return [s for s in CANDIDATES if s == 1 or (ctx + s - 1) // s >= 64]


def buckets(rows: List[int], ctxs: List[int]) -> List[Tuple[Tuple[int, int], Tuple[int, int]]]:
    """The (row range, context range) cells containing the requested points; every cell is
    timed at its upper edge."""
    cells = []
    for rb in ROW_BUCKETS:
        if rows and not any(rb[0] <= r <= rb[1] for r in rows):
            continue
        for cb in CTX_BUCKETS:
            if ctxs and not any(cb[0] <= c <= cb[1] for c in ctxs):
                continue
            cells.append((rb, cb))
    return cells


def choose(times: dict, default_splits: int, margin: float) -> Tuple[int, float, float]:
    """(best split count, its time, the heuristic's time); the heuristic keeps a cell unless a
    candidate is faster by more than ``margin``."""
    base = times[default_splits]
    best = min(times, key=lambda s: (times[s], s))
    if times[best] < base * (1.0 - margin):
        return best, times[best], base
    return default_splits, base, base


def measure(rows: int, ctx: int, qh: int, kvh: int, d: int, iters: int, dev) -> dict:
    """Split count -> seconds per launch (graph-timed), for every candidate and the heuristic."""
    import torch

    from ..bench import kernel_probe
    from ..ops import functional as F
    from ..ops import native
    per = (ctx + 127) // 128
    pages = rows * per
    table = torch.arange(1, pages + 1, dtype=torch.int32, device=dev).view(rows, per)
    kc = torch.randint(-127, 128, (pages + 1, 128, kvh, d), dtype=torch.int8, device=dev)
    vc = torch.randint(-127, 128, (pages + 1, 128, kvh, d), dtype=torch.int8, device=dev)
    ks = (torch.rand(pages + 1, 128, kvh, d // 64, device=dev) * 0.02).half()
    vs = (torch.rand(pages + 1, 128, kvh, d // 64, device=dev) * 0.02).half()
    q = torch.randn(rows, qh, d, device=dev).half()
    row_req = torch.arange(rows, dtype=torch.int32, device=dev)
    row_pos = torch.full((rows,), ctx - 1, dtype=torch.int32, device=dev)
    saved = list(tables.ATTENTION)
    tables.set_attention([])                         # the heuristic, not an older table
    default = F.attention_splits(ctx, rows, kvh)
    tables.set_attention(saved)
    want = F.attention(q, None, row_req, row_pos, table, kc, vc, ks, vs, splits=1).float()
    kernel_probe.GRAPH = True
    times = {}
    for s in sorted(set(candidates(ctx)) | {default}):
        need = native.lib().orinfer_attention_scratch_bytes(rows, qh, d, s)
        scratch = torch.empty(max(need // 4, 1), dtype=torch.float32, device=dev)
        out = torch.empty(rows, qh * d, dtype=torch.float16, device=dev)
        run = lambda i: F.attention(q, None, row_req, row_pos, table, kc, vc, ks, vs, splits=s,
                                    scratch=scratch, out=out)
        run(0)
        torch.cuda.synchronize()
        if float((out.float() - want).abs().max()) > 2e-2 * max(1.0, float(want.abs().max())):
            continue                                   # a split count that changes the result
        times[s] = kernel_probe.timed(run, iters)
    times["default"] = default
    return times


def main(argv=None) -> int:
    from ..config import PRESETS
    ap = argparse.ArgumentParser(prog="orinfer_b200.tuning.attention_tuner", description=__doc__)
    ap.add_argument("--model", choices=sorted(PRESETS), default=None)
    ap.add_argument("--qh", type=int, default=32)
    ap.add_argument("--kvh", type=int, default=8)
    ap.add_argument("--d", type=int, default=128)
    ap.add_argument("--rows", default="", help="comma-separated row counts (default: all buckets)")
    ap.add_argument("--ctx", default="", help="comma-separated contexts (default: all buckets)")
    ap.add_argument("--margin", type=float, default=0.03)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--merge", default=None, help="existing table whose gemm entries are kept")
    ap.add_argument("--out", default="-")
    a = ap.parse_args(argv)
    import torch
    if not torch.cuda.is_available():
        print("the attention tuner measures on a GPU", file=sys.stderr)
        return 2
    from ..ops import native
    dev = torch.device("cuda", 0)
    native.init()
    if a.model:
        cfg = PRESETS[a.model]
        a.qh, a.kvh, a.d = cfg.q_heads, cfg.kv_heads, cfg.head_dim
    ints = lambda text: [int(x) for x in text.split(",") if x]
    entries: List[AttentionSplit] = []
    for (r_lo, r_hi), (c_lo, c_hi) in buckets(ints(a.rows), ints(a.ctx)):
        times = measure(r_hi, c_hi, a.qh, a.kvh, a.d, a.iters, dev)
        default = times.pop("default")
        best, t_best, t_base = choose(times, default, a.margin)
        print(f"rows {r_lo}-{r_hi} ctx {c_lo}-{c_hi}: heuristic {default} splits "
              f"{t_base * 1e6:.1f} us, best {best} splits {t_best * 1e6:.1f} us", file=sys.stderr)
        if best != default:
            entries.append(AttentionSplit(r_lo, r_hi, c_lo, c_hi, a.kvh, best, t_best * 1e6,
                                          t_base * 1e6))
    doc = {"schema": tables.SCHEMA, "device": torch.cuda.get_device_name(0), "gemm": []}
    if a.merge:
        doc["gemm"] = json.loads(open(a.merge).read()).get("gemm", [])
    doc["attention"] = tables.dump_attention(entries)
    text = json.dumps(doc, indent=1) + "\n"
    if a.out == "-":
        sys.stdout.write(text)
    else:
        open(a.out, "w").write(text)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
