"""Tunes the tensor-core GEMM's launch variants on the device it runs on.

    python -m orinfer_b200.tuning.gemm_tuner --model qwen3.5-4b-class --out table.json
    python -m orinfer_b200.tuning.gemm_tuner --shape q4:19456:2560 --rows 512,2048

For every projection shape of the model (or ``--shape fmt:N:K``) and every row bucket
(9..16, 17..32, ... up to ``--max-rows``) the tuner times the launch heuristics and every
valid (M-tile factor, weight-tile width, K splits) candidate at the bucket's upper edge, with
weights cycled through more copies than fit in L2 and the launches inside one CUDA graph
(device time without host launch gaps).  A candidate enters the table when it beats the
heuristics by more than ``--margin``.  Results of all candidates are integers times the same
scales, so every candidate is also checked bit for bit against the heuristic launch before it
may win.  Offline projection tuner of the reference: python/orinfer_build/tuning/.
"""

from __future__ import annotations

import argparse
import itertools
import json
import sys
from typing import Dict, List, Tuple

import torch

from ..config import PRESETS, ModelConfig
from . import tables
from .tables import GemmVariant

BUCKETS = [16, 32, 64, 128, 256, 384, 512, 768, 1024, 1536, 2048, 3072, 4096, 6144, 8192]


def model_shapes(cfg: ModelConfig, tp: int = 1) -> List[Tuple[str, int, int]]:
    """(format, N, K) of every projection GEMM a forward pass of ``cfg`` launches."""
    h = cfg.hidden
    shapes = set()
    qkv = cfg.q_dim + 2 * cfg.kv_dim
    shapes.add((cfg.attn_format, qkv // tp, h))
    shapes.add((cfg.attn_format, h, cfg.q_heads * cfg.head_dim // tp))
    if cfg.ffn:
        shapes.add((cfg.proj_format, 2 * cfg.ffn // tp, h))
        shapes.add((cfg.proj_format, h, cfg.ffn // tp))
    if cfg.shared_expert_ffn:
        shapes.add((cfg.proj_format, 2 * cfg.shared_expert_ffn, h))
        shapes.add((cfg.proj_format, h, cfg.shared_expert_ffn))
    if cfg.arch == "hybrid":
        d = cfg.gdn_head_dim
        conv = (2 * cfg.gdn_k_heads + cfg.gdn_v_heads) * d
        shapes.add((cfg.proj_format, (conv + cfg.gdn_v_heads * d) // tp, h))
        shapes.add((cfg.proj_format, h, cfg.gdn_v_heads * d // tp))
    return sorted(s for s in shapes if s[1] % 8 == 0 and s[2] % 128 == 0)


def candidates(fmt: str, m: int, n: int, k: int) -> List[GemmVariant]:
    out = []
    for mt, nb, splits in itertools.product((1, 2, 4), (128, 64, 32), (1, 2, 3, 4, 6, 8)):
        if mt > 1 and m <= 128 * (mt // 2):
            continue                              # a tile factor whose extra rows are all padding
        v = GemmVariant(fmt, n, k, m, m, mt, nb, splits)
        if not v.problems():
            out.append(v)
    return out


def bucket_ranges(max_rows: int, rows=None) -> List[Tuple[int, int]]:
    edges = sorted(rows) if rows else [b for b in BUCKETS if b <= max_rows]
    lo, out = 9, []                               # rows 1..8 run on the SIMT kernel
    for hi in edges:
        if hi >= lo:
            out.append((lo, hi))
            lo = hi + 1
    return out


def tune_shape(fmt: str, n: int, k: int, ranges, iters: int, margin: float, dev, log=None
               ) -> List[GemmVariant]:
    from ..ops import functional as F
    from ..ops import native
    from ..bench import kernel_probe as KP
    lib = native.lib()
    wbytes = n * k * {"w8": 1.0, "q4": 0.5, "q2": 0.25}[fmt]
    copies = max(2, int(256e6 // wbytes) + 1)
    ws = KP.weights(fmt, n, k, dev, copies)
    sw = (torch.rand(n, device=dev) * 0.01).half()
    KP.GRAPH = True
    chosen = []
    for lo, hi in ranges:
        m = hi
        a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev)
        sa = torch.rand(m, device=dev) * 0.01
        out = torch.empty(m, n, dtype=torch.float16, device=dev)
        run = lambda i: F.qgemm(a, sa, ws[i % copies], sw, fmt, n, out=out, path=2)
        lib.orinfer_qgemm_clear_variants()
        run(0)
        want = out.clone()
        base = KP.timed(run, iters)
        best, best_t = None, base
        for c in candidates(fmt, m, n, k):
            lib.orinfer_qgemm_clear_variants()
            tables.apply([c], lib)
            out.zero_()
            run(0)
            if not torch.equal(out, want):
                raise RuntimeError(f"variant {c} changed the result of the GEMM")
            t = KP.timed(run, iters)
            if t < best_t:
                best, best_t = c, t
        lib.orinfer_qgemm_clear_variants()
        line = {"fmt": fmt, "n": n, "k": k, "rows": [lo, hi], "us_default": base * 1e6}
        if best is not None and best_t < base * (1.0 - margin):
            v = GemmVariant(fmt, n, k, lo, hi, best.mt, best.nb, best.splits, best_t * 1e6,
                            base * 1e6)
            chosen.append(v)
            line.update(us=best_t * 1e6, mt=v.mt, nb=v.nb, splits=v.splits)
        if log is not None:
            print(json.dumps(line), file=log, flush=True)
    return chosen


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", action="append", default=[], choices=sorted(PRESETS))
    ap.add_argument("--shape", action="append", default=[], help="fmt:N:K")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--max-rows", type=int, default=8192)
    ap.add_argument("--rows", default="", help="comma-separated bucket edges (default: built in)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--margin", type=float, default=0.03)
    ap.add_argument("--out", default="")
    ap.add_argument("--merge", default="", help="existing table whose other shapes are kept")
    a = ap.parse_args(argv)
    from ..ops import native
    dev = torch.device("cuda:0")
    native.init()
    shapes = set()
    for name in a.model:
        shapes.update(model_shapes(PRESETS[name], a.tp))
    for s in a.shape:
        fmt, n, k = s.split(":")
        shapes.add((fmt, int(n), int(k)))
    if not shapes:
        ap.error("give --model or --shape")
    rows = [int(x) for x in a.rows.split(",") if x]
    ranges = bucket_ranges(a.max_rows, rows)
    found: Dict[tuple, GemmVariant] = {}
    if a.merge:
        for v in tables.parse(open(a.merge).read()):
            if (v.fmt, v.n, v.k) not in shapes:
                found[(v.fmt, v.n, v.k, v.m_lo)] = v
    for fmt, n, k in sorted(shapes):
        for v in tune_shape(fmt, n, k, ranges, a.iters, a.margin, dev, log=sys.stderr):
            found[(v.fmt, v.n, v.k, v.m_lo)] = v
    text = tables.dump(tables.merge_ranges(found.values()), torch.cuda.get_device_name(0))
    tables.parse(text)                              # the table must load
    if a.out:
        with open(a.out, "w") as f:
            f.write(text)
    else:
        sys.stdout.write(text)
    if native.read_status():
        raise SystemExit("kernel status word set")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
