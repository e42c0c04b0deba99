"""Micro-benchmarks of single kernels with CUDA-event timing and roofline fractions.

    python -m orinfer_b200.bench.kernel_probe gemm --m 512 --n 19456 --k 2560 --fmt q4
    python -m orinfer_b200.bench.kernel_probe attn --tokens 2048
    python -m orinfer_b200.bench.kernel_probe gemm --m 1 --n 19456 --k 2560 --fmt q4
    python -m orinfer_b200.bench.kernel_probe attn-decode --rows 1 --ctx 512
    python -m orinfer_b200.bench.kernel_probe act-prep --rows 1 --k 2560

Each run does warm-up launches, then times ``--iters`` launches between two events on
the launching stream (synchronised on both sides); with ``--rotate`` buffers larger than
L2 are cycled so every launch reads its operands from HBM.  Peaks come from
``MEASURED_PEAKS.json`` at the repository root when present.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from ..ops import functional as F
from ..ops import native

ROOT = Path(__file__).resolve().parents[2]


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


GRAPH = False


def timed(fn, iters, warm=3):
    for _ in range(warm):
        fn(0)
    torch.cuda.synchronize()
    if GRAPH:
        # one graph holding `iters` launches: removes host launch overhead from the timing
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters * 1e-3
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e-3


def weights(fmt, n, k, dev, copies):
    out = []
    for _ in range(copies):
        if fmt == "w8":
            c = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=dev)
        elif fmt == "q4":
            c = torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 128, n, 16), dtype=torch.int64,
                              device=dev).to(torch.int32)
        else:
            c = torch.randint(-2 ** 15, 2 ** 15 - 1, (k // 128, n, 16), dtype=torch.int64,
                              device=dev).to(torch.int16)
        out.append(c)
    return out


def gemm(args, dev):
    m, n, k = args.m, args.n, args.k
    wbytes = n * k * {"w8": 1.0, "q4": 0.5, "q2": 0.25}[args.fmt]
    copies = max(1, int(256e6 // wbytes) + 1) if args.rotate else 1
    ws = weights(args.fmt, n, k, dev, copies)
    a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev)
    sa = torch.rand(m, device=dev) * 0.01
    sw = (torch.rand(n, device=dev) * 0.01).half()
    out = torch.empty(m, n, dtype=torch.float16, device=dev)
    path = {"auto": 0, "simt": 1, "tc": 2}[args.path]
    native.qgemm_set_impl(args.impl)
    if args.probe:
        native.lib().orinfer_qgemm_set_probe(args.probe)
    t = timed(lambda i: F.qgemm(a, sa, ws[i % copies], sw, args.fmt, n, out=out, path=path),
              args.iters)
    hbm, flops, tag = peaks()
    ops = 2.0 * m * n * k
    byts = wbytes + m * k + m * n * 2
    print(json.dumps({"kernel": "qgemm", "impl": args.impl, "probe": args.probe, "fmt": args.fmt, "m": m, "n": n, "k": k,
                      "us": t * 1e6,
                      "tops": ops / t / 1e12, "gbs": byts / t / 1e9,
                      "frac_int8_peak": ops / t / (2 * flops), "frac_hbm": byts / t / hbm,
                      "peaks": tag, "int8_peak_assumed": "2 x bf16 cuBLAS burst"}))


def attn(args, dev):
    qh, kvh, d, n = args.qh, args.kvh, args.d, args.tokens
    pages = (n + 127) // 128
    table = torch.arange(1, pages + 1, dtype=torch.int32, device=dev).view(1, -1)
    kc = torch.randint(-127, 128, (pages + 1, 128, kvh, d), dtype=torch.int8, device=dev)
    vc = torch.randint(-127, 128, (pages + 1, 128, kvh, d), dtype=torch.int8, device=dev)
    ks = (torch.rand(pages + 1, 128, kvh, d // 64, device=dev) * 0.02).half()
    vs = (torch.rand(pages + 1, 128, kvh, d // 64, device=dev) * 0.02).half()
    q = torch.randn(n, qh, d, device=dev).half()
    out = torch.empty(n, qh * d, dtype=torch.float16, device=dev)
    chunks = torch.tensor([[0, n, 0, 0]], dtype=torch.int32, device=dev)
    t = timed(lambda i: F.attention_prefill(q, None, chunks, n, table, kc, vc, ks, vs, out=out),
              args.iters)
    _, flops, tag = peaks()
    ops = 4.0 * qh * d * n * (n + 1) / 2
    print(json.dumps({"kernel": "attention_prefill", "tokens": n, "qh": qh, "kvh": kvh, "d": d,
                      "us": t * 1e6, "tflops_causal": ops / t / 1e12,
                      "frac_f16_peak": ops / t / flops, "peaks": tag}))


def attn_decode(args, dev):
    """Row attention (decode steps): ``rows`` requests, each one query row over ``ctx`` keys."""
    qh, kvh, d, rows, ctx = args.qh, args.kvh, args.d, args.rows, args.ctx
    per = (ctx + 127) // 128
    pages = rows * per
    table = torch.arange(1, pages + 1, dtype=torch.int32, device=dev).view(rows, per)
    kc = torch.randint(-127, 128, (pages + 1, 128, kvh, d), dtype=torch.int8, device=dev)
    vc = torch.randint(-127, 128, (pages + 1, 128, kvh, d), dtype=torch.int8, device=dev)
    ks = (torch.rand(pages + 1, 128, kvh, d // 64, device=dev) * 0.02).half()
    vs = (torch.rand(pages + 1, 128, kvh, d // 64, device=dev) * 0.02).half()
    q = torch.randn(rows, qh, d, device=dev).half()
    out = torch.empty(rows, qh * d, dtype=torch.float16, device=dev)
    row_req = torch.arange(rows, dtype=torch.int32, device=dev)
    row_pos = torch.full((rows,), ctx - 1, dtype=torch.int32, device=dev)
    splits = args.splits or min(F.attention_splits(ctx, rows, kvh), max(512 // rows, 1))
    need = native.lib().orinfer_attention_scratch_bytes(rows, qh, d, splits)
    scratch = torch.empty(max(need // 4, 1), dtype=torch.float32, device=dev)
    t = timed(lambda i: F.attention(q, None, row_req, row_pos, table, kc, vc, ks, vs,
                                    splits=splits, scratch=scratch, out=out), args.iters)
    bw, _, tag = peaks()
    moved = rows * ctx * kvh * (2 * d + 4 * (d // 64))
    print(json.dumps({"kernel": "attention_rows", "rows": rows, "ctx": ctx, "qh": qh, "kvh": kvh,
                      "d": d, "splits": splits, "us": t * 1e6, "gbs": moved / t / 1e9,
                      "frac_hbm": moved / t / bw, "peaks": tag}))


def act_prep(args, dev):
    """Residual add + RMSNorm + rotation + A8 (``--swiglu``: SwiGLU + rotation + A8)."""
    rows, k = args.rows, args.k
    g = torch.Generator(device="cpu").manual_seed(0)
    signs = (1 - 2 * torch.randint(0, 2, (k,), generator=g)).to(torch.int8).to(dev)
    if args.swiglu:
        x = torch.randn(rows, 2 * k, device=dev).half()
        t = timed(lambda i: F.act_prep(x, None, None, signs, swiglu=True), args.iters)
        moved = rows * (4 * k + k + 4)
    else:
        x = torch.randn(rows, k, device=dev).half()
        resid = torch.randn(rows, k, device=dev)
        w = torch.ones(k, device=dev).half()
        t = timed(lambda i: F.act_prep(x, resid, w, signs, eps=1e-6), args.iters)
        moved = rows * (2 * k + 8 * k + k + 4)
    bw, _, tag = peaks()
    print(json.dumps({"kernel": "act_prep", "swiglu": bool(args.swiglu), "rows": rows, "k": k,
                      "us": t * 1e6, "gbs": moved / t / 1e9, "frac_hbm": moved / t / bw,
                      "peaks": tag}))


def gdn(args, dev):
    """Sequential gated-delta scan: ``segs`` requests of ``tokens`` rows each."""
    hk, hv, d, n, segs = args.hk, args.hv, args.d, args.tokens, args.segs
    rows = n * segs
    conv_dim = (2 * hk + hv) * d
    qkv = (torch.randn(rows, conv_dim, device=dev) * 0.1).half()
    ab = torch.randn(rows, 2 * hv, device=dev)
    a_log, dt = torch.zeros(hv, device=dev), torch.zeros(hv, device=dev)
    state = torch.zeros(segs, hv, d, d, device=dev)
    seg = torch.tensor([[i * n, n, 0, 0] for i in range(segs)], dtype=torch.int32, device=dev)
    slot = torch.arange(segs, dtype=torch.int32, device=dev).repeat_interleave(n)
    pos = torch.arange(1, n + 1, dtype=torch.int32, device=dev).repeat(segs)
    out = torch.empty(rows, hv, d, device=dev)
    t = timed(lambda i: F.gdn_scan(qkv, ab, a_log, dt, seg, segs, slot, pos, hk, hv, d, state,
                                   out=out), args.iters)
    bw, _, tag = peaks()
    moved = 2.0 * segs * hv * d * d * 4 + rows * (conv_dim * 2 + hv * d * 4)
    print(json.dumps({"kernel": "gdn_scan", "tokens": n, "segments": segs, "hk": hk, "hv": hv,
                      "d": d, "us": t * 1e6, "us_per_token": t * 1e6 / n,
                      "gbs": moved / t / 1e9, "frac_hbm": moved / t / bw, "peaks": tag}))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--graph", action="store_true",
                    help="time the launches inside one CUDA graph (no host launch overhead)")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=512)
    g.add_argument("--n", type=int, default=19456)
    g.add_argument("--k", type=int, default=2560)
    g.add_argument("--fmt", default="q4", choices=["q4", "q2", "w8"])
    g.add_argument("--path", default="auto", choices=["auto", "simt", "tc"])
    g.add_argument("--rotate", action="store_true")
    g.add_argument("--iters", type=int, default=20)
    g.add_argument("--probe", type=int, default=0,
                   help="timing experiment of the one-tile kernel: 1 no MMAs, 2 no operand "
                        "copies, 4 no decode (bits combine; outputs are then meaningless)")
    g.add_argument("--impl", type=int, default=1, help="0 persistent kernel, 1 one tile per CTA, 2 CTA pairs")
    ad = sub.add_parser("attn-decode")
    ad.add_argument("--rows", type=int, default=1)
    ad.add_argument("--ctx", type=int, default=512)
    ad.add_argument("--qh", type=int, default=32)
    ad.add_argument("--kvh", type=int, default=8)
    ad.add_argument("--d", type=int, default=128)
    ad.add_argument("--splits", type=int, default=0)
    ad.add_argument("--iters", type=int, default=20)
    pp = sub.add_parser("act-prep")
    pp.add_argument("--rows", type=int, default=1)
    pp.add_argument("--k", type=int, default=2560)
    pp.add_argument("--swiglu", action="store_true")
    pp.add_argument("--iters", type=int, default=20)
    a = sub.add_parser("attn")
    a.add_argument("--tokens", type=int, default=2048)
    a.add_argument("--qh", type=int, default=32)
    a.add_argument("--kvh", type=int, default=8)
    a.add_argument("--d", type=int, default=128)
    a.add_argument("--iters", type=int, default=10)
    r = sub.add_parser("gdn")
    r.add_argument("--tokens", type=int, default=1)
    r.add_argument("--segs", type=int, default=128)
    r.add_argument("--hk", type=int, default=16)
    r.add_argument("--hv", type=int, default=32)
    r.add_argument("--d", type=int, default=128)
    r.add_argument("--iters", type=int, default=20)
    args = ap.parse_args(argv)
    global GRAPH
    GRAPH = args.graph
    dev = torch.device("cuda:0")
    native.init()
    {"gemm": gemm, "attn": attn, "gdn": gdn, "attn-decode": attn_decode,
     "act-prep": act_prep}[args.cmd](args, dev)
    st = native.read_status()
    if st:
        raise SystemExit(f"kernel status {st:#x}")


if __name__ == "__main__":
    main()
