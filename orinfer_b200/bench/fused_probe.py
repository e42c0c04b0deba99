"""Device-timed probe of the fused tensor-parallel step against its NCCL form and its roofline.

One step = what sits between two attention/FFN halves of a dense layer:

    row-parallel GEMM (o_proj / down_proj)  ->  reduce  ->  residual+RMSNorm+rotate+A8
    ->  column-parallel GEMM (gate_up / qkv)

* ``fused``: GEMM with reduce-scatter epilogue (peer stores) -> owner norm with all-gather
  push -> GEMM that waits per M tile for its source ranks (three launches, no NCCL);
* ``nccl``: GEMM -> ``all_reduce`` -> norm -> GEMM (the baseline arm).

Roofline of the step: the slower of (INT8 MACs of both GEMMs at 2 x the measured bf16 peak)
and (bytes a rank must send over NVLink: (tp-1)/tp * M*H*2 for the reduce-scatter plus
(tp-1)/tp * M*H*1 for the all-gather, at the measured 770 GB/s per direction).

Run under torchrun, one rank per GPU::

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \
        -m orinfer_b200.bench.fused_probe --rows 8192

Rank 0 prints one JSON line.  Times are CUDA-event times, max over ranks.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os

import torch
import torch.distributed as dist

from ..ops import functional as F
from ..ops import native
from ..ops.native import FMT, check, ptr, stream
from .kernel_probe import peaks
from ..parallel import fused

NVLINK_GBS = 770.0          # measured peer copy per direction per GPU (B200, NVSwitch)


def _weights(n, k, dev, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    codes = torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 128, n, 16), generator=g,
                          dtype=torch.int32).to(dev)
    scale = (torch.rand(n, generator=g) * 0.01 + 0.001).half().to(dev)
    return codes, scale


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--ffn", type=int, default=20480)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    native.init()
    lib = fused._setup_lib()
    m, h = args.rows, args.hidden
    k_row = args.ffn // world // 128 * 128            # down_proj: K = ffn / tp
    n_col = 2 * (args.ffn // world // 128 * 128)      # gate_up: N = 2 * ffn / tp
    mem = fused.PeerMemory(h, m, None, dev)
    w_row, s_row = _weights(h, k_row, dev, 1)
    w_col, s_col = _weights(n_col, h, dev, 2)
    a_row = torch.randint(-127, 128, (m, k_row), dtype=torch.int8, device=dev)
    sa_row = torch.rand(m, device=dev) * 0.01
    resid = torch.zeros(m, h, device=dev)
    norm_w = torch.ones(h, dtype=torch.float16, device=dev)
    signs = torch.ones(h, dtype=torch.int8, device=dev)
    out_col = torch.empty(m, n_col, dtype=torch.float16, device=dev)
    part = torch.empty(m, h, dtype=torch.float16, device=dev)
    q8 = torch.empty(m, h, dtype=torch.int8, device=dev)
    sc = torch.empty(m, dtype=torch.float32, device=dev)
    rows_per = (m + world - 1) // world
    po, ib, ag, ai = mem.peer_out["down"], mem.inbox["down"], mem.ag_out, mem.ag_in

    def step_fused():
        po.rows_per = ag.rows_per = ai.rows_per = rows_per
        check(lib.orinfer_qgemm_peer(FMT["q4"], ptr(a_row), ptr(sa_row), ptr(w_row), ptr(s_row),
                                     ctypes.byref(po), m, h, k_row, 0, stream()), "gemm_rs")
        check(lib.orinfer_act_prep_sp(ctypes.byref(ib), ctypes.byref(ag), ptr(resid), ptr(norm_w),
                                      ptr(signs), m, h, 1e-6, 0, stream(), None), "norm_ag")
        check(lib.orinfer_qgemm_ag(FMT["q4"], ptr(mem.ag_q), ptr(mem.ag_scale), ptr(w_col),
                                   ptr(s_col), ptr(out_col), ctypes.byref(ai), m, n_col, h, 0,
                                   stream()), "ag_gemm")

    def step_nccl():
        F.qgemm(a_row, sa_row, w_row, s_row, "q4", h, out=part)
        dist.all_reduce(part)
        F.act_prep(part, resid, norm_w, signs, q_out=q8, scale_out=sc)
        F.qgemm(q8, sc, w_col, s_col, "q4", n_col, out=out_col)

    def step_local():                                 # the two GEMMs + norm, no communication
        F.qgemm(a_row, sa_row, w_row, s_row, "q4", h, out=part)
        F.act_prep(part, resid, norm_w, signs, q_out=q8, scale_out=sc)
        F.qgemm(q8, sc, w_col, s_col, "q4", n_col, out=out_col)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / args.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t) * 1e-3

    t_fused, t_nccl, t_local = timed(step_fused), timed(step_nccl), timed(step_local)
    _, bf16, tag = peaks()
    ops = 2.0 * m * h * k_row + 2.0 * m * n_col * h
    t_compute = ops / (2 * bf16)
    link_bytes = (world - 1) / world * m * h * 3.0
    t_link = link_bytes / (NVLINK_GBS * 1e9)
    bound = max(t_compute, t_link)
    st = torch.tensor([native.read_status()], device=dev)
    dist.all_reduce(st, op=dist.ReduceOp.MAX)          # any rank's failed wait counts
    status = int(st[0])
    if rank == 0:
        print(json.dumps({
            "probe": "row-parallel GEMM -> reduce -> norm/quant -> column-parallel GEMM",
            "tp": world, "rows": m, "hidden": h, "k_row": k_row, "n_col": n_col,
            "us_fused": t_fused * 1e6, "us_nccl": t_nccl * 1e6, "us_no_comm": t_local * 1e6,
            "fused_vs_nccl": t_nccl / t_fused,
            "roofline_us": {"compute": t_compute * 1e6, "nvlink": t_link * 1e6},
            "frac_of_roofline_fused": bound / t_fused, "frac_of_roofline_nccl": bound / t_nccl,
            "peaks": tag, "int8_peak_assumed": "2 x bf16 cuBLAS burst", "kernel_status": status}))
    dist.barrier()
    torch.cuda.synchronize()
    import threading
    guard = threading.Timer(30.0, lambda: os._exit(0))   # never hang in library teardown
    guard.daemon = True
    guard.start()
    mem.close()
    dist.destroy_process_group()
    guard.cancel()


if __name__ == "__main__":
    main()
