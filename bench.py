#!/usr/bin/env python
"""Headline benchmark: prefill tokens/s at 512-token prompts on the Qwen3.5-4B-class
dense decoder (E8P Q4A8 projections, W8 head, INT8 KV), plus the other rows of the
reference's headline matrix (prefill 8K, decode bs1 / bs8 / bs128) as ``extra``.

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...     # the unmodified reference, when it can run

One *step* is the prefill of one fresh prompt of uniform-random token ids up to its
first sampled token (the reference's prefill_tps = input_tokens / time_to_first_token,
docs/performance.md:42-44).  ``value`` is timed on the device with CUDA events around
the K steps (inputs resident on the device); ``e2e`` runs the same K steps through the
public ``Engine`` API with the prompt copied from pinned host memory and the sampled
token read back every step.  Prints one JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

BASELINE_PREFILL_512 = 3582.9     # Qwen3.5-4B on Jetson AGX Orin, docs/performance.md:47
MODEL = "qwen3.5-4b-class"
PROMPT = 512


def reference_arm(args) -> int:
    """The reference's serving engine is Rust (no cargo/rustc in this image), its kernels
    are TileLang cubins built for sm_87 only, and its CUDA executor refuses any device
    that is not SM 8.7, so the metric cannot be produced from baseline/_ref here."""
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference engine is Rust + sm_87-only TileLang cubins (executor "
                       "requires SM 8.7); only its offline Python toolchain installs here",
    }))
    return 0


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.tmp,
                stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.proc.wait()
        self.tmp.flush()
        self.tmp.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.tmp.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.tmp.name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary metrics")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from orinfer_b200.config import PRESETS, GraphMode, LoadOptions, SchedulerOptions
    from orinfer_b200.engine.engine import Engine
    from orinfer_b200.models.runner import Packet
    from orinfer_b200.models.weights import random_model
    from orinfer_b200.ops import native

    native.init()
    cfg = PRESETS[args.model]
    if world > 1:
        from orinfer_b200.parallel.tp import shard_model
        weights = shard_model(random_model(cfg, seed=0, device=dev), rank, world)
    else:
        weights = random_model(cfg, seed=0, device=dev)
    load = LoadOptions(cuda_graph=GraphMode.FULL, prefix_cache_bytes=0, tp=world)
    sched = SchedulerOptions(max_active=128, prefill_chunk=8192)
    engine = Engine(weights, load=load, sched=sched, kv_pages=128 * 6 + 80, max_context=8192 + 512,
                    max_rows=8192 + 128)
    runner = engine.runner
    gen = torch.Generator(device="cpu").manual_seed(1234 + rank * 0)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    # ---------------------------------------------------------- device-timed prefill
    def device_prefill(n_tokens: int, steps: int, warmup: int):
        pages = (n_tokens + 127) // 128
        table = torch.zeros(1, engine.max_pages_per_req, dtype=torch.int32, device=dev)
        table[0, :pages] = torch.arange(1, pages + 1, dtype=torch.int32, device=dev)
        packets = []
        for _ in range(steps + warmup):
            ids = torch.randint(0, cfg.vocab, (n_tokens,), generator=gen, dtype=torch.int32).to(dev)
            packets.append(Packet(ids, torch.zeros(n_tokens, dtype=torch.int32, device=dev),
                                  torch.arange(n_tokens, dtype=torch.int32, device=dev), table,
                                  n_tokens, n_tokens, torch.tensor([n_tokens - 1], device=dev),
                                  chunks=torch.tensor([[0, n_tokens, 0, 0]], dtype=torch.int32,
                                                      device=dev), max_q_len=n_tokens))
        def run(p):
            # the engine's own full-graph path: a prefill geometry is captured at its second
            # use and replayed afterwards (inputs are copied into the graph's static buffers)
            if engine._prefill_graph(p, (n_tokens,), False) is None:
                runner.greedy(p)

        for p in packets[:warmup]:
            run(p)
        barrier()
        l0 = native.launches()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for p in packets[warmup:]:
            run(p)
        b.record()
        barrier()
        return max_over_ranks(a.elapsed_time(b)) / steps, (native.launches() - l0)

    # ---------------------------------------------------------- end to end via Engine
    def e2e_prefill(n_tokens: int, steps: int, warmup: int):
        prompts = [torch.randint(0, cfg.vocab, (n_tokens,), generator=gen).tolist()
                   for _ in range(steps + warmup)]
        for p in prompts[:warmup]:
            engine.generate([p], max_new=1)
        barrier()
        t0 = time.perf_counter()
        for p in prompts[warmup:]:
            engine.generate([p], max_new=1)
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        barrier()
        return max_over_ranks(ms) / steps

    def decode_rate(batch: int, context: int, new_tokens: int, mtp: bool = False):
        """Aggregate decode tokens/s of `batch` concurrent requests through the Engine
        (CUDA-graph decode, greedy, one token readback per step).  ``mtp`` keeps the adaptive
        draft-head speculation on; random-init weights give it almost nothing to accept, so
        that number shows the controller's cost of finding that out, not a speed-up."""
        saved_drafts = engine.spec.max_drafts
        if not mtp:
            engine.spec.max_drafts = 0
        prompts = [torch.randint(0, cfg.vocab, (context,), generator=gen).tolist()
                   for _ in range(batch)]
        reqs = [engine.submit(p, new_tokens + 8, ignore_eos=True) for p in prompts]
        while any(r.remaining_prefill > 0 or not r.generated for r in reqs):
            engine.step()
        for _ in range(4):                      # graph warm-up + capture
            engine.step()
        barrier()
        start = sum(len(r.generated) for r in reqs)
        t0 = time.perf_counter()
        steps = 0
        while steps < new_tokens - 6 and not any(r.finished for r in reqs):
            engine.step()
            steps += 1
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        produced = sum(len(r.generated) for r in reqs) - start
        for r in reqs:
            engine.cancel(r)
        while engine.has_work():
            engine.step()
        engine.spec.max_drafts = saved_drafts
        return produced / dt, dt / max(steps, 1) * 1e3

    sampler = ClockSampler(local) if rank == 0 else None
    ms_dev, launches = device_prefill(PROMPT, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else {}
    ms_e2e = e2e_prefill(PROMPT, args.steps, args.warmup)
    extra = {}
    if not args.no_extra:
        ms8k, _ = device_prefill(8192, max(2, args.steps // 5), 3)
        extra["prefill_tok_s_8192"] = round(8192 / ms8k * 1e3, 1)
        for b in (1, 8, 128):
            rate, ms = decode_rate(b, 512, 64)
            extra[f"decode_tok_s_bs{b}"] = round(rate, 1)
            extra[f"decode_ms_per_step_bs{b}"] = round(ms, 3)
        if engine.spec.enabled:
            rate, ms = decode_rate(1, 512, 256, mtp=True)
            extra["decode_tok_s_bs1_mtp_adaptive_random_weights"] = round(rate, 1)
    status = native.read_status()
    if rank == 0:
        value = PROMPT / ms_dev * 1e3
        line = {
            "metric": "prefill_tok_s_512", "value": round(value, 1), "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_dev, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": round(value / BASELINE_PREFILL_512, 3),
            "dtype": "int8 (E8P Q4 weights x A8 activations, int32 accumulate; fp16 "
                     "activations, fp32 residual)",
            "data": "synthetic uniform-random token ids; random-init N(0,0.02) weights "
                    "quantised to E8P Q4A8 / W8",
            "config": {"model": args.model, "global_batch": 1, "seq_len": PROMPT,
                       "parallelism": f"tp{world}",
                       "l2": "inputs larger than L2: every step streams 2.2 GB of packed "
                             "weights and a fresh prompt",
                       "kv": "int8 group-64, paged", "cuda_graph": "full"},
            "e2e": {"value": round(PROMPT / ms_e2e * 1e3, 1), "unit": "tok/s",
                    "h2d_bytes_per_step": 3 * PROMPT * 4 + 8 + engine.max_pages_per_req * 4,
                    "d2h_bytes_per_step": 4,
                    "api": "orinfer_b200.engine.Engine.generate"},
            "gpu_launches": int(launches), "clocks": clocks, "extra": extra,
            "kernel_status": status, "impl": "native",
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # Captured decode graphs hold NCCL work; tearing the communicator down under them
        # can block for minutes.  Everything is flushed, so leave without the teardown.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
