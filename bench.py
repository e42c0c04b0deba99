#!/usr/bin/env python
"""Headline benchmark: prefill tokens/s at 512-token prompts on the Qwen3.5-4B-class
dense decoder (E8P Q4A8 projections, W8 head, INT8 KV), plus the other rows of the
reference's headline matrix (prefill 8K, decode bs1 / bs8 / bs128, bs1 with the MTP draft
head) as ``extra``.  ``--model`` selects the other benchmark geometries (27b-class,
35b-a3b-class, 80b-a3b-class); the 4B-class model stays the default headline.

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...     # the unmodified reference, when it can run

One *step* is the prefill of one fresh prompt of uniform-random token ids up to its
first sampled token (the reference's prefill_tps = input_tokens / time_to_first_token,
docs/performance.md:42-44).  ``value`` is timed on the device with CUDA events around
K steps whose prompts are already on the device (``Engine.prefill_device``); the K steps
are repeated ``--reps`` times and the median repetition is reported.  ``e2e`` runs the same
K steps through ``Engine.generate`` with the prompt copied from pinned host memory and the
sampled token read back every step.  On more than one GPU every rank first runs one
prefill packet and a few decode steps through both the fused peer-memory runner and the
NCCL runner and refuses to time anything when their greedy tokens differ.  Prints one JSON
line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

MODEL = "qwen3.5-4b-class"
PROMPT = 512
# Published prefill-512 tok/s of the reference on Jetson AGX Orin (docs/performance.md:47-51)
BASELINE_PREFILL_512 = {"qwen3.5-4b-class": 3582.9, "27b-class": 655.2,
                        "35b-a3b-class": 2204.5, "80b-a3b-class": 979.3}


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


def fused_vs_nccl(shard, cfg, dev, torch, dist):
    """One 512-row packet and three decode steps through the NCCL runner and the fused
    peer-memory runner on the same shard.  Both arms are fed the same tokens (the NCCL arm's),
    so every step compares like with like: the logits must agree (cosine > 0.9995) and the
    greedy token must be equal wherever the NCCL arm's best two logits are further apart than
    the arms' rounding difference (random-init weights give near ties).  Returns a checksum of
    the first step's logits per arm."""
    from orinfer_b200.models.runner import KVPool, Packet
    from orinfer_b200.ops import native
    from orinfer_b200.parallel.fused import FusedTPRunner
    from orinfer_b200.parallel.tp_runner import TPRunner
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    n = PROMPT
    pages = list(range(1, n // 128 + 3))
    outs, sums = {}, {}
    # The NCCL arm reduces with the fused consumer's arithmetic here (FP16 partials summed in
    # FP32 in rank order) instead of NCCL's FP16 ring sum: deep random-init networks amplify
    # that rounding difference (cosine 0.997 at 8 ranks on the 4B-class model), which would say
    # nothing about the fused kernels.  With it, dense models agree bit for bit.
    os.environ["ORINFER_TP_EXACT_REDUCE"] = "1"
    for name, cls in (("nccl", TPRunner), ("fused", FusedTPRunner)):
        runner = cls(shard, KVPool.allocate(shard.config, len(pages) + 1, dev), n + 8)
        gg = torch.Generator().manual_seed(4321)
        ids = torch.randint(0, cfg.vocab, (n,), generator=gg, dtype=torch.int32).to(dev)
        table = t([pages])
        p = Packet(ids, t([0] * n), t(list(range(n))), table, n, n,
                   torch.tensor([n - 1], device=dev),
                   chunks=t([[0, n, 0, 0]]), max_q_len=n)
        tok, lg = runner.greedy(p)
        seq = [(tok.cpu(), lg.float().cpu())]
        for step in range(3):
            feed = tok if name == "nccl" else outs["nccl"][step][0].to(dev)
            p = Packet(feed.clone(), t([0]), t([n + step]), table, 1, n + step + 1)
            tok, lg = runner.greedy(p)
            seq.append((tok.cpu(), lg.float().cpu()))
        torch.cuda.synchronize()
        outs[name] = seq
        sums[name] = round(float(seq[0][1].double().abs().sum()), 3)
        if hasattr(runner, "close"):
            runner.close()
        del runner
    os.environ.pop("ORINFER_TP_EXACT_REDUCE", None)
    # pure mixture-of-experts packets of this size take the expert all-to-all in the fused arm
    # and replicated tokens in the NCCL arm: near-tied routing may flip, so only rough
    # agreement is asked of them
    floor = 0.98 if (cfg.experts and cfg.arch != "hybrid") else 0.9995
    ok = True
    detail = []
    for (tn, ln), (tf, lf) in zip(outs["nccl"], outs["fused"]):
        cos = float(torch.nn.functional.cosine_similarity(ln.flatten(), lf.flatten(), dim=0))
        top2 = torch.topk(ln.flatten(), 2).values
        clear = float(top2[0] - top2[1]) > 4.0 * float((ln - lf).abs().max())
        ok = ok and cos > floor and (bool(torch.equal(tn, tf)) or not clear or floor < 0.99)
        detail.append([round(cos, 6), bool(torch.equal(tn, tf)), clear])
    sums["steps"] = detail
    flag = torch.tensor([0 if ok else 1, native.read_status()], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    return bool(flag[0] == 0) and int(flag[1]) == 0, sums


def bigram_like(weights, torch, strength: float = 0.5) -> None:
    """Turns random-init weights into a model the draft head can partly predict.  The input
    embedding of token t becomes the head row of pi(t) for a fixed random permutation pi, so
    the token after t is mostly pi(t) (a long cycle, not a fixed point), perturbed by the
    attention and FFN branches, whose output projections are scaled by ``strength``; the
    draft head's input projection passes the token embedding through and its own (different)
    branches perturb its guess in another way.  Target and draft therefore agree often but
    not always.  Every GEMM keeps its shape and format; only scales and the embedding order
    change.  Real checkpoints carry a trained draft head; random weights have nothing to
    accept, and speculation on them only measures the cost of finding that out."""
    current = getattr(weights, "_bigram_strength", None)
    if current is None:
        g = torch.Generator(device="cpu").manual_seed(7)
        perm = torch.randperm(weights.embed_q.shape[0], generator=g).to(weights.embed_q.device)
        # new tensors: a tied head keeps the original rows (captured graphs must be dropped)
        weights.embed_q = weights.embed_q.index_select(0, perm).contiguous()
        weights.embed_s = weights.embed_s.index_select(0, perm).contiguous()
        current = 1.0
    weights._bigram_strength = strength
    first, strength = current == 1.0 and not hasattr(weights, "_bigram_fc"), strength / current
    for lw in weights.layers:
        for lin in (lw.o, lw.down, lw.gdn_out, lw.shared_down):
            if lin is not None:
                lin.scale.mul_(strength)
        if lw.expert_down is not None:
            lw.expert_down.scale.mul_(strength)
    m = weights.mtp
    if m is not None:
        if first:
            h = weights.config.hidden
            eye = torch.zeros(h, 2 * h, dtype=torch.int8, device=m.fc.codes.device)
            eye[:, :h] = torch.eye(h, dtype=torch.int8, device=eye.device) * 127
            m.fc.codes.copy_(eye)
            m.fc.scale.fill_(1.0 / 127.0)
            weights._bigram_fc = True
        for lin in (m.layer.o, m.layer.down):
            lin.scale.mul_(strength)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--reps", type=int, default=5,
                    help="repetitions of the K timed steps; the median one is reported")
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--model", default=MODEL, choices=sorted(BASELINE_PREFILL_512))
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary metrics")
    ap.add_argument("--profile-step", choices=["prefill", "decode"], default=None,
                    help="run warm-up, then exactly one step between cudaProfilerStart/Stop "
                         "and leave (for `ncu --profile-from-start off`); prints no result")
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
    from orinfer_b200.models.weights import random_model
    from orinfer_b200.ops import native

    native.init()
    cfg = PRESETS[args.model]
    check = {}
    if world > 1:
        from orinfer_b200.parallel.tp import random_shard
        weights = random_shard(cfg, rank, world, dev, seed=0)
        ok, sums = fused_vs_nccl(weights, cfg, dev, torch, dist)
        check = {"fused_vs_nccl": "ok" if ok else "MISMATCH", "logit_checksum": sums}
        # a mismatch does not stop the run: the line below then carries it beside the numbers
        # and the process exits non-zero at the end
    else:
        weights = random_model(cfg, seed=0, device=dev)
    load = LoadOptions(cuda_graph=GraphMode.FULL, prefix_cache_bytes=0, tp=world)
    sched = SchedulerOptions(max_active=128, prefill_chunk=8192)
    engine = Engine(weights, load=load, sched=sched, kv_pages=128 * 6 + 80,
                    max_context=8192 + 512, max_rows=8192 + 128)
    gen = torch.Generator(device="cpu").manual_seed(1234)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    # ---------------------------------------------------------- device-timed prefill
    def device_prefill(n_tokens: int, steps: int, warmup: int, reps: int):
        """K prompts already on the device, each run up to its first token by the engine's
        full-graph prefill path; CUDA events around the K steps, max over ranks, median of
        `reps` repetitions (every repetition uses fresh prompts)."""
        prompts = [torch.randint(0, cfg.vocab, (n_tokens,), generator=gen,
                                 dtype=torch.int32).to(dev)
                   for _ in range(warmup + steps * reps)]
        run = engine.prefill_device
        if engine.recurrent:
            # recurrent (gated-delta-rule) models have no device-resident prefill entry: the
            # prompt goes through Engine.generate, host round trip included
            host = {id(p): p.tolist() for p in prompts}
            run = lambda p: engine.generate([host[id(p)]], max_new=1)
        for p in prompts[:warmup]:
            run(p)
        times, launches = [], 0
        for r in range(reps):
            batch = prompts[warmup + r * steps:warmup + (r + 1) * steps]
            barrier()
            l0 = native.launches()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for p in batch:
                run(p)
            b.record()
            barrier()
            times.append(max_over_ranks(a.elapsed_time(b)) / steps)
            launches = native.launches() - l0
        return statistics.median(times), launches, times

    # ---------------------------------------------------------- end to end via Engine
    def e2e_prefill(n_tokens: int, steps: int, warmup: int, reps: int):
        prompts = [torch.randint(0, cfg.vocab, (n_tokens,), generator=gen).tolist()
                   for _ in range(warmup + steps * reps)]
        for p in prompts[:warmup]:
            engine.generate([p], max_new=1)
        times = []
        for r in range(reps):
            batch = prompts[warmup + r * steps:warmup + (r + 1) * steps]
            barrier()
            t0 = time.perf_counter()
            for p in batch:
                engine.generate([p], max_new=1)
            torch.cuda.synchronize()
            ms = (time.perf_counter() - t0) * 1e3
            barrier()
            times.append(max_over_ranks(ms) / steps)
        return statistics.median(times)

    def decode_rate(batch: int, context: int, new_tokens: int, mtp: bool = False,
                    policy: str = "auto"):
        """Aggregate decode tokens/s of `batch` concurrent requests through the Engine
        (CUDA-graph decode, greedy, one token readback per step)."""
        from orinfer_b200.engine.speculation import Speculator
        saved_drafts = engine.spec.max_drafts
        if mtp:                                  # a controller that has learnt nothing yet
            engine.spec = Speculator(engine, engine.load.mtp_drafts, engine.load.prompt_lookup)
            engine.spec.policy = policy
            saved_drafts = engine.spec.max_drafts
        else:
            engine.spec.max_drafts = 0
        prompts = [torch.randint(0, cfg.vocab, (context,), generator=gen).tolist()
                   for _ in range(batch)]
        reqs = [engine.submit(p, new_tokens + 8, ignore_eos=True) for p in prompts]
        while any(r.remaining_prefill > 0 or not r.generated for r in reqs):
            engine.step()
        for _ in range(4):                      # graph warm-up + capture
            engine.step()
        barrier()
        spec0 = dict(engine.spec.statistics())
        start = sum(len(r.generated) for r in reqs)
        t0 = time.perf_counter()
        steps = 0
        while not any(r.finished for r in reqs) and \
                sum(len(r.generated) for r in reqs) - start < batch * (new_tokens - 6):
            engine.step()
            steps += 1
        torch.cuda.synchronize()
        dt = max_over_ranks(time.perf_counter() - t0)
        produced = sum(len(r.generated) for r in reqs) - start
        spec1 = engine.spec.statistics()
        for r in reqs:
            engine.cancel(r)
        while engine.has_work():
            engine.step()
        engine.spec.max_drafts = saved_drafts
        prop = spec1.get("proposed_tokens", 0) - spec0.get("proposed_tokens", 0)
        acc = spec1.get("accepted_draft_tokens", 0) - spec0.get("accepted_draft_tokens", 0)
        info = {"acceptance": round(acc / prop, 3) if prop else None,
                "rounds": spec1.get("rounds", 0) - spec0.get("rounds", 0), "steps": steps,
                "resident_steps": engine.stats.resident_steps}
        return produced / dt, dt / max(steps, 1) * 1e3, info

    if args.profile_step:
        if args.profile_step == "prefill":
            prompts = [torch.randint(0, cfg.vocab, (PROMPT,), generator=gen,
                                     dtype=torch.int32).to(dev) for _ in range(5)]
            for p in prompts[:4]:
                engine.prefill_device(p)
            step = lambda: engine.prefill_device(prompts[4])
        else:
            req = engine.submit(torch.randint(0, cfg.vocab, (PROMPT,), generator=gen).tolist(),
                                64, ignore_eos=True)
            engine.spec.max_drafts = 0
            for _ in range(8):
                engine.step()
            step = engine.step
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        step()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        engine.close()
        return 0
    sampler = ClockSampler(local) if rank == 0 else None
    ms_dev, launches, rep_ms = device_prefill(PROMPT, args.steps, args.warmup, args.reps)
    clocks = sampler.stop() if sampler else {}
    ms_e2e = e2e_prefill(PROMPT, args.steps, args.warmup, min(args.reps, 3))
    extra = {}
    if not args.no_extra:
        ms8k, _, _ = device_prefill(8192, max(2, args.steps // 5), 3, 1)
        extra["prefill_tok_s_8192"] = round(8192 / ms8k * 1e3, 1)
        for b in (1, 8, 128):
            rate, ms, _ = decode_rate(b, 512, 64)
            extra[f"decode_tok_s_bs{b}"] = round(rate, 1)
            extra[f"decode_ms_per_step_bs{b}"] = round(ms, 3)
        if engine.spec.enabled and cfg.ffn and not cfg.experts:     # dense draft layer only
            rate, ms, accept = decode_rate(1, 512, 256, mtp=True)
            extra["decode_tok_s_bs1_mtp_random_weights"] = round(rate, 1)
            extra["mtp_random_weights"] = accept
            # a draft head with something to predict (see bigram_like): same GEMMs, same
            # formats, measured acceptance reported beside the rate
            # raise the branch strength until the fixed-width acceptance falls below what a
            # trained draft head reaches (0.6-0.8), keep the last one above it, then measure
            # with the adaptive controller
            chosen, seen = None, {}
            for strength in (0.0005, 0.001, 0.002, 0.004, 0.008, 0.016, 0.03, 0.06, 0.12, 0.25):
                bigram_like(engine.w, torch, strength)
                engine._graphs.clear()            # captured steps hold the old embedding
                engine.__dict__.pop("_prefill_graphs", None)
                _, _, probe = decode_rate(1, 512, 64, mtp=True, policy="fixed3")
                seen[strength] = probe["acceptance"]
                if (probe["acceptance"] or 0.0) < 0.6:
                    break
                chosen = strength
            strength = chosen if chosen is not None else 0.0005
            bigram_like(engine.w, torch, strength)
            engine._graphs.clear()
            extra["mtp_strength_scan"] = seen
            extra["mtp_branch_strength"] = strength
            rate0, _, _ = decode_rate(1, 512, 256)
            rate, ms, accept = decode_rate(1, 512, 256, mtp=True)
            extra["decode_tok_s_bs1_mtp"] = round(rate, 1)
            extra["decode_tok_s_bs1_mtp_off_same_weights"] = round(rate0, 1)
            extra["mtp_acceptance"] = accept["acceptance"]
            extra["mtp"] = accept
    status = native.read_status()
    if world > 1:
        st = torch.tensor([status], device=dev)
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
        status = int(st[0])
    if rank == 0:
        value = PROMPT / ms_dev * 1e3
        line = {
            "metric": "prefill_tok_s_512", "value": round(value, 1), "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_dev, 4), "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": round(value / BASELINE_PREFILL_512[args.model], 3),
            "dtype": "int8 (E8P Q4 weights x A8 activations, int32 accumulate; fp16 "
                     "activations, fp32 residual)",
            "data": "synthetic uniform-random token ids; random-init N(0,0.02) weights "
                    "quantised to E8P Q4A8 / W8",
            "config": {"model": args.model, "global_batch": 1, "seq_len": PROMPT,
                       "parallelism": f"tp{world}",
                       "l2": "inputs larger than L2: every step streams the packed weights "
                             "of the whole model and a fresh prompt",
                       "kv": "int8 group-64, paged", "cuda_graph": "full",
                       "repetitions": args.reps,
                       "ms_per_step_of_each_repetition": [round(t, 4) for t in rep_ms]},
            "e2e": {"value": round(PROMPT / ms_e2e * 1e3, 1), "unit": "tok/s",
                    "h2d_bytes_per_step": 3 * PROMPT * 4 + 8 + engine.max_pages_per_req * 4,
                    "d2h_bytes_per_step": 4 + 16,
                    "api": "orinfer_b200.engine.Engine.generate"},
            "gpu_launches": int(launches), "clocks": clocks, "extra": extra,
            "kernel_status": status, "impl": "native", **check,
        }
        print(json.dumps(line), flush=True)
    sys.stdout.flush()
    sys.stderr.flush()
    # Tear down in dependency order: captured graphs (they hold NCCL and peer-memory work),
    # then the peer mappings, then the process group.  A guard thread ends the process if
    # the library teardown does not return: the result is printed by then.
    guard = threading.Timer(30.0, lambda: os._exit(0))
    guard.daemon = True
    guard.start()
    engine.close()
    if world > 1:
        barrier()
        dist.destroy_process_group()
    guard.cancel()
    return 3 if check.get("fused_vs_nccl") == "MISMATCH" else 0


if __name__ == "__main__":
    sys.exit(main())
