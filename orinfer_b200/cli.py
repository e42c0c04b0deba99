"""``orinfer`` command line: serve, batch, validate-model, plan-model, run-model,
score-model, make-model, devices, info, validate-nccl.

Verbs, flags and defaults mirror the reference's CLI (crates/orinfer-cli/src/args.rs:7-111,
serve.rs:48-260, diag.rs:8-101; flag table docs/serving.md:229-263): listen ``[::]:8088``,
``--scheduler-policy latency|throughput``, ``--cuda-graph decode_only|full|off``,
``--mtp-drafts auto|0..31``, ``--prefix-cache-mib 4096``, ``--kv-offload-mib 0``,
``--max-active-requests 32``, ``--prefill-budget-ms 200``, ``--target-tpot-ms 400``,
``--memory-reserve-mib 1024``, queue / output / drain timeouts 0 / 60000 / 30000 ms.
``--tp N`` is this build's addition (the reference has no multi-GPU CUDA path).
"""

from __future__ import annotations

import argparse
import json
import signal
import sys
import time
from pathlib import Path

from .config import PRESETS, GraphMode, LoadOptions, Policy, SchedulerOptions


def _load_args(p: argparse.ArgumentParser, batch: bool = False) -> None:
    p.add_argument("model_dir", nargs="?", help="model directory (with cache/model.json)")
    p.add_argument("--preset", choices=sorted(PRESETS), help="random-init model of a named "
                   "geometry instead of a model directory")
    p.add_argument("--model", default="qwen3.8-27b", help="API model id")
    p.add_argument("--default-request-params", default="{}")
    p.add_argument("--scheduler-policy", default="throughput" if batch else "latency",
                   choices=["latency", "throughput"])
    p.add_argument("--cuda-graph", "--graph", dest="cuda_graph", default="decode_only",
                   choices=["decode_only", "full", "off"])
    p.add_argument("--mtp-drafts", default="auto")
    p.add_argument("--prompt-lookup", action="store_true")
    p.add_argument("--resident-experts", default="full")
    p.add_argument("--verify-weights", action="store_true")
    p.add_argument("--load-workers", type=int, default=0)
    p.add_argument("--prefix-cache-mib", type=int, default=4096)
    p.add_argument("--kv-offload-mib", type=int, default=0)
    p.add_argument("--max-active-requests", type=int, default=32)
    p.add_argument("--max-batch-tokens", type=int, default=128)
    p.add_argument("--max-speculative-tokens", type=int, default=0)
    p.add_argument("--prefill-budget-ms", type=float, default=200.0)
    p.add_argument("--target-tpot-ms", type=float, default=400.0)
    p.add_argument("--memory-reserve-mib", type=int, default=1024)
    p.add_argument("--prefill-chunk", type=int, default=4096)
    p.add_argument("--prefill-stages", type=int, default=1,
                   help="pause long prompt packets at this many layer boundaries so that "
                        "decoding requests step in between (1 = off)")
    p.add_argument("--max-context", type=int, default=None)
    p.add_argument("--tp", type=int, default=1)
    p.add_argument("--tp-draft-head", action="store_true",
                   help="with --tp: shard the model's draft head too and speculate with it "
                        "(verified on CPU ranks only so far)")
    p.add_argument("--device", default="cuda")


def _options(a):
    drafts = None if a.mtp_drafts == "auto" else int(a.mtp_drafts)
    load = LoadOptions(cuda_graph=GraphMode(a.cuda_graph), verify_weights=a.verify_weights,
                       load_workers=a.load_workers, prefix_cache_bytes=a.prefix_cache_mib << 20,
                       kv_offload_bytes=a.kv_offload_mib << 20, mtp_drafts=drafts,
                       prompt_lookup=a.prompt_lookup,
                       resident_experts=0 if a.resident_experts == "full"
                       else int(a.resident_experts), tp=a.tp)
    sched = SchedulerOptions(policy=Policy(a.scheduler_policy), max_active=a.max_active_requests,
                             max_batch_tokens=a.max_batch_tokens,
                             max_speculative_tokens=a.max_speculative_tokens,
                             prefill_budget_ms=a.prefill_budget_ms,
                             target_tpot_ms=a.target_tpot_ms,
                             memory_reserve_bytes=a.memory_reserve_mib << 20,
                             prefill_chunk=a.prefill_chunk, prefill_stages=a.prefill_stages)
    load.validate()
    sched.validate()
    return load, sched


def _weights(a):
    import torch
    from .models.weights import random_model
    dev = a.device if (a.device != "cuda" or torch.cuda.is_available()) else "cpu"
    if a.preset:
        return random_model(PRESETS[a.preset], seed=0, device=dev), a.preset
    if not a.model_dir:
        raise SystemExit("a model directory or --preset is required")
    from .engine.checkpoint import load_model, read_descriptor
    t0 = time.time()
    w = load_model(a.model_dir, dev, verify=a.verify_weights)
    print(f"MODEL READY after {time.time() - t0:.2f}s", file=sys.stderr)
    return w, read_descriptor(a.model_dir)["name"]


def _engine_factory(a, weights, load, sched):
    from .engine.engine import Engine

    def factory():
        # dimensions, sharding and memory are checked before the engine allocates anything
        from .engine.plan import validate_plan
        device_bytes = None
        dev = weights.embed_q.device
        if dev.type == "cuda":
            import torch
            device_bytes = torch.cuda.get_device_properties(dev).total_memory
        validate_plan(weights.config, load, sched, max_context=a.max_context,
                      device_bytes=device_bytes)
        return Engine(weights, load=load, sched=sched, max_context=a.max_context)
    return factory


def _codec(a, weights, name):
    from .api.chat_codec import ChatCodec
    ctx = a.max_context or min(weights.config.max_context, 32768)
    if a.model_dir:
        codec = ChatCodec.load(Path(a.model_dir), weights.config.vocab, ctx, name)
    else:
        from .api.chat_codec import ByteTokenizer
        codec = ChatCodec(ByteTokenizer(weights.config.vocab), context=ctx, model_name=name)
    codec.tool_format = getattr(a, "tool_format", "xml")
    if getattr(a, "vision", False):
        from .api.images import frontend_for
        codec.images = frontend_for(codec.tokenizer, weights.config.hidden, a.image_cache_mib)
    return codec


def cmd_serve(a) -> int:
    import uvicorn
    from .api.server import Service, create_app
    load, sched = _options(a)
    host, _, port = a.listen.rpartition(":")
    host = host.strip("[]") or "::"
    # bind first: a port conflict must fail before the GPU load starts
    import socket
    probe = socket.socket(socket.AF_INET6 if ":" in host else socket.AF_INET)
    probe.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    try:
        probe.bind((host, int(port)))
    except OSError as e:
        print(f"cannot bind {a.listen}: {e}", file=sys.stderr)
        return 2
    probe.close()
    if not a.model_dir and not a.preset:
        return _serve_manager(a, host, int(port), load, sched)
    if getattr(a, "gpu_lock", None):
        # one holder per device: a second server (or a measurement) on the same GPU is
        # refused at once instead of sharing it unnoticed
        from .bench.telemetry import GpuBusy, GpuLock
        index = int(str(a.device).partition(":")[2] or 0)
        try:
            a._gpu_lock = GpuLock(index, a.gpu_lock).acquire()      # held for the process's life
        except GpuBusy as e:
            print(str(e), file=sys.stderr)
            return 2
    # Listen first, load behind: /health answers `starting` (503) while the weights load, a
    # port conflict shows at once, and clients that retry on 503 need no separate readiness poll
    # (the reference binds before loading too, crates/orinfer-api/src/server/startup.rs:44-160).
    import threading
    from types import SimpleNamespace
    cfg, name = _model_identity(a)
    name = a.model if a.model != "qwen3.8-27b" or not a.preset else name

    teams = []

    def factory():
        if a.tp > 1:
            # rank 0 (this process) leads: it starts the follower ranks, joins the process
            # group, loads its shard and publishes every device command to the followers
            import dataclasses

            import torch
            from .parallel.rank_worker import leader_engine
            if torch.cuda.is_available() and torch.cuda.device_count() < a.tp:
                raise SystemExit(f"--tp {a.tp} needs {a.tp} GPUs, "
                                 f"{torch.cuda.device_count()} visible")
            spec = dict(world=a.tp, device="cuda" if torch.cuda.is_available() else "cpu",
                        preset=a.preset, model_dir=a.model_dir, max_context=a.max_context,
                        draft_head=bool(getattr(a, "tp_draft_head", False)),
                        load={**dataclasses.asdict(load), "cuda_graph": load.cuda_graph.value},
                        sched={**dataclasses.asdict(sched), "policy": sched.policy.value})
            engine, team = leader_engine(spec, deadline_s=max(a.step_timeout_ms / 1e3, 30.0))
            teams.append(team)
            print(f"MODEL READY {name}; tensor parallel over {a.tp} ranks", file=sys.stderr,
                  flush=True)
            return engine
        weights, _ = _weights(a)
        if a.preset:
            print(f"MODEL READY {name}; {weights.nbytes() / 2 ** 20:.0f} MiB of weights",
                  file=sys.stderr, flush=True)
        return _engine_factory(a, weights, load, sched)()

    service = Service(factory, _codec(a, SimpleNamespace(config=cfg), name), name,
                      json.loads(a.default_request_params), a.queue_timeout_ms,
                      a.output_timeout_ms, a.preparation_workers, a.preparation_memory_mib,
                      a.step_timeout_ms, exit_on_stall=True)
    server = uvicorn.Server(uvicorn.Config(
        create_app(service, body_limit=getattr(a, "request_body_mib", 32) << 20),
        host=host, port=int(port), log_level="warning"))
    service.start(wait=False)

    def announce():
        service.worker.ready.wait()
        if service.lifecycle.state != "ready":
            print(f"worker failed: {service.lifecycle.reason}", file=sys.stderr, flush=True)
            server.should_exit = True
            return
        print("WORKER READY", file=sys.stderr)
        print("WARMUP READY", file=sys.stderr)
        print(f"API READY http://{a.listen}/v1; context {service.worker.engine.max_context}; "
              f"continuous_batching=true", file=sys.stderr, flush=True)
    threading.Thread(target=announce, daemon=True).start()

    def drain(*_):
        service.lifecycle.set("draining")
        server.should_exit = True
    signal.signal(signal.SIGINT, drain)
    signal.signal(signal.SIGTERM, drain)
    server.run()
    if service.worker.engine is None:                 # never became ready
        return 1
    service.stop(a.drain_timeout_ms)
    print("SCHEDULER " + json.dumps(service.worker.engine.stats.as_dict()), file=sys.stderr)
    code = 1 if service.lifecycle.state == "failed" else 0
    for team in teams:                                # graphs, peer mappings, followers, group
        team.close(service.worker.engine)
    return code


def _model_identity(a):
    """(geometry, name) of the model to serve without reading any weights."""
    from .config import ModelConfig
    if a.preset:
        return PRESETS[a.preset], a.preset
    if not a.model_dir:
        raise SystemExit("a model directory or --preset is required")
    from .engine.checkpoint import read_descriptor
    cfg = ModelConfig.from_json((Path(a.model_dir) / "config.json").read_text())
    return cfg, read_descriptor(a.model_dir)["name"]


def _state_dir(a) -> Path:
    import os
    return Path(getattr(a, "state_dir", None) or os.environ.get("ORINFER_STATE_DIR")
                or Path.home() / ".local" / "share" / "orinfer")


def _serve_manager(a, host: str, port: int, load, sched) -> int:
    """`orinfer serve` without a model: every registered model behind one listener, runners
    started on demand under the memory budget and retired by keep-alive."""
    import copy

    import uvicorn
    from .api.child_runner import weight_bytes
    from .api.manager import ModelManager, RunnerHandle, create_gateway_app
    from .api.server import Service, create_app

    def start(entry):
        args = copy.copy(a)
        args.model_dir, args.preset = entry.path, None
        weights, name = _weights(args)
        svc = Service(_engine_factory(args, weights, load, sched), _codec(args, weights, entry.name),
                      entry.name, json.loads(a.default_request_params),   # per-name defaults: gateway
                      a.queue_timeout_ms, a.output_timeout_ms, a.preparation_workers,
                      a.preparation_memory_mib)
        svc.start()
        if svc.lifecycle.state != "ready":
            raise RuntimeError(svc.lifecycle.reason or "worker failed")
        return RunnerHandle(svc, create_app(svc)), weights.nbytes()

    def start_process(entry):
        from .api.child_runner import ChildRunner, ProxyApp, weight_bytes
        extra = ["--device", a.device, "--cuda-graph", str(a.cuda_graph),
                 "--scheduler-policy", str(a.scheduler_policy),
                 "--max-active-requests", str(a.max_active_requests),
                 "--prefix-cache-mib", str(a.prefix_cache_mib), "--tp", str(a.tp),
                 "--default-request-params",
                 a.default_request_params]           # per-name defaults are applied by the gateway
        if a.max_context:
            extra += ["--max-context", str(a.max_context)]
        child = ChildRunner(entry.path, entry.name, extra,
                            start_timeout_s=getattr(a, "load_timeout_s", 600.0)).start()
        return RunnerHandle(child, ProxyApp(child.base_url)), weight_bytes(entry.path)

    process = getattr(a, "runners", "process") == "process"

    def stop(handle):                       # ChildRunner.stop takes seconds, Service.stop ms
        handle.service.stop(a.drain_timeout_ms / 1e3 if process else a.drain_timeout_ms)

    manager = ModelManager(_state_dir(a), start_process if process else start, stop,
                           memory_budget_bytes=getattr(a, "memory_budget_mib", 0) << 20,
                           estimate=lambda entry: weight_bytes(entry.path),
                           max_loaded=getattr(a, "max_loaded_models", 0),
                           capacity_wait_s=getattr(a, "capacity_wait_ms", 30000) / 1e3)
    print(f"API READY http://{a.listen}/v1; manager with {len(manager.list())} models",
          file=sys.stderr)
    uvicorn.Server(uvicorn.Config(create_gateway_app(manager), host=host, port=port,
                                  log_level="warning")).run()
    return 0


def cmd_models(a) -> int:
    from .api.manager import ManagerError, ModelManager
    m = ModelManager(_state_dir(a), lambda e: (_ for _ in ()).throw(RuntimeError("offline")),
                     lambda h: None)
    try:
        if a.models_cmd == "import":
            from .engine.checkpoint import validate_model
            validate_model(a.path)
            e = m.register(a.name, str(Path(a.path).resolve()))
            print(json.dumps(e.__dict__))
        elif a.models_cmd == "pull":
            import os
            from .api.pull import PullError, pull
            from .engine.checkpoint import validate_model
            try:
                snap = pull(a.source, _state_dir(a), os.environ.get("HF_TOKEN"),
                            progress=lambda n, i, k: print(f"[{i + 1}/{k}] {n}", file=sys.stderr))
            except PullError as e:
                print(str(e), file=sys.stderr)
                return 2
            validate_model(snap)
            print(json.dumps(m.register(a.name, str(snap)).__dict__))
        elif a.models_cmd == "logs":
            import requests
            r = _session().get(a.url.rstrip("/") + "/api/logs", params={"model": a.name},
                               timeout=10)
            if r.status_code != 200:
                print(r.text, file=sys.stderr)
                return 2
            print("\n".join(r.json()["lines"]))
        elif a.models_cmd == "list":
            print(json.dumps([e.__dict__ for e in m.list()]))
        elif a.models_cmd == "show":
            print(json.dumps(m.show(a.name).__dict__))
        elif a.models_cmd == "cp":
            print(json.dumps(m.copy(a.name, a.destination).__dict__))
        elif a.models_cmd == "rm":
            m.remove(a.name)
    except ManagerError as e:
        print(str(e), file=sys.stderr)
        return 2
    return 0


def cmd_batch(a) -> int:
    from .api.batch_jsonl import BatchError, run_batch
    load, sched = _options(a)
    weights, name = _weights(a)
    engine = _engine_factory(a, weights, load, sched)()
    try:
        counts = run_batch(engine, _codec(a, weights, name), a.input, a.output, resume=a.resume,
                           order=a.batch_order,
                           default_request_params=json.loads(a.default_request_params),
                           model_id=name)
    except BatchError as e:
        print(f"batch failed: {e}", file=sys.stderr)
        return 2
    print(json.dumps(counts))
    print("SCHEDULER " + json.dumps(engine.stats.as_dict()), file=sys.stderr)
    return 0 if counts["failed"] == 0 else 3


def cmd_validate_model(a) -> int:
    from .engine.checkpoint import CheckpointError, validate_model
    try:
        print(json.dumps(validate_model(a.model_dir)))
        return 0
    except CheckpointError as e:
        print(f"invalid model: {e}", file=sys.stderr)
        return 1


def cmd_plan_model(a) -> int:
    """Static plan: geometry, per-layer projections and formats, weight / KV bytes."""
    from .engine.checkpoint import read_descriptor
    from .config import ModelConfig
    from .models.runner import KVPool
    if a.preset:
        cfg = PRESETS[a.preset]
    else:
        read_descriptor(a.model_dir)
        cfg = ModelConfig.from_json((Path(a.model_dir) / "config.json").read_text())
    layers = [{"layer": i, "kind": "attention" if cfg.is_full_attention(i) else "gdn",
               "ffn": "moe" if cfg.experts else "dense"} for i in range(cfg.layers)]
    from .config import LoadOptions, SchedulerOptions
    from .engine.plan import PlanError, validate_plan
    descriptor = None if a.preset else read_descriptor(a.model_dir)
    try:
        plan = validate_plan(cfg, LoadOptions(), SchedulerOptions(),
                             max_context=getattr(a, "max_context", None),
                             world=getattr(a, "tp", None) or 1,
                             device_bytes=(getattr(a, "device_gib", None) or 180) << 30,
                             descriptor=descriptor, exhaustive=True)
    except PlanError as e:
        print(json.dumps({"model": cfg.name, "ok": False, "error": str(e)}))
        return 2
    print(json.dumps({"model": cfg.name, "target": "sm_100a", "ok": True,
                      "memory_plan": plan.as_dict(), "layers": layers,
                      "kv_bytes_per_token": cfg.kv_bytes_per_token(),
                      "kv_bytes_per_page": KVPool.bytes_per_page(cfg, cfg.mtp_layers),
                      "programs": ["prefill", "decode", "mixed", "verify"],
                      "graph_modes": ["decode_only", "full", "off"]}, indent=1))
    return 0


def cmd_run_model(a) -> int:
    """Token-id requests from a JSON file ``{"requests":[{"id", "input_tokens",
    "max_new_tokens"}]}``; reports prefill / decode timings per request
    (crates/orinfer-engine/src/runtime/benchmark.rs:57-212)."""
    import torch
    load, sched = _options(a)
    weights, _ = _weights(a)
    engine = _engine_factory(a, weights, load, sched)()
    spec = json.loads(Path(a.requests).read_text())
    report = []
    for item in spec["requests"]:
        t0 = time.perf_counter()
        req = engine.submit(item["input_tokens"], item.get("max_new_tokens", 16),
                            ignore_eos=True)
        while not req.generated:
            engine.step()
        ttft = time.perf_counter() - t0
        while not req.finished:
            engine.step()
        total = time.perf_counter() - t0
        n_in, n_new = len(req.prompt), len(req.generated)
        report.append({"id": item.get("id"), "ttft_s": ttft, "decode_s": total - ttft,
                       "prefill_tps": n_in / ttft,
                       "decode_tps": (n_new - 1) / max(total - ttft, 1e-9),
                       "tokens": req.generated})
    print(json.dumps({"timing_scope": "no MTP, fixed output length", "requests": report}))
    return 0


def cmd_score_model(a) -> int:
    """Teacher-forced next-token log-probabilities of ``--tokens`` (prefix cache and MTP off)."""
    import numpy as np
    import torch
    from .core import sampling as S
    from .models.runner import Packet
    load, sched = _options(a)
    load.prefix_cache_bytes = 0
    weights, _ = _weights(a)
    engine = _engine_factory(a, weights, load, sched)()
    ids = [int(x) for x in a.tokens.split(",")]
    dev = engine.device
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    pages = engine.pool.take((len(ids) + 127) // 128)
    table = torch.zeros(1, engine.max_pages_per_req, dtype=torch.int32, device=dev)
    table[0, :len(pages)] = t(pages)
    p = Packet(t(ids), t([0] * len(ids)), t(list(range(len(ids)))), table, len(ids), len(ids))
    _, logits = engine.runner.greedy(p)
    logits = logits.float().cpu().numpy()
    if a.jsonl:
        from .bench import quality as Q
        query = Q.queries_from(Q.read_jsonl(a.query_from)) if a.query_from else None
        probes = Q.probes_from_logits(logits, ids, a.case_id, "prefill", query)
        Q.write_jsonl(a.jsonl, probes)
        print(json.dumps({"probes": len(probes), "file": a.jsonl}))
        return 0
    out = []
    opts = S.SamplingOptions()
    for i in range(len(ids) - 1):
        lp, top = S.logprobs(logits[i], [], opts, ids[i + 1], 3)
        out.append({"position": i + 1, "token": ids[i + 1], "logprob": lp, "top3": top})
    print(json.dumps({"nll": -float(np.mean([o["logprob"] for o in out])), "probes": out}))
    return 0


def cmd_generate(a) -> int:
    """One prompt through the single-request reference path (no batching, graphs, prefix cache
    or speculation): the isolation oracle, as token ids or text."""
    load, sched = _options(a)
    load.prefix_cache_bytes = 0
    weights, name = _weights(a)
    engine = _engine_factory(a, weights, load, sched)()
    codec = _codec(a, weights, name)
    if a.tokens:
        ids = [int(x) for x in a.tokens.split(",")]
    else:
        ids = codec.prepare({"messages": [{"role": "user", "content": a.prompt or "Hello"}],
                             "enable_thinking": False}).prompt_ids
    t0 = time.monotonic()
    out = engine.generate_reference(ids, a.max_tokens)
    print(json.dumps({"prompt_tokens": len(ids), "tokens": out,
                      "text": codec.tokenizer.decode(out), "seconds": time.monotonic() - t0}))
    return 0


def cmd_make_model(a) -> int:
    """Random-init weights of a preset geometry quantised to the checkpoint format."""
    import torch
    from .engine.checkpoint import save_model
    from .models.weights import random_model
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    w = random_model(PRESETS[a.preset], seed=a.seed, device=dev)
    print(save_model(w, a.output, a.preset))
    return 0


def cmd_package_install(a) -> int:
    from .engine import packages
    try:
        path = packages.install(a.archive, a.cache)
    except packages.PackageError as e:
        print(f"Package installation: {e}", file=sys.stderr)
        return 2
    print(json.dumps({"digest": path.name, "path": str(path)}))
    return 0


def cmd_package_create(a) -> int:
    from .engine import packages
    print(json.dumps({"digest": packages.create(a.model, a.output), "archive": a.output}))
    return 0


def cmd_devices(a) -> int:
    import torch
    devs = []
    for i in range(torch.cuda.device_count()):
        pr = torch.cuda.get_device_properties(i)
        devs.append({"index": i, "name": pr.name, "sm": f"{pr.major}{pr.minor}",
                     "memory_bytes": pr.total_memory, "multiprocessors": pr.multi_processor_count,
                     "supported": (pr.major, pr.minor) == (10, 0)})
    print(json.dumps({"target": "sm_100a", "devices": devs}))
    return 0


def cmd_info(a) -> int:
    from . import __version__
    from .ops import native
    from . import contracts
    from .core._lib import lib as core_lib
    try:
        core_lib()
        core = True
    except OSError:
        core = False
    print(json.dumps({
        "version": __version__, "target": contracts.TARGET,
        "compute_policy": contracts.COMPUTE_POLICY, "kernel_library": native.loaded(),
        "policy_core": core, "architectures": contracts.architectures(),
        "convertible": ["Qwen3ForCausalLM", "Qwen3MoeForCausalLM", "Qwen3NextForCausalLM",
                        "LlamaForCausalLM", "MistralForCausalLM"],
        "routes": ["/v1/chat/completions", "/v1/completions", "/v1/embeddings", "/v1/rerank",
                   "/v1/audio/transcriptions", "/api/chat", "/api/generate"],
        "presets": sorted(PRESETS)}))
    return 0


def cmd_validate_nccl(a) -> int:
    from .parallel.selftest import main as selftest
    return selftest(a.world)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="orinfer")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve")
    _load_args(s)
    s.add_argument("--listen", default="[::]:8088")
    s.add_argument("--queue-timeout-ms", type=int, default=0)
    s.add_argument("--output-timeout-ms", type=int, default=60000)
    s.add_argument("--preparation-workers", "--preprocess-workers", dest="preparation_workers",
                   type=int, default=4,
                   help="threads that render, tokenise and compile grammars for new requests")
    s.add_argument("--preparation-memory-mib", "--preprocess-memory-mib",
                   dest="preparation_memory_mib", type=int, default=1024,
                   help="host memory that requests being prepared may hold at once")
    s.add_argument("--request-body-mib", type=int, default=32,
                   help="largest HTTP request body that is read (413 beyond it)")
    s.add_argument("--max-loaded-models", type=int, default=0,
                   help="manager mode: at most this many models loaded at once (0 = as many "
                        "as the memory budget allows)")
    s.add_argument("--load-timeout-s", type=float, default=600.0,
                   help="manager mode: how long a model's runner process may take to start")
    s.add_argument("--gpu-lock", default=None,
                   help="directory of the per-GPU advisory locks; with it `serve` takes the "
                        "lock of its device and refuses to start while another holder has it")
    s.add_argument("--drain-timeout-ms", type=int, default=30000)
    s.add_argument("--step-timeout-ms", type=int, default=120000,
                   help="an engine step running longer fails the server closed and exits 70 "
                        "(0 disables the watchdog)")
    s.add_argument("--tool-format", choices=["xml", "dsml"], default="xml",
                   help="tool-call wire syntax the model emits")
    s.add_argument("--vision", action="store_true",
                   help="accept image_url parts (random-init vision tower unless the model "
                        "directory provides one)")
    s.add_argument("--image-cache-mib", type=int, default=256,
                   help="budget of the uuid image cache; 0 disables it")
    s.add_argument("--state-dir", default=None, help="manager registry (serve without a model)")
    s.add_argument("--runners", choices=["process", "inproc"], default="process",
                   help="manager mode: each model in its own child process (its memory returns "
                        "on retirement) or as services inside the gateway process")
    s.add_argument("--memory-budget-mib", type=int, default=0,
                   help="manager mode: evict idle models beyond this many MiB of weights")
    s.add_argument("--capacity-wait-ms", type=int, default=30000,
                   help="manager mode: how long a request waits for a model in use to go idle "
                        "when the memory budget leaves no room for its own model")
    s.set_defaults(fn=cmd_serve)
    b = sub.add_parser("batch")
    _load_args(b, batch=True)
    b.add_argument("--input", required=True)
    b.add_argument("--output", required=True)
    b.add_argument("--resume", action="store_true")
    b.add_argument("--batch-order", default="auto", choices=["input", "auto"])
    b.set_defaults(fn=cmd_batch)
    v = sub.add_parser("validate-model")
    v.add_argument("model_dir")
    v.set_defaults(fn=cmd_validate_model)
    pm = sub.add_parser("plan-model")
    pm.add_argument("model_dir", nargs="?")
    pm.add_argument("--preset", choices=sorted(PRESETS))
    pm.add_argument("--max-context", type=int, default=None)
    pm.add_argument("--tp", type=int, default=1, help="ranks the model is to be split over")
    pm.add_argument("--device-gib", type=int, default=180, help="memory of one device")
    pm.set_defaults(fn=cmd_plan_model)
    r = sub.add_parser("run-model")
    _load_args(r)
    r.add_argument("--requests", required=True)
    r.set_defaults(fn=cmd_run_model)
    sc = sub.add_parser("score-model")
    _load_args(sc)
    sc.add_argument("--tokens", required=True, help="comma-separated token ids")
    sc.add_argument("--jsonl", default=None, help="write paired-probe records to this file")
    sc.add_argument("--query-from", default=None,
                    help="baseline probe file whose top-3 ids are also scored")
    sc.add_argument("--case-id", default="case")
    sc.set_defaults(fn=cmd_score_model)
    ge = sub.add_parser("generate")
    _load_args(ge)
    ge.add_argument("--prompt", default=None)
    ge.add_argument("--tokens", default=None, help="comma-separated prompt token ids")
    ge.add_argument("--max-tokens", type=int, default=32)
    ge.set_defaults(fn=cmd_generate)
    cv = sub.add_parser("convert-model", help="Hugging Face Qwen3 checkpoint -> quantised model")
    cv.add_argument("source")
    cv.add_argument("output")
    cv.add_argument("--device", default="cuda")
    cv.add_argument("--exhaustive", action="store_true")
    cv.add_argument("--name", default=None)
    cv.add_argument("--format", action="append", default=[], metavar="KEY=FMT")
    cv.add_argument("--search", default="nearest", choices=["nearest", "beam8"])
    cv.set_defaults(fn=lambda a: __import__("orinfer_b200.quant.convert", fromlist=["main"]).main(
        [a.source, a.output, "--device", a.device, "--search", a.search]
        + (["--exhaustive"] if a.exhaustive else [])
        + (["--name", a.name] if a.name else []) + [x for f in a.format for x in ("--format", f)]))
    pm = sub.add_parser("promote-model",
                        help="re-encode chosen layers of a converted model as rotated W8")
    pm.add_argument("source", help="the original (unquantised) checkpoint directory")
    pm.add_argument("model_dir")
    pm.add_argument("output")
    pm.add_argument("--layers", required=True, help="comma-separated layer numbers")
    pm.add_argument("--device", default="cpu")
    pm.set_defaults(fn=lambda a: __import__("orinfer_b200.quant.promotion", fromlist=["main"]).main(
        [a.source, a.model_dir, a.output, "--layers", a.layers, "--device", a.device]))
    mk = sub.add_parser("make-model")
    mk.add_argument("--preset", required=True, choices=sorted(PRESETS))
    mk.add_argument("--output", required=True)
    mk.add_argument("--seed", type=int, default=0)
    mk.set_defaults(fn=cmd_make_model)
    mo = sub.add_parser("models")
    mo.add_argument("--state-dir", default=None)
    mos = mo.add_subparsers(dest="models_cmd", required=True)
    mi = mos.add_parser("import")
    mi.add_argument("name")
    mi.add_argument("path")
    mp = mos.add_parser("pull")
    mp.add_argument("name")
    mp.add_argument("source", help="hf:org/repo[@revision] or modelscope:org/repo[@revision]")
    ml = mos.add_parser("logs", help="recent stderr of a running model's process")
    ml.add_argument("name")
    ml.add_argument("--url", default="http://127.0.0.1:8088", help="address of the manager")
    mos.add_parser("list")
    for verb in ("show", "rm"):
        mv = mos.add_parser(verb)
        mv.add_argument("name")
    mc = mos.add_parser("cp")
    mc.add_argument("name")
    mc.add_argument("destination")
    mo.set_defaults(fn=cmd_models)
    pk = sub.add_parser("package")
    pks = pk.add_subparsers(dest="package_cmd", required=True)
    pi = pks.add_parser("install")
    pi.add_argument("archive")
    pi.add_argument("--cache", default=None)
    pi.set_defaults(fn=cmd_package_install)
    pc = pks.add_parser("create")
    pc.add_argument("model")
    pc.add_argument("--output", required=True)
    pc.set_defaults(fn=cmd_package_create)
    sub.add_parser("devices").set_defaults(fn=cmd_devices)
    sub.add_parser("info").set_defaults(fn=cmd_info)
    vn = sub.add_parser("validate-nccl")
    vn.add_argument("--world", type=int, default=0, help="ranks (0 = all visible GPUs)")
    vn.set_defaults(fn=cmd_validate_nccl)
    for verb, help_text in (("ps", "loaded models of a running manager"),
                            ("load", "start a model's runner before its first request"),
                            ("stop", "drain and unload a model, keeping its files"),
                            ("run", "send one prompt (argument or stdin) or chat interactively"),
                            ("transcribe", "transcribe an audio file")):
        c = sub.add_parser(verb, help=help_text)
        c.add_argument("--url", default="http://127.0.0.1:8088", help="server or manager")
        if verb != "ps":
            c.add_argument("name", help="model name")
        if verb == "load":
            c.add_argument("--keep-alive", default=None, help="seconds or a duration like 30m")
        if verb == "stop":
            c.add_argument("--force", action="store_true", help="end requests in flight")
        if verb == "run":
            c.add_argument("prompt", nargs="?", default=None)
            c.add_argument("--params", default="{}", help="JSON merged into every request")
        if verb == "transcribe":
            c.add_argument("input")
            c.add_argument("--language", default=None)
            c.add_argument("--prompt", default=None)
            c.add_argument("--max-tokens", dest="max_tokens", default=None)
        c.set_defaults(fn=cmd_client, verb=verb)
    bn = sub.add_parser("bench", help="HTTP benchmark clients against a running server, and "
                                       "device-timed kernel probes")
    bn.add_argument("tool", choices=sorted(BENCH_TOOLS))
    bn.add_argument("tool_args", nargs=argparse.REMAINDER)
    bn.set_defaults(fn=cmd_bench)
    return ap


def _session():
    """HTTP session of the client verbs; carries ``ORINFER_API_KEY`` as a bearer token."""
    import os

    import requests
    http = requests.Session()
    if os.environ.get("ORINFER_API_KEY"):
        http.headers["Authorization"] = "Bearer " + os.environ["ORINFER_API_KEY"]
    return http


def cmd_client(a) -> int:
    """Verbs that talk to a running server or manager over HTTP: ``ps``, ``load``, ``stop``,
    ``run`` (one prompt, piped stdin, or an interactive chat) and ``transcribe``."""
    import requests
    url = a.url.rstrip("/")
    http = _session()

    def fail(r) -> int:
        print(r.text.strip(), file=sys.stderr)
        return 2

    try:
        if a.verb == "ps":
            r = http.get(url + "/api/ps", timeout=10)
            if r.status_code != 200:
                return fail(r)
            print(json.dumps(r.json()["models"], indent=1))
        elif a.verb == "load":
            body = {"model": a.name}
            if a.keep_alive is not None:
                body["keep_alive"] = a.keep_alive
            r = http.post(url + "/api/load", json=body, timeout=3600)
            if r.status_code != 200:
                return fail(r)
            print(json.dumps(r.json()))
        elif a.verb == "stop":
            r = http.post(url + "/api/stop", json={"model": a.name, "force": a.force},
                              timeout=600)
            if r.status_code != 200:
                return fail(r)
            print(json.dumps(r.json()))
        elif a.verb == "transcribe":
            data = {"model": a.name}
            for key in ("language", "prompt", "max_tokens"):
                if getattr(a, key):
                    data[key] = getattr(a, key)
            with open(a.input, "rb") as f:
                r = http.post(url + "/v1/audio/transcriptions", data=data, timeout=3600,
                                  files={"file": (Path(a.input).name, f)})
            if r.status_code != 200:
                return fail(r)
            print(r.json()["text"])
        else:
            return _client_run(a, url)
    except requests.RequestException as e:
        print(f"cannot reach {url}: {e}", file=sys.stderr)
        return 3
    return 0


def _client_run(a, url: str) -> int:
    import requests
    params = json.loads(a.params)
    history = []

    def turn(text: str) -> int:
        history.append({"role": "user", "content": text})
        body = dict(params, model=a.name, messages=history, stream=True)
        reply = ""
        with requests.post(url + "/v1/chat/completions", json=body, stream=True,
                           timeout=3600) as r:
            if r.status_code != 200:
                print(r.text.strip(), file=sys.stderr)
                return 2
            for raw in r.iter_lines():
                if not raw.startswith(b"data: ") or raw == b"data: [DONE]":
                    continue
                ev = json.loads(raw[6:])
                if "error" in ev:
                    print(json.dumps(ev["error"]), file=sys.stderr)
                    return 2
                for choice in ev.get("choices") or []:
                    piece = (choice.get("delta") or {}).get("content") or ""
                    reply += piece
                    sys.stdout.write(piece)
                    sys.stdout.flush()
        sys.stdout.write("\n")
        history.append({"role": "assistant", "content": reply})
        return 0

    if a.prompt is not None:
        return turn(a.prompt)
    if not sys.stdin.isatty():
        return turn(sys.stdin.read())
    while True:                                   # interactive chat; an empty line or EOF ends it
        try:
            line = input(">>> ")
        except EOFError:
            return 0
        if not line.strip():
            return 0
        code = turn(line)
        if code:
            return code


BENCH_TOOLS = {"hf-reference": "hf_reference", "tokens": "token_bench", "quality": "quality", "concurrency": "concurrency", "agentic": "agentic", "startup": "startup",
               "encoders": "encoders", "scenario": "workloads",
               # device-timed probes of single kernels and of the fused tensor-parallel step
               # (the latter under torch.distributed.run, one rank per GPU)
               "kernel": "kernel_probe", "fused-step": "fused_probe"}


def cmd_bench(a) -> int:
    import importlib
    mod = importlib.import_module(f".bench.{BENCH_TOOLS[a.tool]}", __package__)
    return int(mod.main(a.tool_args) or 0)


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return int(args.fn(args) or 0)


if __name__ == "__main__":
    sys.exit(main())
