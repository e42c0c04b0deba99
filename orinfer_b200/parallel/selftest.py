"""``orinfer validate-nccl``: multi-rank self-test of the communication layer.

Mirrors the reference's ``validate-hccl`` (crates/orinfer-engine/src/backend/ascend/hccl/
validation.rs:41-68,98,191-196): a *preflight gate* first - every rank reports that its
device opened and has >= 512 MiB free, and no rank joins a collective unless all ranks
passed within 30 s (so a bad rank cannot hang its peers inside a collective) - then
all-reduce, all-gather, reduce-scatter, uneven all-to-all, and a captured graph replayed
with changed inputs.  Runs over NCCL on GPUs or gloo on CPU ranks.
"""

from __future__ import annotations

import os
import sys
import time
from typing import List

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

PREFLIGHT_S = 30.0
MIN_FREE = 512 << 20


def _preflight(rank: int, world: int, store, use_cuda: bool) -> None:
    ok, why = True, ""
    try:
        if use_cuda:
            torch.cuda.set_device(rank)
            free, _ = torch.cuda.mem_get_info()
            if free < MIN_FREE:
                ok, why = False, f"only {free >> 20} MiB free"
    except Exception as e:                            # device did not open
        ok, why = False, str(e)
    store.set(f"preflight/{rank}", "ok" if ok else "fail:" + why)
    deadline = time.monotonic() + PREFLIGHT_S
    for r in range(world):
        while True:
            try:
                val = store.get(f"preflight/{r}").decode()
                break
            except Exception:
                if time.monotonic() > deadline:
                    raise RuntimeError(f"rank {r} did not report within {PREFLIGHT_S:.0f} s")
                time.sleep(0.05)
        if val != "ok":
            raise RuntimeError(f"rank {r} failed preflight: {val}")


def run_checks(rank: int, world: int, dev) -> List[str]:
    done = []
    x = torch.full((1024,), float(rank + 1), device=dev)
    dist.all_reduce(x)
    assert float(x[0]) == world * (world + 1) / 2
    done.append("all_reduce")
    parts = [torch.empty(8, device=dev) for _ in range(world)]
    dist.all_gather(parts, torch.full((8,), float(rank), device=dev))
    assert [float(p[0]) for p in parts] == list(map(float, range(world)))
    done.append("all_gather")
    out = torch.empty(4, device=dev)
    dist.reduce_scatter(out, [torch.full((4,), float(rank + r), device=dev)
                              for r in range(world)])
    assert float(out[0]) == sum(range(world)) + world * rank
    done.append("reduce_scatter")
    if dev.type == "cuda" or dist.get_backend() == "gloo":
        # uneven all-to-all: rank r sends (d + 1) elements to rank d
        send = [torch.full((d + 1,), float(rank), device=dev) for d in range(world)]
        recv = [torch.empty(rank + 1, device=dev) for _ in range(world)]
        dist.all_to_all(recv, send) if dev.type == "cuda" else _a2a_gloo(recv, send, rank, world)
        assert [float(r[0]) for r in recv] == list(map(float, range(world)))
        done.append("all_to_all_v")
    if dev.type == "cuda":
        buf = torch.ones(256, device=dev)
        dist.all_reduce(buf)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            dist.all_reduce(buf)
        for v in (2.0, 5.0):
            buf.fill_(v)
            g.replay()
            torch.cuda.synchronize()
            assert float(buf[0]) == v * world
        done.append("graph_replay_changed_input")
    return done


def _a2a_gloo(recv, send, rank, world):
    reqs = []
    for d in range(world):
        if d == rank:
            recv[d].copy_(send[d])
        else:
            reqs.append(dist.isend(send[d], d))
            reqs.append(dist.irecv(recv[d], d))
    for r in reqs:
        r.wait()


def _worker(rank: int, world: int, port: int, use_cuda: bool, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    store = dist.TCPStore("127.0.0.1", port + 1, world, rank == 0, timeout=
                          __import__("datetime").timedelta(seconds=60))
    _preflight(rank, world, store, use_cuda)
    dev = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world,
                            **({"device_id": dev} if use_cuda else {}))
    checks = run_checks(rank, world, dev)
    if rank == 0:
        out.put(checks)
    dist.barrier()
    if use_cuda:
        torch.cuda.synchronize()
        os._exit(0)
    dist.destroy_process_group()


def main(world: int = 0, use_cuda: bool = None, port: int = 0) -> int:
    if use_cuda is None:
        use_cuda = torch.cuda.is_available()
    if world <= 0:
        world = torch.cuda.device_count() if use_cuda else 2
    port = port or 29700 + os.getpid() % 200
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = mp.spawn(_worker, args=(world, port, use_cuda, out), nprocs=world, join=False)
    deadline = time.time() + 180
    while not procs.join(timeout=2):
        if time.time() > deadline:
            for p in procs.processes:
                if p.is_alive():
                    p.kill()
            print("validate-nccl: ranks did not finish within 180 s", file=sys.stderr)
            return 1
    checks = out.get(timeout=5)
    print(f"validate-nccl ok: world={world} backend={'nccl' if use_cuda else 'gloo'} "
          f"checks={','.join(checks)}")
    return 0
