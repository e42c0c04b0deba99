"""Follower ranks of a tensor-parallel server, and the leader-side code that starts and
watches them.

``orinfer serve --tp N`` keeps the HTTP server, the scheduler and every decision in the
process of rank 0.  Ranks 1..N-1 are child processes running ``follower_main``: each joins
the NCCL (or, on CPU, gloo) process group, loads its own shard, builds an ``Engine`` that is
never stepped, and replays the device commands the leader publishes over the rank channel
(``rank_channel.py``).  A follower that fails reports it and leaves; a follower that dies or
stops acknowledging is noticed by the leader's channel or supervisor, and the service fails
closed.  A follower never outlives its leader: a closed connection ends it.

    python -m orinfer_b200.parallel.rank_worker '<json spec>'      # started by the leader

Role of the reference's rank workers
(crates/orinfer-engine/src/models/deepseek_v41/team.rs:286-345, team/channel.rs:202-260).
"""

from __future__ import annotations

import datetime
import json
import os
import subprocess
import sys
import threading
import time
from typing import List, Optional

from .rank_channel import FollowerChannel, LeaderChannel, RankFailure, new_address


def init_group(rank: int, world: int, port: int, device: str, timeout_s: float):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    kw = dict(rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
    if device == "cuda":
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank), **kw)
        return torch.device("cuda", rank)
    dist.init_process_group("gloo", **kw)
    return torch.device("cpu")


def load_shard(spec: dict, rank: int, world: int, device):
    """This rank's weights: a preset is created directly in the sharded geometry; a model
    directory is loaded and cut down to the shard."""
    import dataclasses
    from ..config import PRESETS
    from .tp import random_shard, shard_model
    # ``draft_head``: shard the model's draft head too (speculation with it then runs on every
    # rank through published commands); off unless asked for
    draft = bool(spec.get("draft_head", False))
    if spec.get("preset"):
        cfg = PRESETS[spec["preset"]]
        if spec.get("mtp_layers") is not None:
            cfg = dataclasses.replace(cfg, mtp_layers=int(spec["mtp_layers"]))
        return random_shard(cfg, rank, world, device, seed=0, draft_head=draft)
    from ..engine.checkpoint import load_model
    # cut the shard out on the host and upload only that: no rank holds the whole model on
    # its device (and the loader's arena of the whole model is released with the host copy)
    shard = shard_model(load_model(spec["model_dir"], "cpu", verify=False), rank, world,
                        draft_head=draft)
    out = shard.to(device)
    out.tp, out.global_config = shard.tp, shard.global_config
    return out


def build_engine(spec: dict, weights, channel=None):
    import dataclasses
    from ..config import GraphMode, LoadOptions, Policy, SchedulerOptions
    from ..engine.engine import Engine
    load = LoadOptions(**{**spec["load"], "cuda_graph": GraphMode(spec["load"]["cuda_graph"])})
    sched = SchedulerOptions(**{**spec["sched"], "policy": Policy(spec["sched"]["policy"])})
    # Every device-side effect of a leader's decision is a published command, so the leader
    # keeps the host-side machinery and followers, which take no decisions, need none of it:
    # the radix prefix cache (page-table rows are published), its host tier (one command per
    # page move, carried out by every rank on its own shard), the recurrent-state copies of
    # hybrid models (taken, restored and dropped under handles the leader chooses) and
    # prompt-lookup speculation (verification packets and, for recurrent layers, the commit of
    # the accepted rows) and, when the shards carry a draft head, its captures, draft rounds
    # and backlog clean-up.
    leader = channel is not None
    offload = load.kv_offload_bytes
    load = dataclasses.replace(
        load, prefix_cache_bytes=load.prefix_cache_bytes if leader else 0,
        kv_offload_bytes=offload if leader else 0,
        mtp_drafts=load.mtp_drafts if leader else 0,
        prompt_lookup=load.prompt_lookup and leader)
    engine = Engine(weights, load=load, sched=sched, max_context=spec.get("max_context"),
                    kv_pages=spec.get("kv_pages"), max_rows=spec.get("max_rows"),
                    channel=channel)
    if not leader and offload > 0 and spec["load"].get("prefix_cache_bytes", 0) > 0:
        from ..engine.offload import HostKvStore
        engine.host_kv = HostKvStore(engine.kv, offload)
    return engine


def follower_main(spec: dict) -> int:
    rank, world = spec["rank"], spec["world"]
    from . import affinity
    affinity.bind_rank(rank, world)          # before the device context and reader threads
    device = init_group(rank, world, spec["port"], spec["device"], spec["group_timeout_s"])
    if device.type == "cpu":
        # CPU ranks share the host's cores: every rank spinning up a full-width thread pool
        # for each small operator costs far more than it gives
        import torch
        torch.set_num_threads(max(1, (os.cpu_count() or 1) // (2 * world)))
    # join the channel before building the engine: the leader builds its own engine after it
    # has admitted every follower, and a fused runner's constructor is collective
    ch = FollowerChannel(spec["address"], bytes.fromhex(spec["authkey"]), rank)
    weights = load_shard(spec, rank, world, device)
    engine = build_engine(spec, weights)
    stall_after = spec.get("test_stall_after")          # tests: stop replying after n commands
    done = 0
    code = 0
    while True:
        msg = ch.recv(1.0)
        if msg is None:
            continue
        seq, op, payload = msg
        if op == "close":
            break
        if stall_after is not None and done >= stall_after:
            time.sleep(3600)
        try:
            engine.apply(op, payload)
        except Exception as exc:                        # noqa: BLE001 - report and leave
            ch.fail(f"{type(exc).__name__}: {exc}")
            code = 1
            break
        word = engine._status.value() if engine._status is not None else 0
        if word:
            ch.fail(f"device status {word:#x}")
            code = 1
            break
        for key in engine.take_graph_misses():
            ch.miss(key)
        ch.ack(seq)
        done += 1
    # An orderly close is collective: the leader closes its own engine and destroys the group
    # at the same point.  After a failure nobody waits for anybody.
    try:
        engine.close(collective=code == 0)
    except Exception:                                   # noqa: BLE001 - leaving anyway
        pass
    ch.close()
    _leave_group(orderly=code == 0)
    return code


def _leave_group(orderly: bool) -> None:
    """Gives up the process group.  Orderly: every rank destroys it at the same point of the
    close.  After a failure, destroying an NCCL group would wait for peers that are not coming,
    so its communicators are aborted instead (gloo has no such wait)."""
    import torch.distributed as dist
    if not dist.is_initialized():
        return
    try:
        if orderly or dist.get_backend() != "nccl":
            dist.destroy_process_group()
        else:
            from torch.distributed.distributed_c10d import _abort_process_group
            _abort_process_group()
    except Exception:                                   # noqa: BLE001 - peers may be gone
        pass


class RankTeam:
    """Leader side: starts the follower processes, admits them to the channel and watches
    them.  ``channel`` is what the leader's ``Engine`` publishes to."""

    def __init__(self, spec: dict, *, deadline_s: float = 30.0, accept_s: float = 600.0):
        self.world = spec["world"]
        authkey = os.urandom(16)
        self.channel = LeaderChannel(self.world, new_address(str(spec["port"])), authkey,
                                     deadline_s=deadline_s, accept_s=accept_s)
        self.procs: List[subprocess.Popen] = []
        env = dict(os.environ)
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
        for rank in range(1, self.world):
            child = dict(spec, rank=rank, address=self.channel.address, authkey=authkey.hex())
            self.procs.append(subprocess.Popen(
                [sys.executable, "-m", "orinfer_b200.parallel.rank_worker", json.dumps(child)],
                env=env))
        self._stop = threading.Event()
        self._watch = threading.Thread(target=self._supervise, daemon=True)
        self._watch.start()

    def _supervise(self) -> None:
        """A follower process that exits while the team is live is a failure, at once."""
        while not self._stop.wait(0.2):
            for i, p in enumerate(self.procs):
                if p.poll() is not None and self.channel.failure is None and not self._stop.is_set():
                    self.channel.failure = RankFailure(i + 1, f"process exited with {p.returncode}")

    def admit(self) -> None:
        self.channel.accept_all()

    def close(self, engine=None, wait_s: float = 20.0) -> None:
        """Ends the team.  Orderly (no failure recorded): the followers get the close command,
        then every rank, this one included, closes its engine (the runners meet at a barrier
        before they unmap each other's memory) and destroys the process group, all at the same
        point.  After a failure the followers are ended and this rank gives up the group
        without waiting for anybody (an NCCL group is aborted, not destroyed)."""
        self._stop.set()
        orderly = self.channel.failure is None and all(p.poll() is None for p in self.procs)
        self.channel.close()
        if engine is not None:
            try:
                engine.close(collective=orderly)
            except Exception:                           # noqa: BLE001 - leaving anyway
                orderly = False
        if orderly:
            _leave_group(True)
        end = time.monotonic() + wait_s
        for p in self.procs:
            try:
                p.wait(max(0.1, end - time.monotonic()))
            except subprocess.TimeoutExpired:
                p.kill()
        if not orderly:
            _leave_group(False)


def free_port() -> int:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def leader_engine(spec: dict, *, deadline_s: float = 30.0):
    """Starts the followers, joins the group as rank 0, loads rank 0's shard and returns
    ``(engine, team)``; the engine publishes to the team's channel."""
    spec = dict(spec, rank=0)
    spec.setdefault("port", free_port())
    spec.setdefault("group_timeout_s", 120.0)
    from . import affinity
    affinity.configured(spec["world"])       # a bad placement fails before any rank starts
    team = RankTeam(spec, deadline_s=deadline_s)
    try:
        affinity.bind_rank(0, spec["world"])
        device = init_group(0, spec["world"], spec["port"], spec["device"],
                            spec["group_timeout_s"])
        team.admit()
        weights = load_shard(spec, 0, spec["world"], device)
        engine = build_engine(spec, weights, channel=team.channel)
    except Exception:
        team.close(wait_s=1.0)
        raise
    return engine, team


if __name__ == "__main__":
    sys.exit(follower_main(json.loads(sys.argv[1])))
