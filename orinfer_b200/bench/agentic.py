"""Synthetic agentic trace replay: trajectories of dependent chat requests whose prompts
extend their parents' conversations, replayed at a fixed concurrency under a wall limit.

Shape of the workload (tools/bench/mini_weka_synthetic.py, mini_weka_compact.py and
agentx_mini.py of the reference): every trajectory is the same seven-step dependency graph
``((), (0,), (1,), (1,), (2, 3), (4,), (5,))`` — a chain that forks after step 1 and joins at
step 4.  A step's conversation is its first parent's whole conversation (prompt + reply) plus
a new user turn, so replays keep their prefixes and a prefix cache can hit; the join step
quotes its second parent's reply in that turn.  Everything is generated from a seed, so two
runs send identical first-step prompts.  Reported: completed requests, fully completed
trajectories, output tokens per second over the wall time, TTFT p50 / p95, and the prefix hit
rate ``cached_tokens / prompt_tokens`` from the usage blocks.

    python -m orinfer_b200.bench.agentic --url http://127.0.0.1:8080 --trajectories 512 \
        --concurrency 4 --wall 240
"""

from __future__ import annotations

import argparse
import json
import random
import threading
import time

from .http_client import percentile, stream_chat

GRAPH = ((), (0,), (1,), (1,), (2, 3), (4,), (5,))
WORDS = ("alpha bravo charlie delta echo foxtrot golf hotel india juliet kilo lima mike november "
         "oscar papa quebec romeo sierra tango uniform victor whiskey xray yankee zulu").split()
TOOLS = ("search the repository", "open the failing test", "read the stack trace",
         "propose a patch", "compare both findings", "run the test suite", "write the summary")


class Trajectory:
    def __init__(self, index: int, seed: int, system_words: int, turn_words: int):
        self.index = index
        rng = random.Random(seed * 1_000_003 + index)
        # a system prompt shared by groups of 8 trajectories: hits across trajectories too
        shared = random.Random(seed * 7919 + index // 8)
        self.system = "You are a coding agent. " + " ".join(
            shared.choice(WORDS) for _ in range(system_words))
        self.turns = [f"Task {index}, step {s}: {TOOLS[s]}. Notes: " +
                      " ".join(rng.choice(WORDS) for _ in range(turn_words))
                      for s in range(len(GRAPH))]
        self.replies = [None] * len(GRAPH)
        self.conversations = [None] * len(GRAPH)
        self.issued = [False] * len(GRAPH)

    def ready(self):
        return [s for s, parents in enumerate(GRAPH)
                if not self.issued[s] and all(self.replies[p] is not None for p in parents)]

    def messages(self, step: int):
        parents = GRAPH[step]
        if not parents:
            base = [{"role": "system", "content": self.system}]
        else:
            base = list(self.conversations[parents[0]]) + [
                {"role": "assistant", "content": self.replies[parents[0]]}]
        turn = self.turns[step]
        for other in parents[1:]:
            turn += f"\nFinding of step {other}: {self.replies[other]}"
        msgs = base + [{"role": "user", "content": turn}]
        self.conversations[step] = msgs
        return msgs

    @property
    def complete(self):
        return all(r is not None for r in self.replies)


def run(url: str, trajectories: int = 16, concurrency: int = 4, wall_s: float = 240.0,
        max_tokens: int = 48, seed: int = 20261002, temperature: float = 1.0,
        system_words: int = 120, turn_words: int = 40, in_flight_trajectories: int | None = None,
        timeout: float = 600.0) -> dict:
    trajs = [Trajectory(i, seed, system_words, turn_words) for i in range(trajectories)]
    window = in_flight_trajectories or concurrency
    lock = threading.Condition()
    state = {"opened": 0, "results": [], "stop": False, "running": 0}
    t0 = time.perf_counter()

    def next_step():
        """Under the lock: a ready (trajectory, step), opening new trajectories up to the
        window; None when nothing is ready now; "end" when all work has been handed out."""
        live = [t for t in trajs[:state["opened"]] if not t.complete]
        for t in live:
            r = t.ready()
            if r:
                return t, r[0]
        if len(live) < window and state["opened"] < len(trajs):
            t = trajs[state["opened"]]
            state["opened"] += 1
            return t, 0
        if not live and state["opened"] >= len(trajs):
            return "end"
        return None

    def worker():
        while True:
            with lock:
                while True:
                    if state["stop"] or time.perf_counter() - t0 >= wall_s:
                        state["stop"] = True
                        lock.notify_all()
                        return
                    pick = next_step()
                    if pick == "end":
                        if state["running"] == 0:
                            state["stop"] = True
                            lock.notify_all()
                            return
                    elif pick is not None:
                        break
                    lock.wait(timeout=0.05)
                traj, step = pick
                traj.issued[step] = True
                msgs = traj.messages(step)
                state["running"] += 1
            body = {"messages": msgs, "max_tokens": max_tokens, "temperature": temperature,
                    "seed": seed + traj.index * 16 + step, "ignore_eos": True,
                    "enable_thinking": False}
            r = stream_chat(url, body, timeout=timeout)
            with lock:
                state["running"] -= 1
                finished_in_time = r.ok and (r.end - t0) <= wall_s
                if r.ok:
                    traj.replies[step] = r.text or " "
                else:
                    traj.replies[step] = " "      # do not block the dependants on a failure
                state["results"].append((traj.index, step, r, finished_in_time))
                lock.notify_all()

    threads = [threading.Thread(target=worker, daemon=True) for _ in range(concurrency)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = min(time.perf_counter() - t0, wall_s) or 1e-9
    counted = [r for _, _, r, in_time in state["results"] if in_time]
    per_traj = {}
    for ti, _, r, in_time in state["results"]:
        per_traj[ti] = per_traj.get(ti, 0) + (1 if in_time else 0)
    prompt = sum(r.prompt_tokens for r in counted)
    cached = sum(r.cached_tokens for r in counted)
    out = sum(r.completion_tokens for r in counted)
    return {"trajectories": trajectories, "concurrency": concurrency, "wall_s": wall,
            "completed_requests": len(counted),
            "failed_requests": sum(1 for _, _, r, _ in state["results"] if not r.ok),
            "full_trajectories": sum(1 for v in per_traj.values() if v == len(GRAPH)),
            "output_tokens": out, "output_tps": out / wall,
            "ttft_p50_s": percentile([r.ttft_s for r in counted], 50),
            "ttft_p95_s": percentile([r.ttft_s for r in counted], 95),
            "prompt_tokens": prompt, "cached_tokens": cached,
            "prefix_hit_rate": cached / prompt if prompt else 0.0}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--url", default="http://127.0.0.1:8080")
    ap.add_argument("--trajectories", type=int, default=512)
    ap.add_argument("--concurrency", type=int, default=4)
    ap.add_argument("--wall", type=float, default=240.0)
    ap.add_argument("--max-tokens", type=int, default=48)
    ap.add_argument("--seed", type=int, default=20261002)
    ap.add_argument("--temperature", type=float, default=1.0)
    a = ap.parse_args(argv)
    print(json.dumps(run(a.url, a.trajectories, a.concurrency, a.wall, a.max_tokens, a.seed,
                         a.temperature), indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
