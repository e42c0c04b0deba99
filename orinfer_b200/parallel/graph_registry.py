"""Python face of the graph registry (``csrc/dist/graph_registry.cpp``): per-rank pools of
captured CUDA graphs keyed by launch geometry, with the rule that keeps the ranks' pools in
step (probe on every rank; a miss anywhere invalidates the geometry everywhere and all ranks
capture again).

The registry stores integer handles; ``GraphPool`` keeps the Python objects behind them (the
``torch.cuda.CUDAGraph`` and its static buffers) and drops an object as soon as the registry
hands its handle back (eviction, invalidation, clear).

Counterpart of the reference's graph-callback registry and probe-then-recapture rule
(crates/orinfer-engine/native/ascend/hccl_graph_registry.cc,
crates/orinfer-engine/src/backend/ascend/graph.rs).
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_int, c_longlong, c_uint64, c_void_p
from typing import Any, Dict, Hashable, Optional, Tuple

from ..core._lib import lib

RUN_DIRECT, CAPTURE, REPLAY = 0, 1, 2
E_ARG, E_STICKY, E_TIMEOUT, E_STALE = -1, -2, -3, -4
_ERRORS = {E_ARG: "bad argument", E_STICKY: "registry already failed",
           E_TIMEOUT: "a rank did not vote in time", E_STALE: "pools disagree"}


class GraphRegistryError(RuntimeError):
    """Fatal (error-taxonomy kind ``Peer``): the ranks' graph pools cannot be kept in step."""

    def __init__(self, code: int, rank: int = -1):
        super().__init__(f"graph registry: {_ERRORS.get(code, code)} (rank {rank})")
        self.code, self.rank = code, rank


def _setup():
    L = lib()
    L.orinfer_greg_create.restype = c_void_p
    L.orinfer_greg_create.argtypes = [c_int, c_int, c_int]
    L.orinfer_greg_destroy.argtypes = [c_void_p]
    L.orinfer_greg_probe.argtypes = [c_void_p, c_int, c_uint64]
    out = [POINTER(c_longlong), POINTER(c_longlong), POINTER(c_int)]
    L.orinfer_greg_decide.argtypes = [c_void_p, c_int, c_uint64, c_int] + out
    L.orinfer_greg_follow.argtypes = [c_void_p, c_int, c_uint64, c_int] + out + [POINTER(c_int)]
    L.orinfer_greg_commit.argtypes = [c_void_p, c_int, c_uint64, c_longlong, c_int]
    L.orinfer_greg_evict.restype = c_longlong
    L.orinfer_greg_evict.argtypes = [c_void_p, c_int, c_uint64]
    L.orinfer_greg_clear.argtypes = [c_void_p, c_int, POINTER(c_longlong), c_int]
    L.orinfer_greg_vote.argtypes = [c_void_p, c_int, c_uint64, c_int, c_int]
    L.orinfer_greg_fail.argtypes = [c_void_p, c_int, c_int]
    L.orinfer_greg_status.argtypes = [c_void_p, POINTER(c_int)]
    L.orinfer_greg_stats.argtypes = [c_void_p, POINTER(c_longlong)]
    return L


def key_of(geometry: Hashable) -> int:
    """64-bit key of a launch geometry (a tuple of ints / bools / nested tuples: Python's hash
    of those is the same in every process, so ranks agree on it)."""
    return hash(geometry) & 0xFFFFFFFFFFFFFFFF


class GraphRegistry:
    def __init__(self, world: int = 1, capacity: int = 16, threshold: int = 2):
        self.L = _setup()
        self.h = self.L.orinfer_greg_create(world, capacity, threshold)
        if not self.h:
            raise ValueError("world in 1..64, capacity and threshold at least 1")
        self.world = world

    def close(self) -> None:
        if self.h:
            self.L.orinfer_greg_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:                               # noqa: BLE001 - interpreter shutdown
            pass

    def _check(self, code: int) -> int:
        if code < 0:
            rank = c_int(-1)
            self.L.orinfer_greg_status(self.h, ctypes.byref(rank))
            raise GraphRegistryError(code, rank.value)
        return code

    def probe(self, key: int, rank: int = 0) -> bool:
        return bool(self._check(self.L.orinfer_greg_probe(self.h, rank, key)))

    def decide(self, key: int, all_hit: bool, rank: int = 0) -> Tuple[int, int, int, int]:
        """(decision, graph handle or -1, handle to release or -1, epoch for ``commit``)."""
        g, rel, ep = c_longlong(-1), c_longlong(-1), c_int(0)
        d = self._check(self.L.orinfer_greg_decide(self.h, rank, key, int(all_hit), ctypes.byref(g),
                                                   ctypes.byref(rel), ctypes.byref(ep)))
        return d, g.value, rel.value, ep.value

    def follow(self, key: int, decision: int, rank: int = 0) -> Tuple[int, int, int, int, bool]:
        """Applies the leader's decision; (decision carried out, graph, release, epoch,
        missed)."""
        g, rel, ep, miss = c_longlong(-1), c_longlong(-1), c_int(0), c_int(0)
        d = self._check(self.L.orinfer_greg_follow(self.h, rank, key, decision, ctypes.byref(g),
                                                   ctypes.byref(rel), ctypes.byref(ep),
                                                   ctypes.byref(miss)))
        return d, g.value, rel.value, ep.value, bool(miss.value)

    def commit(self, key: int, graph: int, epoch: int, rank: int = 0) -> bool:
        """False when the capture went stale (a recapture was forced meanwhile)."""
        code = self.L.orinfer_greg_commit(self.h, rank, key, graph, epoch)
        if code == E_STALE:
            return False
        self._check(code)
        return True

    def evict(self, key: int, rank: int = 0) -> int:
        return int(self.L.orinfer_greg_evict(self.h, rank, key))

    def clear(self, rank: int = 0) -> list:
        buf = (c_longlong * 4096)()
        n = self._check(self.L.orinfer_greg_clear(self.h, rank, buf, 4096))
        return [buf[i] for i in range(n)]

    def vote(self, key: int, hit: bool, rank: int, timeout_ms: int = 30000) -> bool:
        """Ranks that share this registry (threads of one process): blocks until all have
        voted on ``key``; True when every rank hit."""
        return bool(self._check(self.L.orinfer_greg_vote(self.h, rank, key, int(hit), timeout_ms)))

    def fail(self, rank: int, code: int = E_STICKY) -> None:
        self.L.orinfer_greg_fail(self.h, rank, code)

    def status(self) -> int:
        return int(self.L.orinfer_greg_status(self.h, None))

    def stats(self) -> Dict[str, int]:
        out = (c_longlong * 6)()
        self.L.orinfer_greg_stats(self.h, out)
        names = ("hits", "captures", "recaptures", "evictions", "entries", "graphs")
        return dict(zip(names, (int(v) for v in out)))


class GraphPool:
    """One rank's pool: the registry's decisions plus the objects behind its handles."""

    def __init__(self, capacity: int = 16, threshold: int = 2):
        self.registry = GraphRegistry(1, capacity, threshold)
        self.objects: Dict[int, Any] = {}
        self._next = 0

    def _release(self, handle: int) -> None:
        if handle >= 0:
            self.objects.pop(handle, None)

    def plan(self, geometry: Hashable) -> Tuple[int, int, Optional[Any], int]:
        """Leading (or only) rank: (decision, key, held object when REPLAY, epoch)."""
        key = key_of(geometry)
        d, g, rel, ep = self.registry.decide(key, self.registry.probe(key))
        self._release(rel)
        return d, key, self.objects.get(g) if d == REPLAY else None, ep

    def follow(self, geometry: Hashable, decision: int) -> Tuple[int, int, Optional[Any], int, bool]:
        key = key_of(geometry)
        d, g, rel, ep, missed = self.registry.follow(key, decision)
        self._release(rel)
        return d, key, self.objects.get(g) if d == REPLAY else None, ep, missed

    def commit(self, key: int, epoch: int, obj: Any) -> bool:
        handle, self._next = self._next, self._next + 1
        if not self.registry.commit(key, handle, epoch):
            return False
        self.objects[handle] = obj
        return True

    def evict(self, key: int) -> None:
        self._release(self.registry.evict(key))

    def clear(self) -> None:
        for handle in self.registry.clear():
            self._release(handle)
        self.objects.clear()

    def __len__(self) -> int:
        return len(self.objects)
