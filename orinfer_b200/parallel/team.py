"""Python face of the rank control plane (``csrc/dist/team.cpp``).

``Team`` runs one worker thread per rank; ``broadcast`` sends a command to every rank and
waits for every reply under a deadline.  The first error / timeout / lost rank is sticky
(``TeamFailure``), later broadcasts fail fast.  Two-phase helpers combine the per-rank replies
of a *plan* command before a *commit* command is sent, so ranks never take different
decisions.  ``FakeComm`` is an in-process sum all-reduce among the rank threads with host-side
failure injection; it stands in for NCCL in tests of the failure path (no GPU is ever faulted).

Contract: crates/orinfer-engine/src/models/deepseek_v41/team.rs:977-996,1404-1451 (two-phase
budget / save decisions), team/channel.rs:12-33,101-169 (deadlines, sticky failure),
backend/ascend/hccl/validation.rs:41-68 (preflight gate) of the reference.
"""

from __future__ import annotations

import ctypes
from ctypes import CFUNCTYPE, POINTER, c_int, c_longlong, c_void_p
from typing import Callable, List, Optional, Sequence

from ..core._lib import lib

TIMEOUT, RANK_ERROR, DISCONNECTED, STICKY = -1, -2, -3, -4
DROP_REPLY, DELAY_MS, ERROR_CODE, EXIT_THREAD = 1, 2, 3, 4
_NAMES = {TIMEOUT: "timeout", RANK_ERROR: "rank error", DISCONNECTED: "rank lost",
          STICKY: "team already failed"}

_HANDLER = CFUNCTYPE(c_longlong, c_void_p, c_int, c_int, POINTER(c_longlong), c_int,
                     POINTER(c_int))


class TeamFailure(RuntimeError):
    """Fatal: the team is retired (error taxonomy kind ``Nccl/Peer``)."""

    def __init__(self, result: int, rank: int, code: int):
        super().__init__(f"{_NAMES.get(result, result)} (rank {rank}, code {code})")
        self.result, self.rank, self.code = result, rank, code


def _setup():
    L = lib()
    L.orinfer_team_create.restype = c_void_p
    L.orinfer_team_create.argtypes = [c_int, _HANDLER, c_void_p, c_int, c_int]
    L.orinfer_team_broadcast.argtypes = [c_void_p, c_int, POINTER(c_longlong), c_int, c_int,
                                         POINTER(c_longlong)]
    L.orinfer_team_failure.argtypes = [c_void_p, POINTER(c_int), POINTER(c_int)]
    L.orinfer_team_inject.argtypes = [c_void_p, c_int, c_int, c_longlong, c_longlong]
    L.orinfer_team_destroy.argtypes = [c_void_p]
    L.orinfer_fakecomm_create.restype = c_void_p
    L.orinfer_fakecomm_create.argtypes = [c_int]
    L.orinfer_fakecomm_destroy.argtypes = [c_void_p]
    L.orinfer_fakecomm_fail_next.argtypes = [c_void_p, c_int, c_int]
    L.orinfer_fakecomm_calls.restype = c_longlong
    L.orinfer_fakecomm_calls.argtypes = [c_void_p]
    L.orinfer_fakecomm_all_reduce.argtypes = [c_void_p, c_int, POINTER(ctypes.c_double), c_int,
                                              c_int]
    return L


class Team:
    """``handler(rank, opcode, args) -> int`` runs on the rank's own thread; raising marks the
    rank failed (status 1)."""

    def __init__(self, ranks: int, handler: Callable[[int, int, List[int]], int], *,
                 fast_ms: int = 30_000, heavy_ms: int = 120_000):
        self._lib = _setup()
        self.ranks = ranks

        def trampoline(_user, rank, opcode, args, nargs, status):
            try:
                return int(handler(rank, opcode, [args[i] for i in range(nargs)]))
            except Exception:                                   # noqa: BLE001 - rank failure
                status[0] = 1
                return 0

        self._cb = _HANDLER(trampoline)                         # keep alive
        self._h = self._lib.orinfer_team_create(ranks, self._cb, None, fast_ms, heavy_ms)
        if not self._h:
            raise ValueError("invalid team size")

    def broadcast(self, opcode: int, args: Sequence[int] = (), heavy: bool = False) -> List[int]:
        arr = (c_longlong * max(len(args), 1))(*args)
        out = (c_longlong * self.ranks)()
        res = self._lib.orinfer_team_broadcast(self._h, opcode, arr, len(args), int(heavy), out)
        if res != 0:
            rank, code = self.failure() or (-1, 0)
            raise TeamFailure(res, rank, code)
        return list(out)

    def failure(self) -> Optional[tuple]:
        r, c = c_int(), c_int()
        if self._lib.orinfer_team_failure(self._h, ctypes.byref(r), ctypes.byref(c)):
            return r.value, c.value
        return None

    def inject(self, rank: int, kind: int, value: int = 0, at: int = 0) -> None:
        self._lib.orinfer_team_inject(self._h, rank, kind, value, at)

    # ---- two-phase decisions: plan on every rank, combine on the owner, then commit
    def budget(self, opcode: int, args: Sequence[int] = ()) -> int:
        """Every rank replies its free bytes; admission uses the minimum."""
        return min(self.broadcast(opcode, args))

    def agree(self, opcode: int, args: Sequence[int] = ()) -> int:
        """Every rank must reply the same key (e.g. a lineage hash); else the plan is void."""
        replies = self.broadcast(opcode, args)
        if len(set(replies)) != 1:
            raise ValueError(f"ranks disagree: {replies}")
        return replies[0]

    def save(self, plan_op: int, commit_op: int, rollback_op: int, args: Sequence[int] = ()) -> bool:
        """Plan -> all ranks must accept (non-zero) -> commit; any refusal rolls back all."""
        if all(self.broadcast(plan_op, args)):
            self.broadcast(commit_op, args)
            return True
        self.broadcast(rollback_op, args)
        return False

    def close(self) -> None:
        if self._h:
            self._lib.orinfer_team_destroy(self._h)
            self._h = None


class FakeComm:
    def __init__(self, ranks: int):
        self._lib = _setup()
        self.ranks = ranks
        self._h = self._lib.orinfer_fakecomm_create(ranks)

    def all_reduce(self, rank: int, values: List[float], timeout_ms: int = 1000) -> List[float]:
        buf = (ctypes.c_double * len(values))(*values)
        res = self._lib.orinfer_fakecomm_all_reduce(self._h, rank, buf, len(values), timeout_ms)
        if res != 0:
            raise RuntimeError(f"collective failed with code {res}")
        return list(buf)

    def fail_next(self, rank: int, code: int) -> None:
        self._lib.orinfer_fakecomm_fail_next(self._h, rank, code)

    @property
    def calls(self) -> int:
        return self._lib.orinfer_fakecomm_calls(self._h)

    def close(self) -> None:
        if self._h:
            self._lib.orinfer_fakecomm_destroy(self._h)
            self._h = None


def preflight(ready: Sequence[Callable[[], bool]], timeout_s: float = 30.0) -> bool:
    """No rank joins a communicator unless all ranks report ready within the window."""
    import concurrent.futures as cf
    with cf.ThreadPoolExecutor(max_workers=len(ready)) as pool:
        futs = [pool.submit(fn) for fn in ready]
        done, pending = cf.wait(futs, timeout=timeout_s)
        return not pending and all(f.exception() is None and f.result() for f in done)
