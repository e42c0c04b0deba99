"""Command plane between the leader rank (which owns every scheduling decision) and the
follower ranks of a tensor-parallel server, one process per GPU.

The leader *publishes* device commands (page-table rows, packets to run, graph replays,
sharded sampling) in order; followers execute them in the same order, so every rank issues
the same kernels and collectives.  Commands are not awaited one by one (the data plane's own
collectives keep the ranks in step); instead every follower acknowledges each command when
it has queued its work, and the leader treats an acknowledgement that is overdue by more
than the deadline, a closed connection, or a follower's own failure report as fatal.  The
first failure is sticky: every later call fails at once, and the engine above fails closed.

Messages travel over local sockets (``multiprocessing.connection``: length-prefixed pickles
with an HMAC handshake).  Role of the reference's rank team and its channel
(crates/orinfer-engine/src/models/deepseek_v41/team.rs:26-116,286-345,
team/channel.rs:12-33,68-169).
"""

from __future__ import annotations

import os
import time
from collections import deque
from multiprocessing.connection import Client, Connection, Listener
from typing import Any, Deque, List, Optional, Tuple


class RankFailure(RuntimeError):
    """Fatal (error-taxonomy kind ``Nccl``): a follower rank is lost, late or failed."""

    def __init__(self, rank: int, what: str):
        super().__init__(f"rank {rank}: {what}")
        self.rank, self.what = rank, what


class LeaderChannel:
    """Leader side: listens, admits ``world - 1`` followers, then publishes commands."""

    def __init__(self, world: int, address, authkey: bytes, *, deadline_s: float = 30.0,
                 accept_s: float = 600.0):
        self.world, self.deadline_s = world, deadline_s
        self.listener = Listener(address, authkey=authkey)
        self.address = self.listener.address
        self.accept_s = accept_s
        self.conns: List[Optional[Connection]] = [None] * world
        self.seq = 0
        # per follower: (sequence number, time sent) of commands not yet acknowledged
        self.pending: List[Deque[Tuple[int, float]]] = [deque() for _ in range(world)]
        self.failure: Optional[RankFailure] = None
        self.misses: List[int] = []          # graph geometries a follower could not replay

    def take_misses(self) -> List[int]:
        """Keys reported by followers since the last call (drains their connections first)."""
        if self.failure is None:
            for rank in range(1, self.world):
                if self.conns[rank] is not None:
                    self._drain(rank)
        out, self.misses = self.misses, []
        return out

    def accept_all(self) -> None:
        """Waits for every follower's hello (its rank); a missing one is a failure."""
        end = time.monotonic() + self.accept_s
        sock = self.listener._listener._socket            # noqa: SLF001 - accept with a timeout
        while any(c is None for c in self.conns[1:]):
            left = end - time.monotonic()
            if left <= 0:
                missing = [r for r in range(1, self.world) if self.conns[r] is None]
                self._fail(missing[0], "never joined")
            sock.settimeout(min(left, 1.0))
            try:
                conn = self.listener.accept()
            except (TimeoutError, OSError):
                continue
            if not conn.poll(10.0):
                conn.close()
                continue
            kind, rank = conn.recv()
            if kind != "hello" or not 1 <= rank < self.world or self.conns[rank] is not None:
                conn.close()
                continue
            self.conns[rank] = conn

    # ------------------------------------------------------------------ publishing
    def _fail(self, rank: int, what: str) -> None:
        if self.failure is None:
            self.failure = RankFailure(rank, what)
        raise self.failure

    def _drain(self, rank: int) -> None:
        conn = self.conns[rank]
        try:
            while conn.poll(0):
                kind, value = conn.recv()
                if kind == "ack":
                    q = self.pending[rank]
                    while q and q[0][0] <= value:
                        q.popleft()
                elif kind == "miss":
                    self.misses.append(int(value))
                elif kind == "fail":
                    self._fail(rank, f"reported {value}")
        except (EOFError, OSError):
            self._fail(rank, "connection lost")

    def check(self) -> None:
        """Raises the sticky failure, or a new one when an acknowledgement is overdue."""
        if self.failure is not None:
            raise self.failure
        now = time.monotonic()
        for rank in range(1, self.world):
            self._drain(rank)
            q = self.pending[rank]
            if q and now - q[0][1] > self.deadline_s:
                self._fail(rank, f"no acknowledgement of command {q[0][0]} within "
                                 f"{self.deadline_s:.1f} s")

    def publish(self, op: str, payload: Any = None) -> int:
        """Sends one command to every follower (in rank order) and returns its number."""
        self.check()
        self.seq += 1
        now = time.monotonic()
        for rank in range(1, self.world):
            try:
                self.conns[rank].send((self.seq, op, payload))
            except (OSError, ValueError):
                self._fail(rank, "connection lost")
            self.pending[rank].append((self.seq, now))
        return self.seq

    def sync(self, timeout_s: Optional[float] = None) -> None:
        """Waits until every follower has acknowledged everything published so far."""
        end = time.monotonic() + (self.deadline_s if timeout_s is None else timeout_s)
        while True:
            self.check()
            if not any(self.pending[r] for r in range(1, self.world)):
                return
            if time.monotonic() > end:
                rank = next(r for r in range(1, self.world) if self.pending[r])
                self._fail(rank, "did not catch up in time")
            time.sleep(0.001)

    def close(self) -> None:
        for conn in self.conns[1:]:
            if conn is not None:
                try:
                    conn.send((0, "close", None))
                except (OSError, ValueError):
                    pass
                conn.close()
        self.conns = [None] * self.world
        self.listener.close()


class FollowerChannel:
    def __init__(self, address, authkey: bytes, rank: int, *, connect_s: float = 120.0):
        end = time.monotonic() + connect_s
        last: Optional[Exception] = None
        self.conn: Optional[Connection] = None
        while time.monotonic() < end:
            try:
                self.conn = Client(address, authkey=authkey)
                break
            except (ConnectionRefusedError, FileNotFoundError, OSError) as e:
                last = e
                time.sleep(0.05)
        if self.conn is None:
            raise RankFailure(rank, f"cannot reach the leader: {last}")
        self.rank = rank
        self.conn.send(("hello", rank))

    def recv(self, timeout_s: Optional[float] = None):
        """Next command ``(seq, op, payload)``; ``None`` when nothing arrived in time.  A
        closed connection reads as a ``close`` command: a follower never outlives its leader."""
        try:
            if timeout_s is not None and not self.conn.poll(timeout_s):
                return None
            return self.conn.recv()
        except (EOFError, OSError):
            return (0, "close", None)

    def ack(self, seq: int) -> None:
        try:
            self.conn.send(("ack", seq))
        except (OSError, ValueError):
            pass

    def miss(self, key: int) -> None:
        """A geometry this rank was asked to replay but holds no graph of (it ran directly)."""
        try:
            self.conn.send(("miss", int(key)))
        except (OSError, ValueError):
            pass

    def fail(self, what: str) -> None:
        try:
            self.conn.send(("fail", what))
        except (OSError, ValueError):
            pass

    def close(self) -> None:
        self.conn.close()


def new_address(tag: str = "") -> str:
    """A fresh Unix-socket path for one server instance."""
    import tempfile
    return os.path.join(tempfile.gettempdir(), f"orinfer-ranks-{os.getpid()}-{tag}.sock")
