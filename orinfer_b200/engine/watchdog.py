"""Step watchdog: a host thread that fails the service closed when one engine step (or the
model load) runs past its deadline.

Every command of the reference's rank team carries a deadline (30 s, 120 s or more for heavy
ones; crates/orinfer-engine/src/models/deepseek_v41/team/channel.rs:12-33) and the first
failure is sticky: later calls fail fast, ``/health`` turns 503 and the process leaves with a
non-zero code so a supervisor restarts it (server/continuous.rs:526-532,947-955).  Device-side
waits here are bounded and report through a status word; this watchdog covers what is left —
a host call that never returns (a collective whose peer is gone, a driver call that blocks).
It never touches the GPU: it only marks the lifecycle failed, answers the waiting clients and,
when asked to, ends the process with ``os._exit`` so no exit hook runs against a stuck driver.
"""

from __future__ import annotations

import threading
import time
from typing import Callable, Optional


class StepWatchdog:
    def __init__(self, on_timeout: Callable[[str, float], None], poll_s: float = 0.05):
        self.on_timeout = on_timeout
        self.poll_s = poll_s
        self._lock = threading.Lock()
        self._deadline: Optional[float] = None
        self._what = ""
        self._armed_at = 0.0
        self.tripped: Optional[str] = None          # sticky: the first overrun
        self.longest_s = 0.0
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="orinfer-watchdog", daemon=True)
        self._thread.start()

    def arm(self, what: str, deadline_s: float) -> None:
        if deadline_s <= 0:
            return
        with self._lock:
            self._what, self._armed_at = what, time.monotonic()
            self._deadline = self._armed_at + deadline_s

    def disarm(self) -> None:
        with self._lock:
            if self._deadline is not None:
                self.longest_s = max(self.longest_s, time.monotonic() - self._armed_at)
            self._deadline = None

    def guard(self, what: str, deadline_s: float):
        """``with watchdog.guard("step", 30): ...``"""
        dog = self

        class _Guard:
            def __enter__(self):
                dog.arm(what, deadline_s)

            def __exit__(self, *exc):
                dog.disarm()
                return False

        return _Guard()

    def _run(self) -> None:
        while not self._stop.wait(self.poll_s):
            with self._lock:
                late = self._deadline is not None and time.monotonic() > self._deadline
                what, waited = self._what, time.monotonic() - self._armed_at
                if late:
                    self._deadline = None
            if late and self.tripped is None:
                self.tripped = what
                self.on_timeout(what, waited)

    def close(self) -> None:
        self._stop.set()
        self._thread.join(timeout=2)
