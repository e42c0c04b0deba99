"""Read-only machine telemetry for benchmark runs, and the GPU file lock that keeps two
measurements off one device.

``Sampler`` polls NVML on a thread (SM / memory clocks, power, temperature, utilisation, memory
in use, clock-event reasons) and summarises the samples taken while a measurement ran; a run
that saw a thermal or hardware slowdown, or clocks far below their maximum with no reason
given, is marked ``rejected`` so its number is taken again.  Nothing here sets a clock, a power
limit or any other device setting — the reference's samplers make the same promise
(tools/bench/sample_machine.py, check_gpu.py:1-6: "never touches clocks/power", measurements
under a non-blocking GPU file lock, python/orinfer_build/common/gpu.py).
"""

from __future__ import annotations

import fcntl
import os
import statistics
import threading
import time
from pathlib import Path
from typing import List, Optional

# NVML clock-event ("throttle") reason bits
REASONS = {
    0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap",
    0x8: "hw_slowdown", 0x10: "sync_boost", 0x20: "sw_thermal_slowdown",
    0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
}
REJECTING = {"hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
             "hw_power_brake_slowdown"}


def decode_reasons(mask: int) -> List[str]:
    return [name for bit, name in REASONS.items() if mask & bit]


class GpuBusy(RuntimeError):
    pass


class GpuLock:
    """Non-blocking advisory lock per device index: a second measurement on the same GPU fails
    at once instead of queueing behind (and disturbing) the first."""

    def __init__(self, index: int = 0, directory: Optional[str] = None):
        root = Path(directory or os.environ.get("ORINFER_LOCK_DIR") or "/tmp")
        self.path = root / f"orinfer-gpu-{index}.lock"
        self._fd: Optional[int] = None

    def acquire(self) -> "GpuLock":
        fd = os.open(self.path, os.O_CREAT | os.O_RDWR, 0o666)
        try:
            fcntl.flock(fd, fcntl.LOCK_EX | fcntl.LOCK_NB)
        except BlockingIOError:
            os.close(fd)
            raise GpuBusy(f"GPU lock {self.path} is held by another measurement") from None
        os.ftruncate(fd, 0)
        os.write(fd, f"{os.getpid()}\n".encode())
        self._fd = fd
        return self

    def release(self) -> None:
        if self._fd is not None:
            fcntl.flock(self._fd, fcntl.LOCK_UN)
            os.close(self._fd)
            self._fd = None

    __enter__ = acquire

    def __exit__(self, *exc):
        self.release()


class Sampler:
    """``with Sampler(index) as s: run(); report = s.summary()``.  ``nvml`` is the ``pynvml``
    module (or an object with the same read-only calls, which is how the CPU tests drive it)."""

    def __init__(self, index: int = 0, period_s: float = 0.2, nvml=None):
        if nvml is None:
            import pynvml as nvml
        self.nvml = nvml
        self.index, self.period_s = index, period_s
        self.samples: List[dict] = []
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.max_sm_mhz = 0

    def _read(self, handle) -> dict:
        n = self.nvml
        mem = n.nvmlDeviceGetMemoryInfo(handle)
        util = n.nvmlDeviceGetUtilizationRates(handle)
        return {"t": time.monotonic(),
                "sm_mhz": n.nvmlDeviceGetClockInfo(handle, n.NVML_CLOCK_SM),
                "mem_mhz": n.nvmlDeviceGetClockInfo(handle, n.NVML_CLOCK_MEM),
                "power_w": n.nvmlDeviceGetPowerUsage(handle) / 1000.0,
                "temperature_c": n.nvmlDeviceGetTemperature(handle, n.NVML_TEMPERATURE_GPU),
                "gpu_util": util.gpu, "memory_used_mib": mem.used >> 20,
                "reasons": decode_reasons(
                    n.nvmlDeviceGetCurrentClocksThrottleReasons(handle))}

    def _run(self) -> None:
        n = self.nvml
        n.nvmlInit()
        try:
            handle = n.nvmlDeviceGetHandleByIndex(self.index)
            self.max_sm_mhz = n.nvmlDeviceGetMaxClockInfo(handle, n.NVML_CLOCK_SM)
            while True:
                self.samples.append(self._read(handle))
                if self._stop.wait(self.period_s):
                    break
        finally:
            n.nvmlShutdown()

    def __enter__(self) -> "Sampler":
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=5)

    def summary(self, busy_util: int = 50) -> dict:
        """Statistics over the samples taken under load (utilisation >= ``busy_util``; all
        samples when none qualify)."""
        rows = [s for s in self.samples if s["gpu_util"] >= busy_util] or self.samples
        if not rows:
            return {"samples": 0, "rejected": False, "reasons": []}
        reasons = sorted({r for s in rows for r in s["reasons"]} - {"gpu_idle"})
        sm = statistics.median(s["sm_mhz"] for s in rows)
        stuck = self.max_sm_mhz > 0 and sm < 0.7 * self.max_sm_mhz and \
            not (set(reasons) - {"applications_clocks_setting"})
        bad = sorted(set(reasons) & REJECTING)
        return {"samples": len(rows), "sm_mhz": sm, "sm_max_mhz": self.max_sm_mhz,
                "mem_mhz": statistics.median(s["mem_mhz"] for s in rows),
                "power_w_mean": statistics.mean(s["power_w"] for s in rows),
                "power_w_max": max(s["power_w"] for s in rows),
                "temperature_c_max": max(s["temperature_c"] for s in rows),
                "memory_used_mib_max": max(s["memory_used_mib"] for s in rows),
                "reasons": reasons, "rejected": bool(bad) or stuck,
                "rejected_because": bad or (["clocks_below_max_without_reason"] if stuck else [])}
