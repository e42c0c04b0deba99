"""Telemetry sampler against a fake NVML, and the GPU file lock."""
import time
from types import SimpleNamespace

import pytest

from orinfer_b200.bench.telemetry import GpuBusy, GpuLock, Sampler, decode_reasons


class FakeNvml:
    NVML_CLOCK_SM, NVML_CLOCK_MEM, NVML_TEMPERATURE_GPU = 1, 2, 0

    def __init__(self, sm=1900, reasons=0x4, util=99):
        self.sm, self.reasons, self.util = sm, reasons, util
        self.calls = []

    def __getattr__(self, name):                       # any call not listed below is a write
        raise AssertionError(f"unexpected NVML call {name}")

    def nvmlInit(self):
        self.calls.append("init")

    def nvmlShutdown(self):
        self.calls.append("shutdown")

    def nvmlDeviceGetHandleByIndex(self, i):
        return i

    def nvmlDeviceGetMaxClockInfo(self, h, kind):
        return 1965

    def nvmlDeviceGetClockInfo(self, h, kind):
        return self.sm if kind == self.NVML_CLOCK_SM else 3996

    def nvmlDeviceGetPowerUsage(self, h):
        return 950_000

    def nvmlDeviceGetTemperature(self, h, kind):
        return 61

    def nvmlDeviceGetMemoryInfo(self, h):
        return SimpleNamespace(used=40 << 30, total=180 << 30)

    def nvmlDeviceGetUtilizationRates(self, h):
        return SimpleNamespace(gpu=self.util, memory=50)

    def nvmlDeviceGetCurrentClocksThrottleReasons(self, h):
        return self.reasons


def run(fake):
    with Sampler(0, period_s=0.01, nvml=fake) as s:
        time.sleep(0.08)
    return s.summary()


def test_summary_keeps_power_cap_and_rejects_thermal_or_stuck_clocks():
    assert decode_reasons(0x4 | 0x40) == ["sw_power_cap", "hw_thermal_slowdown"]
    fake = FakeNvml()
    ok = run(fake)
    assert ok["samples"] >= 3 and ok["sm_mhz"] == 1900 and ok["sm_max_mhz"] == 1965
    assert ok["reasons"] == ["sw_power_cap"] and not ok["rejected"]
    assert ok["power_w_max"] == 950.0 and ok["memory_used_mib_max"] == 40 << 10
    assert fake.calls == ["init", "shutdown"]                       # and nothing that writes
    hot = run(FakeNvml(reasons=0x4 | 0x20))
    assert hot["rejected"] and hot["rejected_because"] == ["sw_thermal_slowdown"]
    stuck = run(FakeNvml(sm=900, reasons=0))
    assert stuck["rejected"] and stuck["rejected_because"] == ["clocks_below_max_without_reason"]
    capped = run(FakeNvml(sm=1200, reasons=0x4))                    # low, but a reason is given
    assert not capped["rejected"]
    idle = run(FakeNvml(util=0, reasons=0x1))
    assert idle["reasons"] == [] and idle["samples"] >= 3


def test_gpu_lock_is_exclusive_and_non_blocking(tmp_path):
    first = GpuLock(3, str(tmp_path)).acquire()
    t0 = time.monotonic()
    with pytest.raises(GpuBusy):
        GpuLock(3, str(tmp_path)).acquire()
    assert time.monotonic() - t0 < 0.5
    with GpuLock(4, str(tmp_path)):                                  # another device is free
        pass
    first.release()
    with GpuLock(3, str(tmp_path)) as again:
        assert again.path.read_text().strip().isdigit()
