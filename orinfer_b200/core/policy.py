"""ctypes face of the scheduler policy, adaptive MTP control and prompt lookup
(``csrc/core/sched_core.cpp``, ``csrc/core/mtp_core.cpp``)."""

from __future__ import annotations

import ctypes
import enum
from ctypes import POINTER, c_double, c_int, c_longlong, c_uint32, c_void_p
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np

from ._lib import lib


class ErrorKind(enum.IntEnum):
    """Error taxonomy (crates/orinfer-engine/src/error.rs:6-97; Nccl replaces Ascend)."""
    REQUEST = 0
    CAPACITY = 1
    OUT_OF_MEMORY = 2
    CUDA = 3
    NCCL = 4
    INVARIANT = 5

    @property
    def fatal(self) -> bool:
        return bool(lib().orinfer_error_is_fatal(int(self)))


class EngineError(RuntimeError):
    def __init__(self, kind: ErrorKind, message: str, code: int = 0):
        super().__init__(message)
        self.kind, self.code = kind, code

    @property
    def fatal(self) -> bool:
        return self.kind.fatal


class _Waiting(ctypes.Structure):
    _fields_ = [("age_s", c_double), ("remaining_s", c_double), ("restore_s", c_double),
                ("startup_s", c_double), ("remaining_tokens", c_longlong)]


@dataclass
class Waiting:
    age_s: float
    remaining_s: float
    restore_s: float = 0.0
    startup_s: float = 0.0
    remaining_tokens: int = 0


def _arr(reqs: Sequence[Waiting]):
    a = (_Waiting * len(reqs))()
    for i, r in enumerate(reqs):
        a[i] = _Waiting(r.age_s, r.remaining_s, r.restore_s, r.startup_s, r.remaining_tokens)
    return a


def _L():
    l = lib()
    if getattr(l, "_policy_ready", False):
        return l
    l.orinfer_prefill_window.restype = c_double
    l.orinfer_prefill_window.argtypes = [c_double] * 3
    l.orinfer_decode_quantum_s.restype = c_double
    l.orinfer_decode_quantum_s.argtypes = [c_double] * 3
    l.orinfer_joint_prefill_worthwhile.argtypes = [c_int, c_int, c_double, c_double]
    l.orinfer_admission_should_yield.argtypes = [c_int, c_int, c_double, c_int]
    l.orinfer_usable_host_bytes.restype = c_longlong
    l.orinfer_usable_host_bytes.argtypes = [c_longlong, c_longlong]
    l.orinfer_replenish.argtypes = [POINTER(c_double), c_int, c_double]
    for n in ("timing", "lengths", "acceptance", "lookup"):
        getattr(l, f"orinfer_{n}_create").restype = c_void_p
        getattr(l, f"orinfer_{n}_destroy").argtypes = [c_void_p]
    l.orinfer_timing_observe.argtypes = [c_void_p, c_double]
    l.orinfer_timing_mean.restype = c_double
    l.orinfer_timing_mean.argtypes = [c_void_p]
    l.orinfer_timing_upper.restype = c_double
    l.orinfer_timing_upper.argtypes = [c_void_p]
    l.orinfer_timing_samples.restype = c_longlong
    l.orinfer_timing_samples.argtypes = [c_void_p]
    l.orinfer_lengths_observe.argtypes = [c_void_p, c_longlong, c_longlong]
    l.orinfer_lengths_estimate.restype = c_double
    l.orinfer_lengths_estimate.argtypes = [c_void_p, c_longlong, c_longlong]
    l.orinfer_acceptance_observe.argtypes = [c_void_p, POINTER(c_int), POINTER(c_int), c_int]
    l.orinfer_acceptance_rate.restype = c_double
    l.orinfer_acceptance_rate.argtypes = [c_void_p, c_int, c_double]
    l.orinfer_acceptance_expected.restype = c_double
    l.orinfer_acceptance_expected.argtypes = [c_void_p, c_int]
    l.orinfer_mtp_allocate.argtypes = [POINTER(c_double), POINTER(c_int), c_int, c_int, c_double,
                                       POINTER(c_int)]
    l.orinfer_mtp_progress.restype = c_double
    l.orinfer_mtp_progress.argtypes = [POINTER(c_double), c_int, c_int, c_int]
    l.orinfer_lookup_propose.argtypes = [c_void_p, POINTER(c_uint32), c_int, c_int, c_int,
                                         POINTER(c_uint32)]
    l.orinfer_lookup_observe.argtypes = [c_void_p, c_int, c_int, c_int]
    l._policy_ready = True
    return l


def select_waiting(reqs: Sequence[Waiting]) -> Optional[int]:
    if not reqs:
        return None
    return int(_L().orinfer_select_waiting(_arr(reqs), len(reqs)))


def rank_throughput_waiting(reqs: Sequence[Waiting], expected: Sequence[float],
                            cohort_remaining: Optional[float]) -> List[int]:
    assert len(reqs) == len(expected)
    e = (c_double * len(reqs))(*expected)
    out = (c_int * len(reqs))()
    _L().orinfer_rank_throughput_waiting(_arr(reqs), e, len(reqs),
                                         int(cohort_remaining is not None),
                                         c_double(cohort_remaining or 0.0), out)
    return list(out)


def replenish(credits: List[float], quantum_s: float) -> List[float]:
    a = (c_double * len(credits))(*credits)
    _L().orinfer_replenish(a, len(credits), quantum_s)
    return list(a)


def prefill_window(slack_s, decode_s, ceiling_ms) -> float:
    return float(_L().orinfer_prefill_window(slack_s, decode_s, ceiling_ms))


def joint_prefill_worthwhile(loses_large_tile, measured, joint_s, native_s) -> bool:
    return bool(_L().orinfer_joint_prefill_worthwhile(int(loses_large_tile), int(measured),
                                                      joint_s, native_s))


def decode_quantum_s(prefill_s, prefill_budget_ms, tpot_ms) -> float:
    return float(_L().orinfer_decode_quantum_s(prefill_s, prefill_budget_ms, tpot_ms))


def admission_should_yield(has_decoders, admitted, elapsed_s, batchable_start) -> bool:
    return bool(_L().orinfer_admission_should_yield(int(has_decoders), admitted, elapsed_s,
                                                    int(batchable_start)))


def usable_host_bytes(meminfo_text: str) -> int:
    """MemAvailable minus one sixteenth of MemTotal, from /proc/meminfo text."""
    vals = {}
    for line in meminfo_text.splitlines():
        name, _, rest = line.partition(":")
        if name in ("MemTotal", "MemAvailable"):
            parts = rest.split()
            if len(parts) != 2 or parts[1] != "kB" or name in vals:
                raise ValueError("Invalid host memory budget")
            vals[name] = int(parts[0])
    if "MemTotal" not in vals or "MemAvailable" not in vals:
        raise ValueError("Missing MemTotal / MemAvailable")
    out = int(_L().orinfer_usable_host_bytes(vals["MemTotal"], vals["MemAvailable"]))
    if out < 0:
        raise ValueError("Invalid or missing MemAvailable")
    return out


class _Handle:
    _kind = ""

    def __init__(self):
        self._l = _L()
        self._h = c_void_p(getattr(self._l, f"orinfer_{self._kind}_create")())

    def __del__(self):
        if getattr(self, "_h", None):
            getattr(self._l, f"orinfer_{self._kind}_destroy")(self._h)
            self._h = None


class Timing(_Handle):
    """First-use observation primes a shape; later samples train its hot cost."""
    _kind = "timing"

    def observe(self, seconds: float) -> None:
        self._l.orinfer_timing_observe(self._h, seconds)

    @property
    def mean(self) -> float:
        return float(self._l.orinfer_timing_mean(self._h))

    @property
    def upper(self) -> float:
        return float(self._l.orinfer_timing_upper(self._h))

    @property
    def samples(self) -> int:
        return int(self._l.orinfer_timing_samples(self._h))


class OutputLengths(_Handle):
    _kind = "lengths"

    def observe(self, n_input: int, n_output: int) -> None:
        self._l.orinfer_lengths_observe(self._h, n_input, n_output)

    def estimate(self, n_input: int, limit: int) -> float:
        return float(self._l.orinfer_lengths_estimate(self._h, n_input, limit))


class Acceptance(_Handle):
    _kind = "acceptance"

    def observe(self, counts: Sequence[Tuple[int, int]]) -> None:
        p = (c_int * len(counts))(*[c[0] for c in counts])
        a = (c_int * len(counts))(*[c[1] for c in counts])
        self._l.orinfer_acceptance_observe(self._h, p, a, len(counts))

    def rate(self, position: int, prior: float = 0.7) -> float:
        return float(self._l.orinfer_acceptance_rate(self._h, position, prior))

    def expected(self, drafts: int) -> float:
        return float(self._l.orinfer_acceptance_expected(self._h, drafts))


class _Cand(ctypes.Structure):
    _fields_ = [("id", c_int), ("width", c_int), ("expected_tokens", c_double),
                ("maximum_tokens", c_double), ("remaining_tokens", c_longlong),
                ("mean_s", c_double), ("upper_s", c_double), ("transition_s", c_double),
                ("warm_ready", c_int), ("review_acceptance", c_int), ("samples", c_int),
                ("last", c_longlong)]


class _Sel(ctypes.Structure):
    _fields_ = [("normal_s", c_double), ("fixed_s", c_double), ("batch", c_int),
                ("slack_s", c_double), ("available_s", c_double), ("calibration_s", c_double),
                ("allow_exploration", c_int), ("calls", c_longlong), ("normal_last", c_longlong)]


@dataclass
class Candidate:
    id: int
    width: int
    expected_tokens: float
    maximum_tokens: float
    remaining_tokens: int
    mean_s: float
    upper_s: float
    transition_s: float = 0.0
    warm_ready: bool = True
    review_acceptance: bool = False
    samples: int = 0
    last: Optional[int] = None


def mtp_select(normal_s: float, batch: int, slack_s: float, candidates: Sequence[Candidate], *,
               fixed_s: float = 0.0, available_s: float = 0.0, calibration_s: float = 0.0,
               allow_exploration: bool = True, calls: int = 0,
               normal_last: Optional[int] = None):
    """-> (candidate id or None, exploring, calibrating)."""
    arr = (_Cand * max(len(candidates), 1))()
    for i, c in enumerate(candidates):
        arr[i] = _Cand(c.id, c.width, c.expected_tokens, c.maximum_tokens, c.remaining_tokens,
                       c.mean_s, c.upper_s, c.transition_s, int(c.warm_ready),
                       int(c.review_acceptance), c.samples, -1 if c.last is None else c.last)
    sel = _Sel(normal_s, fixed_s, batch, slack_s, available_s, calibration_s,
               int(allow_exploration), calls, -1 if normal_last is None else normal_last)
    flags = c_int()
    l = _L()
    l.orinfer_mtp_select.argtypes = [POINTER(_Sel), POINTER(_Cand), c_int, POINTER(c_int)]
    cid = l.orinfer_mtp_select(ctypes.byref(sel), arr, len(candidates), ctypes.byref(flags))
    return (None if cid < 0 else cid), bool(flags.value & 1), bool(flags.value & 2)


def mtp_allocate(rates: Sequence[float], caps: Sequence[int], budget: int,
                 floor: float = 0.0) -> List[int]:
    """Draft rows per request for one verification packet of ``budget`` draft rows: request r
    accepts each draft with probability ``rates[r]`` given the previous one, may take at most
    ``caps[r]``, and a row is placed only while its expected yield is at least ``floor``."""
    n = len(rates)
    if n != len(caps):
        raise ValueError("one cap per request")
    if n == 0:
        return []
    out = (c_int * n)()
    _L().orinfer_mtp_allocate((c_double * n)(*rates), (c_int * n)(*caps), n, int(budget),
                              float(floor), out)
    return list(out)


def mtp_progress(yields: Sequence[float], batch: int, latency: bool) -> float:
    a = (c_double * len(yields))(*yields)
    return float(_L().orinfer_mtp_progress(a, len(yields), batch, int(latency)))


class PromptLookup(_Handle):
    _kind = "lookup"

    def propose(self, history: Sequence[int], count: int, confident: bool = False) -> List[int]:
        h = np.ascontiguousarray(history, dtype=np.uint32)
        out = np.empty(max(count, 1), np.uint32)
        n = self._l.orinfer_lookup_propose(self._h, h.ctypes.data_as(POINTER(c_uint32)), len(h),
                                           count, int(confident),
                                           out.ctypes.data_as(POINTER(c_uint32)))
        return out[:n].tolist()

    def observe(self, accepted: int, proposed: int, progress: int) -> None:
        self._l.orinfer_lookup_observe(self._h, accepted, proposed, progress)


# ---------------------------------------------------------------- packet cost curves
class _Work(ctypes.Structure):
    _fields_ = [("tokens", ctypes.c_uint32), ("context", ctypes.c_uint32),
                ("decode_rows", ctypes.c_uint32), ("decode_context", ctypes.c_uint32),
                ("domain", ctypes.c_int)]


DIRECT, REPLAY, SHARED = 0, 1, 2


class CostCurves:
    """Bounded table of measured packet times (``csrc/core/cost_curves.cpp``): exact cell,
    then another path of the same shape, then interpolation over token counts, then the cold
    prior.  ``fit_tokens`` sizes a prefill chunk against a time budget."""

    def __init__(self, cold_tokens_per_s: float = 20000.0):
        L = _L()
        L.orinfer_costs_create.restype = ctypes.c_void_p
        L.orinfer_costs_create.argtypes = [ctypes.c_double]
        L.orinfer_costs_destroy.argtypes = [ctypes.c_void_p]
        L.orinfer_costs_cells.argtypes = [ctypes.c_void_p]
        L.orinfer_costs_observe.argtypes = [ctypes.c_void_p, ctypes.POINTER(_Work), ctypes.c_int,
                                            ctypes.c_double, ctypes.c_double]
        L.orinfer_costs_estimate.argtypes = [ctypes.c_void_p, ctypes.POINTER(_Work), ctypes.c_int,
                                             ctypes.POINTER(ctypes.c_double)]
        L.orinfer_costs_fit_tokens.argtypes = [ctypes.c_void_p, ctypes.POINTER(_Work),
                                               ctypes.c_int, ctypes.c_double, ctypes.c_int,
                                               ctypes.c_int]
        self._h = L.orinfer_costs_create(cold_tokens_per_s)
        if not self._h:
            raise ValueError("cold rate must be positive")

    def __del__(self):
        if getattr(self, "_h", None):
            _L().orinfer_costs_destroy(self._h)
            self._h = None

    @staticmethod
    def _w(tokens, context, decode_rows=0, decode_context=0, domain=0) -> _Work:
        return _Work(int(tokens), int(context), int(decode_rows), int(decode_context), int(domain))

    def observe(self, seconds: float, *, tokens: int, context: int, decode_rows: int = 0,
                decode_context: int = 0, domain: int = 0, path: int = DIRECT,
                setup_s: float = 0.0) -> None:
        w = self._w(tokens, context, decode_rows, decode_context, domain)
        _L().orinfer_costs_observe(self._h, ctypes.byref(w), path, seconds, setup_s)

    def estimate(self, *, tokens: int, context: int, decode_rows: int = 0,
                 decode_context: int = 0, domain: int = 0, path: int = -1):
        """-> (seconds, upper_s, samples, path)."""
        w = self._w(tokens, context, decode_rows, decode_context, domain)
        out = (ctypes.c_double * 4)()
        _L().orinfer_costs_estimate(self._h, ctypes.byref(w), path, out)
        return out[0], out[1], int(out[2]), int(out[3])

    def fit_tokens(self, budget_s: float, limit: int, quantum: int = 128, *, context: int,
                   decode_rows: int = 0, decode_context: int = 0, domain: int = 0,
                   path: int = -1) -> int:
        w = self._w(0, context, decode_rows, decode_context, domain)
        return _L().orinfer_costs_fit_tokens(self._h, ctypes.byref(w), path, budget_s, limit,
                                             quantum)

    @property
    def cells(self) -> int:
        return _L().orinfer_costs_cells(self._h)
