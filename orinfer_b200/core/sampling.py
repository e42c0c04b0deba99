"""Sampling options, the deterministic counter RNG and the host sampling law.

Thin ctypes layer over ``csrc/core/sampling_core.cpp``.  Streams: ordinary
decode draws use stream 0; speculative rounds use DRAFT / ACCEPT / CORRECTION
(crates/orinfer-engine/src/mtp.rs:24-39 of the reference).
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_double, c_float, c_int, c_int32, c_uint32, c_uint64
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from ._lib import CoreError, last_error, lib

EVALUATION_SEED = 20_261_002
DRAFT_STREAM = 0x4D545001
ACCEPT_STREAM = 0x4D545002
CORRECTION_STREAM = 0x4D545003


class _COptions(ctypes.Structure):
    _fields_ = [("temperature", c_double), ("top_p", c_double), ("top_k", c_int32),
                ("presence_penalty", c_double), ("frequency_penalty", c_double),
                ("repetition_penalty", c_double), ("seed", c_uint64), ("bias_count", c_int32),
                ("bias_ids", POINTER(c_uint32)), ("bias_values", POINTER(c_double)),
                ("top_logprobs", c_int32)]


@dataclass
class SamplingOptions:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: int = EVALUATION_SEED
    logit_bias: Dict[int, float] = field(default_factory=dict)
    top_logprobs: Optional[int] = None

    def _c(self):
        ids = np.array(sorted(self.logit_bias), dtype=np.uint32)
        vals = np.array([self.logit_bias[int(i)] for i in ids], dtype=np.float64)
        c = _COptions(self.temperature, self.top_p, self.top_k, self.presence_penalty,
                      self.frequency_penalty, self.repetition_penalty, self.seed & (2 ** 64 - 1),
                      len(ids), ids.ctypes.data_as(POINTER(c_uint32)),
                      vals.ctypes.data_as(POINTER(c_double)),
                      -1 if self.top_logprobs is None else self.top_logprobs)
        return c, (ids, vals)

    def validate(self) -> None:
        c, _keep = self._c()
        if lib().orinfer_sampling_validate(ctypes.byref(c)) != 0:
            raise CoreError(last_error())

    @property
    def is_greedy(self) -> bool:
        """Temperature 0 and nothing that rewrites the scores: the arg-max is the answer.
        (Same predicate as ``orinfer_sampling_is_greedy``; evaluated here because the engine
        asks it for every row of every step.)"""
        return (self.temperature == 0.0 and self.presence_penalty == 0.0
                and self.frequency_penalty == 0.0 and self.repetition_penalty == 1.0
                and not self.logit_bias)

    @property
    def device_topk(self) -> bool:
        """Servable by the device top-k sampler: no host state (penalties, bias, report)."""
        return (self.temperature >= 1e-5 and 1 <= self.top_k <= 64 and 0.0 < self.top_p <= 1.0
                and self.presence_penalty == 0.0 and self.frequency_penalty == 0.0
                and self.repetition_penalty == 1.0 and not self.logit_bias
                and self.top_logprobs is None)

    @property
    def device_categorical(self) -> bool:
        c, _keep = self._c()
        return bool(lib().orinfer_sampling_device_categorical(ctypes.byref(c)))


GREEDY = SamplingOptions(temperature=0.0)


def _setup():
    l = lib()
    l.orinfer_splitmix64.restype = c_uint64
    l.orinfer_splitmix64.argtypes = [c_uint64]
    l.orinfer_counter_uniform.restype = c_double
    l.orinfer_counter_uniform.argtypes = [c_uint64, c_uint64, c_uint64]
    l.orinfer_round_step.restype = c_uint64
    l.orinfer_round_step.argtypes = [c_uint64, c_uint64]
    return l


_L = None


def _l():
    global _L
    if _L is None:
        _L = _setup()
    return _L


def splitmix64(x: int) -> int:
    return int(_l().orinfer_splitmix64(x & (2 ** 64 - 1)))


def counter_uniform(seed: int, stream: int, step: int) -> float:
    return float(_l().orinfer_counter_uniform(seed & (2 ** 64 - 1), stream, step))


def categorical_key(seed: int, step: int) -> Tuple[int, int]:
    out = (c_uint32 * 2)()
    _l().orinfer_categorical_key(c_uint64(seed & (2 ** 64 - 1)), c_uint64(step), out)
    return int(out[0]), int(out[1])


def philox2x32_10(counter: Tuple[int, int], key: int) -> Tuple[int, int]:
    out = (c_uint32 * 2)()
    _l().orinfer_philox2x32_10(c_uint32(counter[0]), c_uint32(counter[1]), c_uint32(key), out)
    return int(out[0]), int(out[1])


def round_step(round_index: int, position: int) -> int:
    if round_index >= 2 ** 32 - 1 or position > 2 ** 32 - 1:
        raise CoreError("Speculative sampling counter overflow")
    return int(_l().orinfer_round_step(round_index, position))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


def _ptr(a: Optional[np.ndarray], typ):
    return None if a is None else a.ctypes.data_as(POINTER(typ))


def sample(logits, history: Sequence[int], options: SamplingOptions, uniform: float,
           mask: Optional[np.ndarray] = None) -> int:
    lg, hist = _f32(logits), _u32(history)
    m = None if mask is None else _u32(mask)
    c, _keep = options._c()
    tok = c_uint32()
    rc = _l().orinfer_sample(_ptr(lg, c_float), c_int(lg.shape[0]), _ptr(hist, c_uint32),
                             c_int(hist.shape[0]), ctypes.byref(c), _ptr(m, c_uint32),
                             c_double(uniform), ctypes.byref(tok))
    if rc != 0:
        raise CoreError(last_error())
    return int(tok.value)


def law(logits, history: Sequence[int], options: SamplingOptions,
        mask: Optional[np.ndarray] = None) -> List[Tuple[int, float]]:
    lg, hist = _f32(logits), _u32(history)
    m = None if mask is None else _u32(mask)
    c, _keep = options._c()
    ids = np.empty(lg.shape[0], np.uint32)
    probs = np.empty(lg.shape[0], np.float64)
    n = _l().orinfer_sampling_law(_ptr(lg, c_float), c_int(lg.shape[0]), _ptr(hist, c_uint32),
                                  c_int(hist.shape[0]), ctypes.byref(c), _ptr(m, c_uint32),
                                  _ptr(ids, c_uint32), _ptr(probs, c_double), c_int(lg.shape[0]))
    if n < 0:
        raise CoreError(last_error())
    return list(zip(ids[:n].tolist(), probs[:n].tolist()))


def logprobs(logits, history: Sequence[int], options: SamplingOptions, chosen: int,
             top_n: int = 0, mask: Optional[np.ndarray] = None):
    """(chosen logprob, [(id, logprob)] top-n): after penalties/bias/mask, before top-k/p."""
    lg, hist = _f32(logits), _u32(history)
    m = None if mask is None else _u32(mask)
    c, _keep = options._c()
    out = c_double()
    ids = np.empty(max(top_n, 1), np.uint32)
    lps = np.empty(max(top_n, 1), np.float64)
    n = _l().orinfer_logprobs(_ptr(lg, c_float), c_int(lg.shape[0]), _ptr(hist, c_uint32),
                              c_int(hist.shape[0]), ctypes.byref(c), _ptr(m, c_uint32),
                              c_uint32(chosen), c_int(top_n), ctypes.byref(out),
                              _ptr(ids, c_uint32), _ptr(lps, c_double))
    if n < 0:
        raise CoreError(last_error())
    return float(out.value), list(zip(ids[:n].tolist(), lps[:n].tolist()))


def greedy_commit(drafts: Sequence[int], target: Sequence[int]) -> List[int]:
    d, t = _u32(drafts), _u32(target)
    out = np.empty(len(t) + 1, np.uint32)
    n = _l().orinfer_greedy_commit(_ptr(d, c_uint32), c_int(len(d)), _ptr(t, c_uint32),
                                   c_int(len(t)), _ptr(out, c_uint32))
    if n < 0:
        raise CoreError(last_error())
    return out[:n].tolist()


def sampled_commit(drafts: Sequence[int], draft_probs: Optional[np.ndarray], target_logits,
                   history: Sequence[int], options: SamplingOptions, step: int) -> List[int]:
    """Exact rejection sampling of one verification round; ``draft_probs`` is None for a
    deterministic (point-mass) proposer, else float64 [n_drafts, vocab]."""
    d, hist = _u32(drafts), _u32(history)
    lg = _f32(target_logits)
    vocab = lg.shape[-1]
    q = None if draft_probs is None else np.ascontiguousarray(draft_probs, dtype=np.float64)
    c, _keep = options._c()
    out = np.empty(len(d) + 1, np.uint32)
    n = _l().orinfer_sampled_commit(_ptr(d, c_uint32), c_int(len(d)), _ptr(q, c_double),
                                    _ptr(lg, c_float), c_int(vocab), _ptr(hist, c_uint32),
                                    c_int(len(hist)), ctypes.byref(c), c_uint64(step),
                                    _ptr(out, c_uint32))
    if n < 0:
        raise CoreError(last_error())
    return out[:n].tolist()
