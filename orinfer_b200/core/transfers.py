"""Python face of ``csrc/core/transfers.cpp``: the bounded staging ring and the input packer."""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_int, c_int64, c_uint8, c_uint64, c_void_p
from typing import List, Optional, Sequence, Tuple

import numpy as np

from ._lib import lib

_ready = False


def _l():
    global _ready
    L = lib()
    if not _ready:
        L.orinfer_ring_create.restype = c_void_p
        L.orinfer_ring_create.argtypes = [c_uint64, c_uint64]
        L.orinfer_ring_destroy.argtypes = [c_void_p]
        L.orinfer_ring_acquire.restype = c_int64
        L.orinfer_ring_acquire.argtypes = [c_void_p, c_uint64, POINTER(c_uint64)]
        L.orinfer_ring_retire_through.argtypes = [c_void_p, c_uint64]
        L.orinfer_ring_stats.argtypes = [c_void_p, POINTER(c_uint64)]
        L.orinfer_pack_inputs.argtypes = [POINTER(c_uint8), c_uint64, POINTER(c_uint64),
                                          POINTER(c_uint64), POINTER(c_void_p), c_int, c_uint64,
                                          POINTER(c_uint64), POINTER(c_uint64), c_int]
        _ready = True
    return L


class StagingRing:
    """Bookkeeping of a pinned staging buffer of ``capacity`` bytes used in submission order.
    ``acquire`` returns (ticket, offset), or None when the caller has to wait for the stream and
    ``retire_through`` some tickets; a request larger than the ring raises."""

    def __init__(self, capacity: int, alignment: int = 256):
        self._h = _l().orinfer_ring_create(capacity, alignment)
        if not self._h:
            raise ValueError("ring capacity must be a positive multiple of a power-of-two alignment")

    def __del__(self):
        if getattr(self, "_h", None):
            _l().orinfer_ring_destroy(self._h)
            self._h = None

    def acquire(self, nbytes: int) -> Optional[Tuple[int, int]]:
        off = c_uint64()
        t = _l().orinfer_ring_acquire(self._h, nbytes, ctypes.byref(off))
        if t < 0:
            raise ValueError(f"an upload of {nbytes} bytes can never fit the staging ring")
        return (int(t), int(off.value)) if t else None

    def retire_through(self, ticket: int) -> int:
        n = _l().orinfer_ring_retire_through(self._h, ticket)
        if n < 0:
            raise ValueError("ticket was never issued")
        return n

    def stats(self) -> dict:
        v = (c_uint64 * 5)()
        _l().orinfer_ring_stats(self._h, v)
        return dict(zip(("capacity", "used", "live", "peak", "refused"), map(int, v)))


def pack_inputs(stage: np.ndarray, writes: Sequence[Tuple[int, np.ndarray]], merge_gap: int = 0
                ) -> List[Tuple[int, int]]:
    """Apply ``writes`` = [(byte offset, array)] to the staging image ``stage`` (uint8, mirrors
    the device input block) in order and return the disjoint (offset, length) ranges to copy."""
    if stage.dtype != np.uint8 or not stage.flags["C_CONTIGUOUS"]:
        raise ValueError("the staging image must be a contiguous uint8 array")
    n = len(writes)
    arrays = [np.ascontiguousarray(a).view(np.uint8).reshape(-1) for _, a in writes]
    offs = np.asarray([o for o, _ in writes] or [0], dtype=np.uint64)
    lens = np.asarray([a.size for a in arrays] or [0], dtype=np.uint64)
    srcs = (c_void_p * max(n, 1))(*[a.ctypes.data for a in arrays])
    out_o = np.zeros(max(n, 1), dtype=np.uint64)
    out_l = np.zeros(max(n, 1), dtype=np.uint64)
    count = _l().orinfer_pack_inputs(
        stage.ctypes.data_as(POINTER(c_uint8)), stage.size, offs.ctypes.data_as(POINTER(c_uint64)),
        lens.ctypes.data_as(POINTER(c_uint64)), srcs, n, merge_gap,
        out_o.ctypes.data_as(POINTER(c_uint64)), out_l.ctypes.data_as(POINTER(c_uint64)),
        max(n, 1))
    if count < 0:
        raise ValueError("an input write falls outside its block")
    return [(int(out_o[i]), int(out_l[i])) for i in range(count)]
