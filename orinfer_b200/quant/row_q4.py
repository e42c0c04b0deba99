"""Scalar 4-bit weights with a fixed non-uniform level table ("row Q4").

Each weight is one nibble: bits 0..2 pick a magnitude from ``LEVELS`` (INT8 values, denser
near zero), bit 3 is the sign; two nibbles per byte, low nibble first.  One FP16 scale per
output row; the matrix lives in the block-128 rotated input basis like every other weight
format.  Because the levels are INT8 values, ``integers()`` is exactly what a W8A8 GEMM
consumes: the runtime expands such a matrix to INT8 once at load time
(``expand_to_w8``) and runs it through the W8 kernels, so the format costs 4 bits on disk
and in host memory.

Container and fitting rule follow python/orinfer_build/quantization/row_q4.py:16-111
(levels, nibble layout, three start scales times four Lloyd steps per 128-row group).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import numpy as np

from .e8p import hadamard_rotate

LEVELS = (3, 10, 19, 31, 46, 67, 93, 127)
START_SCALES = (0.9, 1.0, 1.15)
LLOYD_STEPS = 4


@dataclass(frozen=True)
class RowQ4Weight:
    packed: np.ndarray            # uint8 [N, K/2]
    scales: np.ndarray            # float16 [N]
    signs: np.ndarray             # int8 [K]

    def validate(self) -> Tuple[int, int]:
        if self.packed.dtype != np.uint8 or self.packed.ndim != 2:
            raise ValueError("row Q4 needs a two-dimensional byte matrix")
        n, k = self.packed.shape[0], 2 * self.packed.shape[1]
        if n <= 0 or k <= 0 or k % 128:
            raise ValueError("row Q4 needs a non-empty matrix with K % 128 == 0")
        if (self.scales.dtype != np.float16 or self.scales.shape != (n,)
                or not np.isfinite(self.scales).all() or (self.scales <= 0).any()):
            raise ValueError("row Q4 needs one positive finite FP16 scale per row")
        if (self.signs.dtype != np.int8 or self.signs.shape != (k,)
                or not np.isin(self.signs, (-1, 1)).all()):
            raise ValueError("row Q4 needs one rotation sign per input channel")
        return n, k

    def integers(self) -> np.ndarray:
        """INT8 [N, K] in the rotated basis."""
        self.validate()
        nib = np.stack((self.packed & 15, self.packed >> 4), axis=-1).reshape(
            self.packed.shape[0], -1)
        mag = np.asarray(LEVELS, np.int8)[nib & 7]
        return np.where(nib < 8, mag, -mag).astype(np.int8)

    def dequantize_rotated(self) -> np.ndarray:
        return self.integers().astype(np.float32) * self.scales.astype(np.float32)[:, None]

    @property
    def bits_per_weight(self) -> float:
        n, k = self.validate()
        # the 16 shared signed levels are counted once per matrix
        return 8.0 * (self.packed.nbytes + self.scales.nbytes + self.signs.nbytes + 16) / (n * k)


def fit(weight, signs) -> RowQ4Weight:
    w = np.asarray(weight, np.float32)
    s = np.asarray(signs)
    if w.ndim != 2 or min(w.shape) <= 0 or not np.isfinite(w).all():
        raise ValueError("row Q4 fitting needs a non-empty finite matrix")
    if s.dtype != np.int8:
        raise ValueError("rotation signs must be INT8")
    rot = hadamard_rotate(w, s)
    n, k = rot.shape
    levels = np.asarray(LEVELS, np.float32)
    edges = (levels[:-1] + levels[1:]) * 0.5
    packed = np.empty((n, k // 2), np.uint8)
    scales = np.empty(n, np.float16)
    for lo in range(0, n, 128):
        raw = rot[lo:lo + 128]
        mag = np.abs(raw)
        start = np.sqrt(np.mean(raw * raw, axis=1)) * np.float32(2.7 / 127)
        best = np.full(len(raw), np.inf, np.float32)
        nib = np.empty(raw.shape, np.uint8)
        chosen = np.empty(len(raw), np.float16)
        for mult in START_SCALES:
            sc = np.maximum(start * np.float32(mult), 2.0 ** -24)
            for _ in range(LLOYD_STEPS):
                idx = np.searchsorted(edges, mag / sc[:, None])
                dec = levels[idx]
                sc = np.maximum((mag * dec).sum(1) / np.maximum((dec * dec).sum(1), 1e-30),
                                2.0 ** -24)
            sc16 = sc.astype(np.float16)
            if not np.isfinite(sc16).all():
                raise ValueError("row scale not representable in FP16")
            scf = sc16.astype(np.float32)[:, None]
            idx = np.searchsorted(edges, mag / scf).astype(np.uint8)
            loss = ((mag - levels[idx] * scf) ** 2).sum(1)
            better = loss < best
            best[better] = loss[better]
            nib[better] = idx[better] | np.where(raw[better] < 0, 8, 0).astype(np.uint8)
            chosen[better] = sc16[better]
        packed[lo:lo + len(raw)] = nib[:, 0::2] | (nib[:, 1::2] << 4)
        scales[lo:lo + len(raw)] = chosen
    out = RowQ4Weight(packed, scales, s.copy())
    out.validate()
    return out


def expand_to_w8(q: RowQ4Weight) -> Tuple[np.ndarray, np.ndarray]:
    """(INT8 [N, K], FP16 scale [N]) for the W8A8 kernels; exact."""
    return q.integers(), q.scales.copy()
