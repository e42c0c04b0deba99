"""Lattice-coded embedding rows (per-layer-embedding tables and other lookup-only banks).

A row packet is an FP16 scale followed by little-endian U16 E8P codes, one code per eight
channels, in the *fully rotated* basis (``rotation.transform(mode="full")``, so the
160-channel per-layer-embedding width needs no padding).  Lookup decodes the packet and
applies the inverse rotation; model inputs are never rotated for it.

``encode`` is this package's own fitter (nearest codes at three start scales with a
least-squares refit); ``pack`` / ``decode`` and the bounded ``Decoder`` cache follow
python/orinfer_build/quantization/embedding_vq.py:17-95.
"""

from __future__ import annotations

from collections import OrderedDict

import numpy as np

from . import e8p
from .rotation import PALEY_ORDER, full_width_ok, paley20, transform, walsh


def pack(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    if codes.dtype != np.uint16 or codes.ndim != 2:
        raise ValueError("codes must be a U16 matrix")
    if scales.dtype != np.float16 or scales.shape != (len(codes),):
        raise ValueError("one FP16 scale per row")
    if not np.isfinite(scales).all() or (scales <= 0).any():
        raise ValueError("scales must be positive and finite")
    out = np.empty((len(codes), 2 + 2 * codes.shape[1]), np.uint8)
    out[:, :2] = scales.astype("<f2").view(np.uint8).reshape(-1, 2)
    out[:, 2:] = codes.astype("<u2").view(np.uint8).reshape(len(codes), -1)
    return out


def _split(packets: np.ndarray, k: int):
    if packets.dtype != np.uint8 or packets.ndim != 2 or packets.shape[1] != 2 + k // 4:
        raise ValueError("packet width does not match the channel count")
    scale = np.ascontiguousarray(packets[:, :2]).view("<f2").reshape(-1).astype(np.float32)
    if not np.isfinite(scale).all() or (scale <= 0).any():
        raise ValueError("invalid row scale")
    return scale, np.ascontiguousarray(packets[:, 2:]).view("<u2")


def decode(packets: np.ndarray, signs: np.ndarray, table: np.ndarray | None = None) -> np.ndarray:
    """uint8 [R, 2 + K/4] -> float32 [R, K] in the model's own basis."""
    scale, codes = _split(packets, len(signs))
    rot = e8p.decode(codes, table).reshape(len(packets), len(signs)).astype(np.float32)
    return transform(rot * scale[:, None], signs, mode="full", inverse=True)


def encode(rows, signs, refine: int = 2) -> np.ndarray:
    """float [R, K] -> packets; K = 20 * 2**p and K % 8 == 0."""
    x = np.asarray(rows, np.float32)
    s = np.asarray(signs)
    if x.ndim != 2 or x.shape[1] % 8 or not full_width_ok(x.shape[1]):
        raise ValueError("embedding width must be 20 * 2**p and a multiple of 8")
    rot = transform(x, s, mode="full")
    r, k = rot.shape
    codes = np.zeros((r, k // 8), np.uint16)
    scales = np.full(r, np.float16(2.0 ** -24))
    best = np.full(r, np.inf)
    base = np.sqrt(np.mean(rot * rot, axis=1)) / 4.0
    for mult in (0.85, 1.0, 1.15):
        sc = np.maximum(base * mult, 2.0 ** -24).astype(np.float16)
        for it in range(refine + 1):
            scf = sc.astype(np.float32)[:, None]
            c = e8p.encode_nearest((rot / scf).reshape(-1, 8)).reshape(r, k // 8)
            q = e8p.decode(c).reshape(r, k).astype(np.float32)
            if it < refine:
                sc = np.maximum((rot * q).sum(1) / np.maximum((q * q).sum(1), 1e-30),
                                2.0 ** -24).astype(np.float16)
        err = ((rot - q * sc.astype(np.float32)[:, None]) ** 2).sum(1)
        better = err < best
        best[better], codes[better], scales[better] = err[better], c[better], sc[better]
    return pack(codes, scales)


class Decoder:
    """Lookup decoder owned by one checkpoint reader: keeps one 65536-entry integer codebook
    (512 KiB) and at most 128 validated sign vectors.  Both are keyed by content, so a changed
    table or sign vector never reuses stale state."""

    MAX_SIGNS = 128

    def __init__(self):
        self._table_key = None
        self._book = None
        self._signs: "OrderedDict[tuple, None]" = OrderedDict()
        p = paley20() * np.float32(PALEY_ORDER ** -0.5)
        p.setflags(write=False)
        self._paley = p

    def decode(self, packets: np.ndarray, signs, table: np.ndarray | None = None) -> np.ndarray:
        s = np.asarray(signs)
        if s.ndim != 1 or not full_width_ok(len(s)):
            raise ValueError("invalid embedding transform dimension")
        key = (s.dtype.str, s.tobytes())
        if key not in self._signs:
            if not np.isin(s, (-1, 1)).all():
                raise ValueError("a rotation needs one +1/-1 sign per channel")
            if len(self._signs) == self.MAX_SIGNS:
                self._signs.popitem(last=False)
            self._signs[key] = None
        self._signs.move_to_end(key)
        tab = np.asarray(e8p.basis() if table is None else table)
        if tab.dtype != np.int8 or tab.shape != (256, 8):
            raise ValueError("invalid E8P table")
        tkey = tab.tobytes()
        if tkey != self._table_key:
            book = e8p.decode(np.arange(65536, dtype=np.uint32).astype(np.uint16), tab)
            book.setflags(write=False)
            self._book, self._table_key = book, tkey
        scale, codes = _split(packets, len(s))
        rot = self._book[codes].reshape(len(packets), len(s)).astype(np.float32) * scale[:, None]
        q = len(s) // PALEY_ORDER
        mixed = np.einsum("ji,...jc->...ic", self._paley, rot.reshape(len(packets), PALEY_ORDER, q))
        return walsh(mixed).reshape(rot.shape) * s.astype(np.float32)
