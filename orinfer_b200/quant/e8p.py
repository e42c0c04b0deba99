"""E8P lattice codec (CPU oracle, numpy).

A 16-bit code stores eight weights.  The high byte selects one of 256 basis
vectors of even integers; the low byte stores seven sign flips and, folded into
its parity, a +/-1 shift of the whole vector, so every decoded coordinate is an
odd integer in [-11, 11].  Two such codes (coarse in the low half of a U32,
residual in the high half) give the "Q4" format: ``w = s * (4*q0 + q1)`` with
one FP16 scale ``s`` per output row.  A single code per eight weights is "Q2".
Weights are quantised after a signed block-128 Hadamard rotation of the input
channels; the same rotation is applied to activations at run time.

The format matches the reference's checkpoints bit for bit
(python/orinfer_build/quantization/e8p.py:15-25 basis,
python/orinfer_build/quantization/vq.py:17,34-43 decode, :20-31 rotation,
python/orinfer_build/quantization/e8p_q4.py:32-70 Q4 container).
"""

from __future__ import annotations

import functools
from dataclasses import dataclass

import numpy as np

# Bit position inside the sign byte that carries the flip of coordinate i.
COORD_BIT = np.array([0, 4, 1, 5, 2, 6, 3, 7], dtype=np.uint16)
Q4_COEFF = (4, 1)
BLOCK = 128


@functools.lru_cache(maxsize=1)
def basis() -> np.ndarray:
    """The 256x8 INT8 basis: 227 inner-shell vectors plus 29 outer ones."""
    digits = np.stack(np.unravel_index(np.arange(3 ** 8), (3,) * 8), axis=1)
    cand = (4 * digits + 2).astype(np.int16)          # entries in {2, 6, 10}
    inner = cand[(cand.astype(np.int32) ** 2).sum(1) <= 160]
    # Outer shell: five coordinates raised to 6; 29 of the 56 choices, spread evenly.
    five_sets = []
    idx = list(range(5))
    while True:                                        # lexicographic 5-subsets of 0..7
        five_sets.append(tuple(idx))
        j = 4
        while j >= 0 and idx[j] == 3 + j:
            j -= 1
        if j < 0:
            break
        idx[j] += 1
        for t in range(j + 1, 5):
            idx[t] = idx[t - 1] + 1
    outer = np.full((29, 8), 2, np.int16)
    for i in range(29):
        outer[i, list(five_sets[i * len(five_sets) // 29])] = 6
    table = np.concatenate([inner, outer], axis=0)
    flip = (table.sum(1) // 4) % 2 == 1
    table[flip, 7] = -table[flip, 7]
    if table.shape != (256, 8):
        raise AssertionError("E8P basis must have 256 rows")
    out = table.astype(np.int8)
    out.setflags(write=False)
    return out


def decode(codes: np.ndarray, table: np.ndarray | None = None) -> np.ndarray:
    """U16 codes [...] -> INT8 coordinates [..., 8]."""
    table = basis() if table is None else table
    c = np.asarray(codes).astype(np.uint16)
    low = c & 0xFF
    par = np.zeros_like(low)
    for b in range(8):
        par ^= (low >> b) & 1
    flips = low ^ par                                  # bit 0 cleared of the parity
    neg = ((flips[..., None] >> COORD_BIT) & 1).astype(np.int16)
    shift = (1 - 2 * par.astype(np.int16))[..., None]
    vec = table[c >> 8].astype(np.int16)
    return (vec * (1 - 2 * neg) + shift).astype(np.int8)


def decode_q4(packed: np.ndarray) -> np.ndarray:
    """U32 [N, K/8] -> INT8 integer weights [N, K] (4*coarse + residual)."""
    p = np.asarray(packed).astype(np.uint32)
    q0 = decode((p & 0xFFFF).astype(np.uint16)).astype(np.int16)
    q1 = decode((p >> 16).astype(np.uint16)).astype(np.int16)
    q = Q4_COEFF[0] * q0 + Q4_COEFF[1] * q1
    return q.reshape(p.shape[0], -1).astype(np.int8)


def decode_q2(codes: np.ndarray) -> np.ndarray:
    """U16 [N, K/8] -> INT8 integer weights [N, K]."""
    c = np.asarray(codes)
    return decode(c).reshape(c.shape[0], -1)


def encode_nearest(x: np.ndarray, table: np.ndarray | None = None) -> np.ndarray:
    """Exhaustive nearest-codeword search; float [V, 8] -> U16 [V].

    For each parity shift p the target is moved by -(1-2p); within a basis row
    the best signs are the signs of the moved target, except that the number of
    flips is constrained: popcount parity of the stored byte must equal p, which
    may force one extra flip on the coordinate where it costs least.
    """
    table = basis() if table is None else table
    x = np.asarray(x, dtype=np.float32)
    if x.ndim != 2 or x.shape[1] != 8:
        raise ValueError("expected [vectors, 8]")
    v = x.shape[0]
    mag = np.abs(table.astype(np.float32))            # [256, 8]
    tneg = table < 0                                  # basis' own sign pattern
    best_code = np.zeros(v, np.uint16)
    best_dist = np.full(v, np.inf, np.float32)
    rows = np.arange(v)
    for p in (0, 1):
        t = x - np.float32(1 - 2 * p)
        want_neg = t < 0                              # desired sign of each output coord
        a = np.abs(t)
        # Output coord = table*(1-2*flip) + shift; sign of output (before shift)
        # is sign(table) xor flip  =>  flip = want_neg xor tneg.
        flip = want_neg[:, None, :] ^ tneg[None, :, :]          # [V,256,8]
        dist = ((a[:, None, :] - mag[None]) ** 2).sum(2)        # [V,256]
        # Stored byte is flips' bits with bit0 replaced by flips0 ^ p, which the
        # decoder undoes only if popcount(byte) % 2 == p, i.e. if the flip mask
        # itself has an even number of set bits.
        odd = (flip.sum(2) % 2) == 1
        # Fix an odd mask by toggling the cheapest coordinate: cost 4*a*mag.
        toggle_cost = 4.0 * a[:, None, :] * mag[None]
        cheapest = toggle_cost.argmin(2)
        dist = dist + np.where(odd, toggle_cost.min(2), 0.0)
        pick = dist.argmin(1)
        fl = flip[rows, pick].copy()
        need = odd[rows, pick]
        fl[rows[need], cheapest[rows, pick][need]] ^= True
        low = (fl.astype(np.uint16) << COORD_BIT[None, :]).sum(1).astype(np.uint16)
        low ^= np.uint16(p)
        code = (pick.astype(np.uint16) << 8) | low
        d = ((x - decode(code, table).astype(np.float32)) ** 2).sum(1)
        better = d < best_dist
        best_code = np.where(better, code, best_code)
        best_dist = np.where(better, d, best_dist)
    return best_code.astype(np.uint16)


def hadamard_rotate(x: np.ndarray, signs: np.ndarray) -> np.ndarray:
    """y = H_128 (x * signs) / sqrt(128), block-wise over the last axis."""
    x = np.asarray(x, dtype=np.float32)
    k = x.shape[-1]
    if k % BLOCK or signs.shape != (k,):
        raise ValueError("rotation needs K % 128 == 0 and one sign per channel")
    y = (x * signs.astype(np.float32)).reshape(*x.shape[:-1], k // BLOCK, BLOCK).copy()
    h = 1
    while h < BLOCK:
        y = y.reshape(*y.shape[:-1], BLOCK // (2 * h), 2, h)
        a = y[..., 0, :] + y[..., 1, :]
        b = y[..., 0, :] - y[..., 1, :]
        y = np.stack([a, b], axis=-2).reshape(*x.shape[:-1], k // BLOCK, BLOCK)
        h *= 2
    return (y * np.float32(BLOCK ** -0.5)).reshape(x.shape)


def inverse_rotate(y: np.ndarray, signs: np.ndarray) -> np.ndarray:
    """Inverse of :func:`hadamard_rotate` (H is symmetric and orthogonal)."""
    ones = np.ones_like(signs)
    return hadamard_rotate(y, ones) * signs.astype(np.float32)


def random_signs(k: int, seed: int = 0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return (1 - 2 * rng.integers(0, 2, size=k)).astype(np.int8)


@dataclass(frozen=True)
class Q4Weight:
    """Two-stage E8P weight of a linear layer [N, K]."""

    packed: np.ndarray      # U32 [N, K/8], low half coarse, high half residual
    scales: np.ndarray      # FP16 [N]
    signs: np.ndarray       # INT8 [K]

    @property
    def shape(self):
        return self.packed.shape[0], self.packed.shape[1] * 8

    def integers(self) -> np.ndarray:
        return decode_q4(self.packed)

    def dequantize_rotated(self) -> np.ndarray:
        """Weights in the rotated basis (what the GEMM multiplies)."""
        return self.integers().astype(np.float32) * self.scales.astype(np.float32)[:, None]

    def dequantize(self) -> np.ndarray:
        """Weights in the original basis."""
        return inverse_rotate(self.dequantize_rotated(), self.signs)

    def kmajor(self) -> np.ndarray:
        """Runtime layout U32 [K/128, N, 16] (storage.py:38-86 of the reference)."""
        n, k = self.shape
        return np.ascontiguousarray(self.packed.reshape(n, k // BLOCK, 16).transpose(1, 0, 2))


@dataclass(frozen=True)
class Q2Weight:
    codes: np.ndarray       # U16 [N, K/8]
    scales: np.ndarray      # FP16 [N]
    signs: np.ndarray       # INT8 [K]

    @property
    def shape(self):
        return self.codes.shape[0], self.codes.shape[1] * 8

    def integers(self) -> np.ndarray:
        return decode_q2(self.codes)

    def dequantize_rotated(self) -> np.ndarray:
        return self.integers().astype(np.float32) * self.scales.astype(np.float32)[:, None]

    def dequantize(self) -> np.ndarray:
        return inverse_rotate(self.dequantize_rotated(), self.signs)

    def kmajor(self) -> np.ndarray:
        n, k = self.shape
        return np.ascontiguousarray(self.codes.reshape(n, k // BLOCK, 16).transpose(1, 0, 2))


def _encode_rows(x: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    flat = x.reshape(-1, 8)
    codes = np.concatenate([encode_nearest(flat[i:i + 4096]) for i in range(0, len(flat), 4096)])
    q = decode(codes).reshape(x.shape).astype(np.float32)
    return codes.reshape(x.shape[0], -1), q


def _fp16_scale(v: float) -> np.float16:
    s = np.float16(max(v, 2.0 ** -24))
    if not np.isfinite(s):
        raise ValueError("scale not representable in FP16")
    return s


def fit_q4(weight: np.ndarray, signs: np.ndarray, refine: int = 2) -> Q4Weight:
    """Quantise [N, K] float weights to two-stage E8P with alternating refits.

    Per row: try three initial scales around rms/16, alternate (refit scale by
    least squares, re-encode coarse given residual, re-encode residual) and keep
    the lowest squared error (python/orinfer_build/quantization/e8p_q4.py:115-169).
    """
    a, b = Q4_COEFF
    w = hadamard_rotate(np.asarray(weight, np.float32), signs)
    n, k = w.shape
    packed = np.zeros((n, k // 8), np.uint32)
    scales = np.zeros(n, np.float16)
    for r in range(n):
        row = w[r:r + 1]
        base = float(np.sqrt(np.mean(row * row))) / (4 * a)
        best = np.inf
        for mult in (0.9, 1.0, 1.1):
            s = _fp16_scale(base * mult)
            c0, q0 = _encode_rows(row / (np.float32(s) * a))
            c1, q1 = _encode_rows((row / np.float32(s) - a * q0) / b)
            for _ in range(refine):
                q = a * q0 + b * q1
                s = _fp16_scale(float((row * q).sum()) / max(float((q * q).sum()), 1e-30))
                c0, q0 = _encode_rows((row / np.float32(s) - b * q1) / a)
                c1, q1 = _encode_rows((row / np.float32(s) - a * q0) / b)
            err = float(((row - np.float32(s) * (a * q0 + b * q1)) ** 2).sum())
            if err < best:
                best = err
                packed[r] = c0[0].astype(np.uint32) | (c1[0].astype(np.uint32) << 16)
                scales[r] = s
    return Q4Weight(packed, scales, signs.astype(np.int8).copy())


def fit_q2(weight: np.ndarray, signs: np.ndarray, refine: int = 2) -> Q2Weight:
    """Single-stage E8P (2 bits/weight), one FP16 scale per output row."""
    w = hadamard_rotate(np.asarray(weight, np.float32), signs)
    n, k = w.shape
    codes = np.zeros((n, k // 8), np.uint16)
    scales = np.zeros(n, np.float16)
    for r in range(n):
        row = w[r:r + 1]
        base = float(np.sqrt(np.mean(row * row))) / 4.0
        best = np.inf
        for mult in (0.85, 1.0, 1.15):
            s = _fp16_scale(base * mult)
            c, q = _encode_rows(row / np.float32(s))
            for _ in range(refine):
                s = _fp16_scale(float((row * q).sum()) / max(float((q * q).sum()), 1e-30))
                c, q = _encode_rows(row / np.float32(s))
            err = float(((row - np.float32(s) * q) ** 2).sum())
            if err < best:
                best, codes[r], scales[r] = err, c[0], s
    return Q2Weight(codes, scales, signs.astype(np.int8).copy())


# ---- W8 / A8 / INT8-KV reference math ---------------------------------------

def quantize_w8(weight: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Per-output-row symmetric INT8; returns (INT8 [N,K], FP16 scale [N])."""
    w = np.asarray(weight, np.float32)
    amax = np.abs(w).max(1)
    scale = np.where(amax > 0, np.maximum(amax / 127.0, 2.0 ** -24), 1.0).astype(np.float16)
    q = np.clip(np.rint(w / scale.astype(np.float32)[:, None]), -127, 127).astype(np.int8)
    return q, scale


def quantize_a8(x: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Per-token absmax INT8 after an FP16 boundary; FP16 scale, round-half-even
    (python/orinfer_build/quantization/reference_math.py:6-21)."""
    x = np.asarray(x).astype(np.float16).astype(np.float32)
    amax = np.abs(x).max(-1)
    scale = np.where(amax > 0, np.maximum(amax / 127.0, 2.0 ** -24), 1.0).astype(np.float16)
    q = np.clip(np.rint(x / scale.astype(np.float32)[..., None]), -127, 127).astype(np.int8)
    return q, scale


def quantize_kv(x: np.ndarray, group: int = 64) -> tuple[np.ndarray, np.ndarray]:
    """INT8 KV: per token, per head, per 64-channel group FP16 scale (min 2^-24)."""
    x = np.asarray(x).astype(np.float16).astype(np.float32)
    g = x.reshape(*x.shape[:-1], x.shape[-1] // group, group)
    scale = np.maximum(np.abs(g).max(-1) / 127.0, 2.0 ** -24).astype(np.float16)
    q = np.clip(np.rint(g / scale.astype(np.float32)[..., None]), -127, 127).astype(np.int8)
    return q.reshape(x.shape), scale
