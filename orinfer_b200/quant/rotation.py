"""Signed orthogonal input rotations used by the offline quantiser.

Two transforms share one interface (``transform(x, signs, mode=..., inverse=...)``):

``block128``
    the runtime's rotation: each 128-channel block is sign-flipped and multiplied by the
    order-128 Walsh-Hadamard matrix (``e8p.hadamard_rotate``).  It is its own inverse up to
    the signs.

``full``
    one rotation over the whole channel dimension ``K = 20 * 2**p`` (640, 1280, 2560, ...,
    and the 160-channel per-layer-embedding width): the Kronecker product of the order-20
    Paley Hadamard matrix and a power-of-two Walsh-Hadamard matrix, so such widths need no
    padding.  The order-20 factor is not symmetric, hence forward and inverse differ.

Role of python/orinfer_build/quantization/rotation.py:12-50 (Paley construction of the
order-20 factor, forward ``P (W (s * x))``, inverse ``s * W (P^T y)``).
"""

from __future__ import annotations

import numpy as np

from .e8p import hadamard_rotate, inverse_rotate

PALEY_ORDER = 20


def paley20() -> np.ndarray:
    """Order-20 Hadamard matrix by Paley's first construction over GF(19).

    With chi the quadratic character of GF(19) and Q[i, j] = chi(i - j), the matrix
    ``[[1, 1^T], [-1, Q + I]]`` has orthogonal rows because 19 = 3 (mod 4)."""
    p = PALEY_ORDER - 1
    squares = {(v * v) % p for v in range(1, p)}
    idx = np.arange(p)
    diff = (idx[:, None] - idx[None, :]) % p
    core = np.where(np.isin(diff, sorted(squares)) | (diff == 0), 1.0, -1.0)
    h = np.ones((PALEY_ORDER, PALEY_ORDER), np.float32)
    h[1:, 0] = -1.0
    h[1:, 1:] = core
    return h


def walsh(x: np.ndarray) -> np.ndarray:
    """Orthonormal Walsh-Hadamard transform over the last axis (a power of two)."""
    y = np.array(x, dtype=np.float32, copy=True)
    n = y.shape[-1]
    if n <= 0 or n & (n - 1):
        raise ValueError("Walsh transform needs a power-of-two length")
    lead = y.shape[:-1]
    h = 1
    while h < n:
        v = y.reshape(*lead, n // (2 * h), 2, h)
        y = np.stack([v[..., 0, :] + v[..., 1, :], v[..., 0, :] - v[..., 1, :]],
                     axis=-2).reshape(*lead, n)
        h *= 2
    return y * np.float32(n ** -0.5)


def _check_signs(x: np.ndarray, signs: np.ndarray) -> None:
    if x.ndim == 0 or signs.shape != (x.shape[-1],) or not np.isin(signs, (-1, 1)).all():
        raise ValueError("a rotation needs one +1/-1 sign per channel")


def full_width_ok(k: int) -> bool:
    q = k // PALEY_ORDER
    return k > 0 and k % PALEY_ORDER == 0 and q & (q - 1) == 0


def transform(x, signs, *, mode: str = "full", inverse: bool = False) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    s = np.asarray(signs)
    _check_signs(x, s)
    if mode == "block128":
        return inverse_rotate(x, s) if inverse else hadamard_rotate(x, s)
    if mode != "full" or not full_width_ok(x.shape[-1]):
        raise ValueError("the full rotation needs K = 20 * 2**p channels")
    q = x.shape[-1] // PALEY_ORDER
    p = paley20() * np.float32(PALEY_ORDER ** -0.5)
    sf = s.astype(np.float32)
    if inverse:
        mixed = np.einsum("ji,...jc->...ic", p, x.reshape(*x.shape[:-1], PALEY_ORDER, q))
        return walsh(mixed).reshape(x.shape) * sf
    spread = walsh((x * sf).reshape(*x.shape[:-1], PALEY_ORDER, q))
    return np.einsum("ij,...jc->...ic", p, spread).reshape(x.shape)


def matrix(signs, *, mode: str = "full") -> np.ndarray:
    """The rotation as a dense [K, K] matrix R with ``transform(x) = x @ R.T`` (tests, and
    rotating a covariance: ``H_rot = R H R^T``)."""
    k = len(signs)
    return transform(np.eye(k, dtype=np.float32), signs, mode=mode).T
