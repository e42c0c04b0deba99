"""Block LDL rounding with error feedback (BlockLDLQ) for the lattice codec.

Plain nearest rounding minimises ``|W - Q|^2``; what matters for a layer's output is the
proxy loss ``tr((W - Q) H (W - Q)^T)`` with ``H = E[x x^T]`` the covariance of the layer's
(rotated) inputs.  Factor ``H = L D L^T`` with ``L`` unit *block* lower triangular (block =
the codec's 8-wide vector).  Rounding the column blocks from last to first, each block's
target is the weight plus the already committed error of the later blocks fed back through
``L``; the proxy loss then telescopes into ``sum_b |e_b D_b^{1/2}|^2`` of the per-block
rounding errors (QuIP#, arXiv 2402.04396).

``factor`` / ``round_blocks`` are the mathematical core and carry no codec; ``fit_q4_ldlq``
and ``fit_q2_ldlq`` pair them with the E8P codes of this package at a fixed per-row scale.
Role of python/orinfer_build/quantization/block_ldlq.py:13-59.
"""

from __future__ import annotations

from typing import Callable, Tuple

import numpy as np

from . import e8p

VEC = 8


def factor(covariance, *, block: int = VEC, damping: float = 0.01
           ) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Returns ``(H', L, D)``: the normalised, damped covariance, the unit block-lower factor
    and the diagonal blocks, with ``H' = L blockdiag(D) L^T``.

    ``H' = H / mean(diag H) + damping * I`` keeps the factorisation well conditioned for
    covariances estimated from few tokens."""
    h = np.asarray(covariance, dtype=np.float64)
    if h.ndim != 2 or h.shape[0] != h.shape[1] or h.shape[0] == 0 or not np.isfinite(h).all():
        raise ValueError("the covariance must be a finite square matrix")
    k = h.shape[0]
    if not isinstance(block, int) or block <= 0 or k % block:
        raise ValueError("the block size must divide the dimension")
    if not np.isfinite(damping) or damping <= 0:
        raise ValueError("damping must be positive")
    if not np.allclose(h, h.T, rtol=1e-8, atol=1e-10):
        raise ValueError("the covariance must be symmetric")
    level = float(np.trace(h)) / k
    if level <= 0:
        raise ValueError("the covariance needs a positive mean diagonal")
    hn = (h + h.T) * (0.5 / level) + damping * np.eye(k)
    c = np.linalg.cholesky(hn)                       # hn = c c^T, c lower triangular
    nb = k // block
    lower = np.empty_like(c)
    diag = np.empty((nb, block, block))
    for b in range(nb):
        sl = slice(b * block, (b + 1) * block)
        cb = c[sl, sl]
        lower[:, sl] = c[:, sl] @ np.linalg.inv(cb)  # unit diagonal block, zeros above
        diag[b] = cb @ cb.T
    return hn, lower, diag


def round_blocks(weight, lower, quantizer: Callable[[np.ndarray], np.ndarray], *,
                 block: int = VEC) -> np.ndarray:
    """Sequential rounding, last block first.  ``quantizer`` maps an [N, block] target to
    its reconstruction; the return value is the reconstructed [N, K] matrix."""
    w = np.asarray(weight, dtype=np.float64)
    lo = np.asarray(lower, dtype=np.float64)
    if w.ndim != 2 or lo.shape != (w.shape[1], w.shape[1]):
        raise ValueError("weight and factor shapes differ")
    if not (np.isfinite(w).all() and np.isfinite(lo).all()):
        raise ValueError("weight and factor must be finite")
    k = w.shape[1]
    if not isinstance(block, int) or block <= 0 or k % block:
        raise ValueError("the block size must divide the weight dimension")
    q = np.zeros_like(w)
    for lo_col in range(k - block, -1, -block):
        hi_col = lo_col + block
        feedback = (w[:, hi_col:] - q[:, hi_col:]) @ lo[hi_col:, lo_col:hi_col]
        target = w[:, lo_col:hi_col] + feedback
        got = np.asarray(quantizer(target), dtype=np.float64)
        if got.shape != target.shape or not np.isfinite(got).all():
            raise ValueError("the quantizer must return a finite block of the same shape")
        q[:, lo_col:hi_col] = got
    return q


def proxy_loss(weight, recon, covariance) -> float:
    e = np.asarray(weight, np.float64) - np.asarray(recon, np.float64)
    return float(np.einsum("nk,kj,nj->", e, np.asarray(covariance, np.float64), e))


def _row_scales(w: np.ndarray, levels: float) -> np.ndarray:
    rms = np.sqrt(np.mean(w * w, axis=1))
    s = np.maximum(rms / levels, 2.0 ** -24).astype(np.float16)
    if not np.isfinite(s).all():
        raise ValueError("scale not representable in FP16")
    return s


def fit_q4_ldlq(weight, signs, covariance, *, damping: float = 0.01) -> e8p.Q4Weight:
    """Two-stage E8P codes chosen by block LDL rounding in the rotated basis.

    ``covariance`` is that of the *rotated* inputs ([K, K]).  The per-row scale is fixed
    beforehand (rms / 16, the centre of the nearest-rounding search), since the feedback
    targets depend on it."""
    a, b = e8p.Q4_COEFF
    w = e8p.hadamard_rotate(np.asarray(weight, np.float32), np.asarray(signs)).astype(np.float64)
    n, k = w.shape
    _, lower, _ = factor(covariance, damping=damping)
    scale = _row_scales(w, 4.0 * a)
    sf = scale.astype(np.float64)[:, None]
    packed = np.zeros((n, k // VEC), np.uint32)
    cursor = [k // VEC]

    def quantizer(target: np.ndarray) -> np.ndarray:
        t = (target / sf).astype(np.float32)
        c0 = e8p.encode_nearest(t / a)
        q0 = e8p.decode(c0).astype(np.float32)
        c1 = e8p.encode_nearest((t - a * q0) / b)
        q1 = e8p.decode(c1).astype(np.float32)
        cursor[0] -= 1
        packed[:, cursor[0]] = c0.astype(np.uint32) | (c1.astype(np.uint32) << 16)
        return (a * q0 + b * q1).astype(np.float64) * sf

    round_blocks(w, lower, quantizer)
    return e8p.Q4Weight(packed, scale, np.asarray(signs, np.int8).copy())


def fit_q2_ldlq(weight, signs, covariance, *, damping: float = 0.01) -> e8p.Q2Weight:
    """Single-stage E8P codes chosen by block LDL rounding (see ``fit_q4_ldlq``)."""
    w = e8p.hadamard_rotate(np.asarray(weight, np.float32), np.asarray(signs)).astype(np.float64)
    n, k = w.shape
    _, lower, _ = factor(covariance, damping=damping)
    scale = _row_scales(w, 4.0)
    sf = scale.astype(np.float64)[:, None]
    codes = np.zeros((n, k // VEC), np.uint16)
    cursor = [k // VEC]

    def quantizer(target: np.ndarray) -> np.ndarray:
        c = e8p.encode_nearest((target / sf).astype(np.float32))
        cursor[0] -= 1
        codes[:, cursor[0]] = c
        return e8p.decode(c).astype(np.float64) * sf

    round_blocks(w, lower, quantizer)
    return e8p.Q2Weight(codes, scale, np.asarray(signs, np.int8).copy())
