"""Activation-weighted precision screening of one linear layer (CPU, model-independent).

Whether a projection tolerates 4-bit or 8-bit integers is a property of ``X @ dW`` on real
activations ``X``, not of ``dW`` alone: correlated input channels can amplify or cancel the
weight error.  These helpers score candidate precisions on recorded activations:

* ``quantize_rows``: symmetric per-row integers with an optional clipping factor;
* ``screen_linear``: picks the clipping factor on training activations, reports the
  normalised output error on disjoint held-out activations, with the activation-only and
  weight-only parts shown beside the joint error so that neither can hide the other;
* ``fit_output_scales``: bounded, shrunk weighted least squares for the output scales of
  fixed integer codes;
* ``refine_integer_codes``: greedy coordinate descent over signed 4-bit codes, one legal
  +-1 step per output row and pass, driven by the sample covariance of the activations.

Role of python/orinfer_build/quantization/activation.py:10-145.
"""

from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np


def _matrix(v) -> np.ndarray:
    m = np.asarray(v, dtype=np.float32)
    if m.ndim != 2 or min(m.shape) == 0 or not np.isfinite(m).all():
        raise ValueError("expected a non-empty finite matrix")
    return m


def relative_mse(candidate, reference) -> float:
    c, r = _matrix(candidate), _matrix(reference)
    if c.shape != r.shape:
        raise ValueError("output shapes differ")
    num = np.square(c - r, dtype=np.float64).sum()
    return float(num / max(np.square(r, dtype=np.float64).sum(), 1e-30))


def quantize_rows(values, bits: int = 8, clip: float = 1.0) -> np.ndarray:
    """Fake-quantised copy: symmetric integers per row, scale = clip * max|row| / (2^(b-1)-1)."""
    v = _matrix(values)
    if bits not in (4, 8) or not 0 < clip <= 1:
        raise ValueError("bits is 4 or 8 and clip within (0, 1]")
    top = (1 << (bits - 1)) - 1
    scale = np.maximum(np.abs(v).max(1, keepdims=True) * clip / top, 1e-30)
    return np.clip(np.rint(v / scale), -top - 1, top) * scale


def statistics(activation) -> Dict[str, float]:
    a = _matrix(activation)
    energy = np.square(a, dtype=np.float64).sum(0)
    return {"rows": int(a.shape[0]), "channels": int(a.shape[1]),
            "mean_square": float(energy.sum() / a.size), "max_abs": float(np.abs(a).max()),
            "max_channel_energy_fraction": float(energy.max() / max(energy.sum(), 1e-30))}


def screen_linear(weight, train, holdout, *, bits: int, quantize_activation: bool = False,
                  clips: Sequence[float] = (0.8, 0.9, 0.95, 1.0)) -> Dict[str, object]:
    w, xt, xh = _matrix(weight), _matrix(train), _matrix(holdout)
    if xt.shape[1] != w.shape[1] or xh.shape[1] != w.shape[1] or not clips:
        raise ValueError("activation widths must equal the weight's input width")
    at = quantize_rows(xt) if quantize_activation else xt
    ah = quantize_rows(xh) if quantize_activation else xh
    want = xt @ w.T
    loss, clip = min((relative_mse(at @ quantize_rows(w, bits, c).T, want), c) for c in clips)
    wq = quantize_rows(w, bits, clip)
    want = xh @ w.T
    return {"bits": bits, "activation_bits": 8 if quantize_activation else None, "clip": clip,
            "train_nmse": loss, "holdout_nmse": relative_mse(ah @ wq.T, want),
            "activation_only_nmse": relative_mse(ah @ w.T, want),
            "weight_only_nmse": relative_mse(xh @ wq.T, want)}


def fit_output_scales(products, reference, scales, weights: Optional[np.ndarray] = None, *,
                      shrink: float = 0.5, limit: float = 0.05) -> np.ndarray:
    """New output scales for fixed integer codes: per output column the weighted least-squares
    factor between ``products`` (activations times integer codes) and ``reference``, kept
    within ``limit`` of the old scale and moved only ``shrink`` of the way."""
    p, r = _matrix(products), _matrix(reference)
    s = np.asarray(scales, dtype=np.float32)
    if p.shape != r.shape or s.shape != (p.shape[1],):
        raise ValueError("products, reference and scales do not match")
    if not np.isfinite(s).all() or (s <= 0).any():
        raise ValueError("scales must be positive and finite")
    if not 0 <= shrink <= 1 or not 0 <= limit < 1:
        raise ValueError("shrink within [0, 1], limit within [0, 1)")
    wt = np.ones_like(p) if weights is None else np.asarray(weights, dtype=np.float32)
    if wt.shape != p.shape or not np.isfinite(wt).all() or (wt < 0).any():
        raise ValueError("weights must be finite, non-negative and shaped like the products")
    den = np.sum(wt * p * p, axis=0, dtype=np.float64)
    num = np.sum(wt * p * r, axis=0, dtype=np.float64)
    fitted = np.divide(num, den, out=s.astype(np.float64), where=den > 1e-20)
    fitted = np.clip(fitted, s * (1 - limit), s * (1 + limit))
    return (s + shrink * (fitted - s)).astype(np.float32)


def refine_integer_codes(activation, reference, codes, scales, weights, *, steps: int = 4
                         ) -> np.ndarray:
    """Signed 4-bit codes [N, K] improved by greedy coordinate descent on the weighted output
    error ``sum w * (reference - (X @ codes^T) * scales)^2``: every pass moves, per output row,
    the one code whose +-1 step lowers the error most."""
    x, r, wt = _matrix(activation), _matrix(reference), _matrix(weights)
    q, s = np.asarray(codes), np.asarray(scales, dtype=np.float32)
    ok = (q.ndim == 2 and np.issubdtype(q.dtype, np.integer)
          and q.shape == (r.shape[1], x.shape[1]) and len(x) == len(r) and wt.shape == r.shape
          and s.shape == (len(q),) and q.min() >= -8 and q.max() <= 7 and (wt >= 0).all()
          and np.isfinite(s).all() and (s > 0).all() and 1 <= steps <= 16)
    if not ok:
        raise ValueError("need matched activations, non-negative importance and signed "
                         "4-bit codes")
    q = q.astype(np.int8, copy=True)
    resid = r - (x @ q.astype(np.float32).T) * s
    curv = np.square(s[:, None]) * (wt.T @ np.square(x))          # second-order term of a step
    rows = np.arange(len(q))
    for _ in range(steps):
        grad = (wt * resid).T @ x
        up = np.where(q < 7, curv - 2 * s[:, None] * grad, np.inf)
        down = np.where(q > -8, curv + 2 * s[:, None] * grad, np.inf)
        gain = np.minimum(up, down)
        col = gain.argmin(1)
        act = rows[gain[rows, col] < 0]
        if len(act) == 0:
            break
        col = col[act]
        step = np.where(up[act, col] < down[act, col], 1, -1).astype(np.int8)
        q[act, col] += step
        resid[:, act] -= x[:, col] * (step * s[act])
    return q
