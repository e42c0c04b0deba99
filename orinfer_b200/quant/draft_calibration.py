"""Offline calibration of a draft head's confidence into prefix-survival probabilities.

A speculative round proposes ``W`` draft tokens; the draft head reports a confidence (the
probability it gave its own choice) for each.  What the width controller needs is the
probability that the first ``j`` drafts are *all* accepted.  Raw confidences are
over- or under-confident in a position-dependent way, so each position gets a temperature on
the confidence's logit, and the survival of a prefix is the running product of the tempered
conditionals::

    p_j = sigmoid(logit(c_j) / T_j)          survival_j = p_1 * ... * p_j

Temperatures are fitted position by position on recorded rounds (confidences + number of
drafts accepted) by grid search on the Brier score of the *cumulative* survival: once a draft
is rejected the later labels are zero because the prefix died, not because each later token
would have been rejected on its own, so they must not be scored as independent conditionals.

Same model and fitting rule as python/orinfer_build/quantization/speculative.py:6-92; the
adaptive controller's priors (``csrc/core/mtp_core.cpp``) can be seeded from
``expected_committed``.
"""

from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np

EPS = 1e-7


def survival(confidence, temperatures) -> np.ndarray:
    """[rounds, W] confidences in [0, 1] and [W] positive temperatures -> [rounds, W]
    probability that drafts 1..j all survive verification."""
    c = np.asarray(confidence, dtype=np.float64)
    t = np.asarray(temperatures, dtype=np.float64)
    if c.ndim != 2 or t.shape != (c.shape[1],):
        raise ValueError("confidence is [rounds, width], temperatures [width]")
    if not np.isfinite(c).all() or ((c < 0) | (c > 1)).any():
        raise ValueError("confidences must be finite and within [0, 1]")
    if not np.isfinite(t).all() or (t <= 0).any():
        raise ValueError("temperatures must be finite and positive")
    v = np.clip(c, EPS, 1 - EPS)
    z = (np.log(v) - np.log1p(-v)) / t
    step = 1.0 / (1.0 + np.exp(np.clip(-z, -80.0, 80.0)))
    return np.cumprod(step, axis=1)


def labels(accepted, width: int) -> np.ndarray:
    """[rounds] accepted counts -> bool [rounds, width]: did draft j survive."""
    a = np.asarray(accepted)
    if a.ndim != 1 or not np.issubdtype(a.dtype, np.integer) or ((a < 0) | (a > width)).any():
        raise ValueError("accepted counts must be integers within 0..width")
    return a[:, None] > np.arange(width)[None, :]


def fit(confidence, accepted, grid: Optional[Sequence[float]] = None) -> np.ndarray:
    """Per-position temperatures, fitted left to right (position j's survival depends on the
    temperatures before it).  Ties go to the temperature nearest 1."""
    c = np.asarray(confidence, dtype=np.float64)
    if c.ndim != 2 or c.shape[0] == 0 or c.shape[1] == 0:
        raise ValueError("calibration needs at least one round of at least one draft")
    y = labels(accepted, c.shape[1])
    if len(y) != len(c):
        raise ValueError("confidence rows and accepted counts differ in number")
    g = np.geomspace(0.25, 8.0, 65) if grid is None else np.asarray(grid, dtype=np.float64)
    g = np.unique(np.append(g, 1.0))
    temps = np.ones(c.shape[1])
    survival(c, temps)                                   # validates the inputs once
    for j in range(c.shape[1]):
        best_key, best_t = None, 1.0
        for cand in g:
            trial = temps.copy()
            trial[j] = cand
            s = survival(c, trial)[:, j]
            key = (float(np.mean((s - y[:, j]) ** 2)), abs(float(np.log(cand))))
            if best_key is None or key < best_key:
                best_key, best_t = key, float(cand)
        temps[j] = best_t
    return temps


def expected_committed(confidence, temperatures) -> float:
    """Mean tokens committed per round the calibration predicts (the verified token plus the
    surviving drafts)."""
    return float(1.0 + survival(confidence, temperatures).sum(1).mean())


def metrics(confidence, accepted, temperatures) -> Dict[str, object]:
    """Held-out quality of a calibration: cumulative Brier score, expected calibration error
    of every prefix length (10 equal-width bins), predicted against actual tokens per round."""
    s = survival(confidence, temperatures)
    y = labels(accepted, s.shape[1])
    if len(y) != len(s) or len(y) == 0:
        raise ValueError("evaluation needs matched, non-empty rounds")
    ece = []
    for j in range(s.shape[1]):
        bins = np.minimum((s[:, j] * 10).astype(int), 9)
        err = 0.0
        for b in range(10):
            rows = bins == b
            if rows.any():
                err += rows.mean() * abs(s[rows, j].mean() - y[rows, j].mean())
        ece.append(float(err))
    return {"windows": int(len(s)), "cumulative_brier": float(np.mean((s - y) ** 2)),
            "prefix_ece": ece, "predicted_committed_per_round": expected_committed(confidence,
                                                                                  temperatures),
            "actual_committed_per_round": float(1.0 + np.asarray(accepted).mean())}
