"""Gated-delta-rule linear attention in plain PyTorch: the oracle of the GDN kernels.

Per layer and request: a width-4 causal depthwise convolution over the q|k|v channels with a
three-row history, SiLU, per-head L2 normalisation of q and k; gates
``g = -exp(A_log) * softplus(a + dt_bias)`` and ``beta = sigmoid(b)``; the recurrence on an
FP32 state ``S[HV, DK, DV]``::

    S *= exp(g);  pred = S^T k;  delta = beta * (v - pred);  S += k (x) delta;  o = S^T (q / sqrt(DK))

and a gated per-head RMSNorm ``rmsnorm(o) * w * silu(z)`` (``sigmoid(z)`` for the Flash-Next
flavour).  Restates the reference's oracles
(python/orinfer_build/validation/cuda/gdn_reference.py:20-37,
python/orinfer_build/models/flash_next/reference/math.py:64-93) and kernel contracts
(kernels/cuda/operators/op08_gdn_conv_prep.py:23-278, op09_gdn_gates.py:26-76,
op17_gdn_gated_norm.py:15-71).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops_ref as R


def conv_silu_l2(x: torch.Tensor, history: torch.Tensor, weight: torch.Tensor, dk_total: int,
                 head_dim: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """x f16-valued [T, C] (q|k|v channels), history [3, C] (older rows first), weight [C, 4]
    (tap 3 multiplies the current row).  Returns (y [T, C] with q and k heads L2-normalised,
    new history)."""
    t = x.shape[0]
    full = torch.cat([history.float(), x.float()], dim=0)            # [T+3, C]
    w = weight.float()
    y = sum(full[j:j + t] * w[:, j][None, :] for j in range(4))
    y = R.f16(y * torch.sigmoid(y))
    qk = y[:, :2 * dk_total].reshape(t, -1, head_dim)
    qk = qk * torch.rsqrt((qk * qk).sum(-1, keepdim=True) + 1e-6)
    y = torch.cat([R.f16(qk).reshape(t, 2 * dk_total), y[:, 2 * dk_total:]], dim=1)
    return y, R.f16(full[-3:])


def gates(ab: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor):
    """ab fp32 [T, 2*HV] (a | b) -> (g [T, HV] natural-log decay <= 0, beta [T, HV])."""
    hv = a_log.shape[0]
    a, b = ab[:, :hv].float(), ab[:, hv:].float()
    g = -torch.exp(a_log.float())[None] * torch.nn.functional.softplus(a + dt_bias.float()[None])
    return g, torch.sigmoid(b)


def recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor,
               beta: torch.Tensor, state: torch.Tensor):
    """q, k [T, HK, D]; v [T, HV, D]; g, beta [T, HV]; state fp32 [HV, D, D] (dk, dv).
    Returns (o fp32 [T, HV, D], new state)."""
    t, hv, d = v.shape
    rep = hv // q.shape[1]
    qe = q.float().repeat_interleave(rep, 1) * (d ** -0.5)
    ke = k.float().repeat_interleave(rep, 1)
    s = state.float().clone()
    out = torch.empty(t, hv, d)
    for i in range(t):
        s = s * torch.exp(g[i])[:, None, None]
        pred = torch.einsum("hk,hkv->hv", ke[i], s)
        delta = beta[i][:, None] * (v[i].float() - pred)
        s = s + ke[i][:, :, None] * delta[:, None, :]
        out[i] = torch.einsum("hk,hkv->hv", qe[i], s)
    return out, s


def recurrence_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor,
                       beta: torch.Tensor, state: torch.Tensor, chunk: int = 16):
    """The same recurrence in chunkwise (WY) form: inside a chunk of ``C`` tokens everything
    is a small matrix product, so a kernel can put it on tensor cores (the reference's
    kernels/cuda/model/gdn_chunk.py:12,102 uses C = 16 with FP16 operands and an FP32 state).

    With ``G_i`` the running sum of ``g`` inside the chunk and ``S0`` the state before it::

        A[i, j] = beta_i * exp(G_i - G_j) * (k_i . k_j)          for j < i, else 0
        B[i]    = beta_i * (v_i - exp(G_i) * S0^T k_i)
        Delta   = (I + A)^-1 B                                   (unit lower-triangular solve)
        o_i     = exp(G_i) * S0^T q_i + sum_{j <= i} exp(G_i - G_j) * (k_j . q_i) * Delta_j
        S_C     = exp(G_C) * S0 + sum_j exp(G_C - G_j) * k_j (x) Delta_j

    which follows from unrolling ``S_i = exp(g_i) S_{i-1} + k_i (x) delta_i``.  Same operands
    and results as ``recurrence``; the two agree to fp32 rounding."""
    t, hv, d = v.shape
    rep = hv // q.shape[1]
    qe = (q.float().repeat_interleave(rep, 1) * (d ** -0.5)).transpose(0, 1)     # [HV, T, D]
    ke = k.float().repeat_interleave(rep, 1).transpose(0, 1)
    ve = v.float().transpose(0, 1)
    gt, bt = g.float().t(), beta.float().t()                                     # [HV, T]
    s = state.float().clone()
    out = torch.empty(hv, t, d)
    for lo in range(0, t, chunk):
        hi = min(t, lo + chunk)
        c = hi - lo
        kc, qc, vc = ke[:, lo:hi], qe[:, lo:hi], ve[:, lo:hi]
        big_g = torch.cumsum(gt[:, lo:hi], dim=1)                                # [HV, C]
        decay = torch.exp(big_g[:, :, None] - big_g[:, None, :])                 # e^(G_i - G_j)
        lower = torch.tril(torch.ones(c, c), -1)
        a = bt[:, lo:hi, None] * decay * (kc @ kc.transpose(1, 2)) * lower
        b = bt[:, lo:hi, None] * (vc - torch.exp(big_g)[:, :, None] * (kc @ s))
        delta = torch.linalg.solve_triangular(torch.eye(c)[None] + a, b, upper=False,
                                              unitriangular=True)
        causal = torch.tril(torch.ones(c, c))
        out[:, lo:hi] = torch.exp(big_g)[:, :, None] * (qc @ s) + \
            ((qc @ kc.transpose(1, 2)) * decay * causal) @ delta
        tail = torch.exp(big_g[:, -1:] - big_g)                                  # e^(G_C - G_j)
        s = torch.exp(big_g[:, -1])[:, None, None] * s + \
            (kc * tail[:, :, None]).transpose(1, 2) @ delta
    return out.transpose(0, 1).contiguous(), s


def gated_norm(o: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float,
               sigmoid_gate: bool = False) -> torch.Tensor:
    """o fp32 [T, HV, D], z f16-valued [T, HV, D] -> f16-valued [T, HV*D]."""
    n = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * weight.float()
    zf = z.float()
    gate = torch.sigmoid(zf) if sigmoid_gate else zf * torch.sigmoid(zf)
    return R.f16(n * gate).reshape(o.shape[0], -1)


class GdnRefState:
    """Per-request recurrent state for the single-request reference forward."""

    def __init__(self):
        self.state = {}
        self.hist = {}


def gdn_layer(cfg, lw, y: torch.Tensor, kv, layer: int, quantized: bool) -> torch.Tensor:
    """Mixer of one GDN layer for ONE request (used by ref.cpu_forward)."""
    from .cpu_forward import _linear_fp, _linear_q
    if not hasattr(kv, "gdn"):
        kv.gdn = GdnRefState()
    st = kv.gdn
    hk, hv, d = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
    dk, dv = hk * d, hv * d
    proj = _linear_q(lw.gdn_qkvz, y) if quantized else R.f16(_linear_fp(lw.gdn_qkvz, y))
    ab = R.f16(y).float() @ lw.gdn_ab.float().t()
    conv_dim = 2 * dk + dv
    hist = st.hist.get(layer, torch.zeros(3, conv_dim))
    state = st.state.get(layer, torch.zeros(hv, d, d))
    yc, st.hist[layer] = conv_silu_l2(proj[:, :conv_dim], hist, lw.gdn_conv, dk, d)
    t = y.shape[0]
    q = yc[:, :dk].reshape(t, hk, d)
    k = yc[:, dk:2 * dk].reshape(t, hk, d)
    v = yc[:, 2 * dk:].reshape(t, hv, d)
    g, beta = gates(ab, lw.gdn_a_log, lw.gdn_dt_bias)
    o, st.state[layer] = recurrence(q, k, v, g, beta, state)
    z = proj[:, conv_dim:].reshape(t, hv, d)
    return gated_norm(o, z, lw.gdn_norm, cfg.eps)
