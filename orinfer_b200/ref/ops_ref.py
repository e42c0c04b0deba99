"""Plain PyTorch restatement of every device op (the numerics oracle).

Each function states, in fp32 torch code, exactly what the matching CUDA
kernel in ``csrc/kernels`` computes, including the explicit FP16 rounding
boundaries, so kernel tests can compare tightly.  The precision contract is
the reference's (AGENTS.md:27-33; kernels/cuda/model/integer_core.py:19):
FP32 residual stream, FP16 activations at named boundaries, INT8 per-token
activations, INT32 accumulation, FP32 rescale ``(acc * s_w) * s_a``.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

BLOCK = 128


def f16(x: torch.Tensor) -> torch.Tensor:
    """Round to FP16 and come back to fp32 (an explicit rounding boundary)."""
    return x.to(torch.float16).to(torch.float32)


def hadamard_rotate(x: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
    k = x.shape[-1]
    y = (x.float() * signs.float()).reshape(*x.shape[:-1], k // BLOCK, BLOCK)
    h = 1
    while h < BLOCK:
        y = y.reshape(*y.shape[:-1], BLOCK // (2 * h), 2, h)
        y = torch.stack([y[..., 0, :] + y[..., 1, :], y[..., 0, :] - y[..., 1, :]], dim=-2)
        y = y.reshape(*x.shape[:-1], k // BLOCK, BLOCK)
        h *= 2
    return (y * (BLOCK ** -0.5)).reshape(x.shape)


def a8(z: torch.Tensor):
    """Per-row absmax INT8; scale is an FP16 value (>= 2^-24, 1 for zero rows)."""
    amax = z.abs().amax(-1)
    scale = torch.where(amax > 0, torch.clamp(amax / 127.0, min=2.0 ** -24), torch.ones_like(amax))
    scale = f16(scale)
    q = torch.clamp(torch.round(z / scale[..., None]), -127, 127).to(torch.int8)
    return q, scale


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    g = gate.float()
    return f16((g * torch.sigmoid(g)) * up.float())


def rms_norm(v: torch.Tensor, w: torch.Tensor, eps: float, zero_centered: bool) -> torch.Tensor:
    v = v.float()
    r = torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)
    return f16((v * r) * (w.float() + (1.0 if zero_centered else 0.0)))


def act_prep(x: Optional[torch.Tensor], resid: Optional[torch.Tensor],
             norm_w: Optional[torch.Tensor], signs: Optional[torch.Tensor], eps: float = 1e-6,
             zero_centered: bool = False, swiglu: bool = False):
    """residual-add -> RMSNorm -> (SwiGLU) -> block-128 rotation -> A8.

    Returns ``(q int8 [M,K], scale f32 [M], resid_out f32 or None, y f16-valued)``.
    Restates residual_norm_rotate_a8 / rotate_activation_a8 of the reference
    (kernels/cuda/model/rotation_a8.py:267,608-659).
    """
    if swiglu:
        f = x.shape[-1] // 2
        y = silu_mul(x[..., :f], x[..., f:])
        resid_out = None
    else:
        v = x.float() if x is not None else torch.zeros_like(resid)
        if resid is not None:
            v = v + resid
        resid_out = v if resid is not None else None
        y = rms_norm(v, norm_w, eps, zero_centered) if norm_w is not None else f16(v)
    z = hadamard_rotate(y, signs) if signs is not None else y
    q, scale = a8(z)
    return q, scale, resid_out, y


def qgemm(q: torch.Tensor, s_a: torch.Tensor, w_int: torch.Tensor, s_w: torch.Tensor,
          out_f32: bool = False) -> torch.Tensor:
    """out[m,n] = (sum_k q[m,k] * w[n,k]) * s_w[n] * s_a[m]; exact integer sum."""
    acc = (q.double() @ w_int.double().t()).float()          # exact: |acc| < 2^31 << 2^53
    out = (acc * s_w.float()[None, :]) * s_a.float()[:, None]
    return out if out_f32 else f16(out)


def embed_w8(ids: torch.Tensor, table_q: torch.Tensor, table_s: torch.Tensor) -> torch.Tensor:
    return f16(table_q[ids.long()].float() * table_s.float()[ids.long()][:, None])


def rope_tables(positions: torch.Tensor, dim: int, theta: float, rotary_dim: int = 0):
    """cos/sin [M, dim/2] in fp32 for NeoX-style rotary embedding (pairs ``(i, i + dim/2)``).

    ``rotary_dim`` (0 = the whole head) turns only ``rotary_dim / 2`` pairs, with frequencies
    ``theta ** (-2i / rotary_dim)``; the other pairs get angle 0.  A checkpoint whose partial
    rotary acts on the first ``rotary_dim`` channels in pairs ``(i, i + rotary_dim/2)`` is
    brought to this pairing by permuting its q / k channels at conversion time."""
    half = dim // 2
    r = rotary_dim or dim
    inv = torch.zeros(half, dtype=torch.float64, device=positions.device)
    inv[: r // 2] = theta ** (-torch.arange(0, r, 2, dtype=torch.float64,
                                            device=positions.device) / r)
    ang = positions.double()[:, None] * inv[None, :]
    return ang.cos().float(), ang.sin().float()


def qk_norm_rope(x: torch.Tensor, w: Optional[torch.Tensor], cos: torch.Tensor, sin: torch.Tensor,
                 eps: float, zero_centered: bool) -> torch.Tensor:
    """x [M, heads, D] -> per-head RMSNorm (FP16 boundary) then NeoX rotation, FP16 result."""
    y = rms_norm(x, w, eps, zero_centered) if w is not None else f16(x.float())
    half = x.shape[-1] // 2
    a, b = y[..., :half], y[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return f16(torch.cat([a * c - b * s, b * c + a * s], dim=-1))


def kv_quant(x: torch.Tensor, group: int = 64):
    """x f16-valued [..., D] -> INT8 and FP16-valued scales [..., D/group] (min 2^-24)."""
    g = x.float().reshape(*x.shape[:-1], x.shape[-1] // group, group)
    scale = f16(torch.clamp(g.abs().amax(-1) / 127.0, min=2.0 ** -24))
    q = torch.clamp(torch.round(g / scale[..., None]), -127, 127).to(torch.int8)
    return q.reshape(x.shape), scale


def kv_dequant(q: torch.Tensor, scale: torch.Tensor, group: int = 64) -> torch.Tensor:
    g = q.float().reshape(*q.shape[:-1], q.shape[-1] // group, group)
    return (g * scale.float()[..., None]).reshape(q.shape)


def causal_gqa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_offset: int,
               gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One request: q [Tq, QH, D]; k, v [Tk, KVH, D] (already dequantised).

    Query row i sits at absolute position ``q_offset + i`` and sees keys
    ``0..q_offset+i``.  Optional sigmoid output gate.  Returns f16-valued [Tq, QH*D].
    """
    tq, qh, d = q.shape
    tk, kvh, _ = k.shape
    rep = qh // kvh
    kk = k.float().repeat_interleave(rep, dim=1)
    vv = v.float().repeat_interleave(rep, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kk) / math.sqrt(d)
    qpos = q_offset + torch.arange(tq, device=q.device)
    mask = torch.arange(tk, device=q.device)[None, :] > qpos[:, None]
    s = s.masked_fill(mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("hqk,khd->qhd", p, vv)
    if gate is not None:
        o = o * torch.sigmoid(gate.float())
    return f16(o.reshape(tq, qh * d))


def argmax_lowest(logits: torch.Tensor) -> torch.Tensor:
    """Greedy token with the lowest-index tie rule (kernels/cuda/model/greedy.py:11,83)."""
    m = logits.amax(-1, keepdim=True)
    idx = torch.arange(logits.shape[-1], device=logits.device).expand_as(logits)
    big = torch.full_like(idx, logits.shape[-1])
    return torch.where(logits == m, idx, big).amin(-1).to(torch.int32)
