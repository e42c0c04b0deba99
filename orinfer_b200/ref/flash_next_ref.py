"""fp32 PyTorch statement of the Flash-Next specific blocks: hyper-connection streams (HC),
the per-layer embedding memory block (PLE) and query-selected sparse attention (QSA).

These are oracles for a Flash-Next class model (hybrid GDN / gated attention stack with 512
experts, which the hybrid MoE runner already covers) — the three blocks below are what that
family adds.  The arithmetic restates the reference's own Torch oracle
(python/orinfer_build/models/flash_next/reference/math.py:15-61 and reference/qsa.py:7-72):

* HC keeps ``S`` residual streams per token.  Reading a block input mixes the streams with
  input-dependent sigmoid gates from a low-rank projection; writing adds the block output to
  every stream under a second input-dependent gate ``2 * sigmoid(.)``.
* PLE injects rows of a conditional memory (``core/host_rows.py``) into the streams: a
  key / value projection of the gathered features, a signed-square-root gate from the
  key-query agreement, and a dilated causal depthwise convolution over time.
* QSA scores groups of four keys by ``sum_h relu(q_h . k) / sqrt(128)`` against pooled index
  keys, keeps the best 512 groups (stable, lower index wins ties) plus the incomplete tail
  group, and runs softmax attention over the selected positions only.

Unlike the reference oracle, ``causal_conv`` and ``ple`` take and return the convolution
history, so a prompt processed in chunks gives the same result as in one pass.
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

GROUP = 4              # keys per index group
TOP_GROUPS = 512       # groups kept per query
INDEX_DIM = 128
ROPE_DIM = 64


def rms(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Zero-centred RMSNorm in fp32, rounded to the input dtype."""
    v = x.float()
    return (v * torch.rsqrt(v.square().mean(-1, keepdim=True) + eps)
            * (weight.float() + 1.0)).to(x.dtype)


# ------------------------------------------------------------------ hyper-connections
def hc_read(x: torch.Tensor, w: Dict[str, torch.Tensor], inject: bool = True
            ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """x [T, S, H] -> (block input [T, H], write gate [T, S] or None).
    w: norm [S*H], down [R, S*H], up [S*H, R], inject [S, S*H]."""
    t, s, h = x.shape
    n = rms(x, w["norm"].reshape(s, h))
    flat = n.flatten(1)
    low = F.silu(F.linear(flat, w["down"]) / s)
    gates = torch.sigmoid(F.linear(low, w["up"]).reshape(t, s, h))
    mixed = (n * gates).mean(1)
    gate = 2.0 * torch.sigmoid(F.linear(flat, w["inject"]) / s) if inject else None
    return mixed, gate


def hc_write(x: torch.Tensor, block: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """Add a block output [T, H] to every stream of x [T, S, H] under gate [T, S]."""
    return x + block[:, None, :] * gate[:, :, None]


# ------------------------------------------------------------------ PLE
def causal_conv(x: torch.Tensor, weight: torch.Tensor, dilation: int = 1,
                history: Optional[torch.Tensor] = None, round_before_silu: bool = False
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Depthwise causal convolution + SiLU over time.  x [T, C], weight [C, K]; ``history``
    holds the last (K-1)*dilation input rows of the request (zeros at its start).  Returns
    (output [T, C], new history)."""
    if x.ndim != 2 or weight.ndim != 2 or x.shape[1] != weight.shape[0] or dilation < 1:
        raise ValueError("invalid causal convolution operands")
    reach = (weight.shape[1] - 1) * dilation
    if history is None:
        history = x.new_zeros(reach, x.shape[1])
    if history.shape != (reach, x.shape[1]):
        raise ValueError("convolution history has the wrong extent")
    seq = torch.cat([history, x]).float()
    y = F.conv1d(seq.t()[None], weight.float()[:, None], groups=x.shape[1],
                 dilation=dilation)[0].t()
    if round_before_silu:
        y = y.to(x.dtype).float()
    return F.silu(y).to(x.dtype), seq[seq.shape[0] - reach:].to(x.dtype)


def ple(x: torch.Tensor, features: torch.Tensor, w: Dict[str, torch.Tensor], dilation: int = 3,
        history: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [T, S, H] streams, features [T, F] gathered memory rows ->
    (updated streams, convolution history)."""
    t, s, h = x.shape
    key = rms(F.linear(features, w["key"]).reshape(t, s, h), w["norm_key"].reshape(s, h))
    value = F.linear(features, w["value"])                         # [T, H]
    query = rms(x, w["norm_query"].reshape(s, h))
    agree = (key * query).sum(-1, keepdim=True) / math.sqrt(h)
    gate = agree.abs().clamp_min(1e-6).sqrt() * agree.sign()       # signed square root
    gated = torch.sigmoid(gate) * value[:, None, :]
    normed = rms(gated, w["norm_conv"].reshape(s, h))
    conv, history = causal_conv(normed.flatten(1), w["conv"], dilation, history,
                                round_before_silu=True)
    return x + (gated.flatten(1) + conv).reshape(t, s, h), history


# ------------------------------------------------------------------ QSA
def qsa_rope(x: torch.Tensor, positions: torch.Tensor, theta: float = 1e7) -> torch.Tensor:
    """NeoX rotation of the first 64 channels of the last axis; x [T, heads, D]."""
    pos = torch.as_tensor(positions, dtype=torch.float32, device=x.device)
    inv = theta ** (-torch.arange(0, ROPE_DIM, 2, device=x.device).float() / ROPE_DIM)
    ang = pos[:, None, None] * inv[None, None, :]
    a, b = x[..., :ROPE_DIM].float().chunk(2, -1)
    out = x.clone()
    out[..., :ROPE_DIM] = torch.cat([a * ang.cos() - b * ang.sin(),
                                     b * ang.cos() + a * ang.sin()], -1).to(x.dtype)
    return out


def qsa_index(qk: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, first: int = 0
              ) -> Tuple[torch.Tensor, torch.Tensor]:
    """qk [T, 5, 128]: four index-query heads and one index key per token, tokens at positions
    ``first ..`` (``first`` a multiple of 4).  Returns (queries [T, 4, 128] normed + rotated at
    their positions, group keys [T // 4, 128]: mean of four keys, rounded, normed, rotated at
    the first member's position)."""
    t = qk.shape[0]
    pos = torch.arange(first, first + t, device=qk.device)
    q = qsa_rope(rms(qk[:, :GROUP], q_weight), pos)
    groups = t // GROUP
    pooled = qk[:groups * GROUP, GROUP].float().reshape(groups, GROUP, qk.shape[-1]).mean(1).to(
        qk.dtype)
    k = qsa_rope(rms(pooled[:, None], k_weight), pos[:groups * GROUP:GROUP])[:, 0]
    return q, k


def qsa_select(query: torch.Tensor, cache: torch.Tensor, positions, top: int = TOP_GROUPS
               ) -> torch.Tensor:
    """For each query [4, 128] at ``positions[i]``: the selected key positions, padded with
    -1 to ``top * 4 + 3``.  All complete causal groups are candidates; at most ``top`` are kept
    by exact score order (ties to the lower index); the incomplete tail group always follows."""
    width = top * GROUP + GROUP - 1
    rows = []
    for q, p in zip(query, positions):
        p = int(p)
        n = (p + 1) // GROUP
        if n <= top:
            ids = torch.arange(n, device=q.device)
        else:
            score = (q.float() @ cache[:n].float().t()).relu().sum(0) * INDEX_DIM ** -0.5
            ids = score.argsort(descending=True, stable=True)[:top]
        chosen = (ids[:, None] * GROUP + torch.arange(GROUP, device=q.device)).flatten()
        tail = torch.arange(n * GROUP, p + 1, device=q.device)
        chosen = torch.cat([chosen, tail]).int()
        rows.append(F.pad(chosen, (0, width - chosen.numel()), value=-1))
    return torch.stack(rows)


def qsa_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                  gate: torch.Tensor, selected: torch.Tensor, scale: Optional[float] = None
                  ) -> torch.Tensor:
    """query [T, Hq, D]; key / value [context, Hkv, D]; gate [T, Hq, D]; selected [T, width].
    Softmax attention over the selected positions, output times sigmoid(gate)."""
    rep = query.shape[1] // key.shape[1]
    scale = scale if scale is not None else query.shape[-1] ** -0.5
    out = []
    for q, g, ids in zip(query, gate, selected):
        ids = ids[ids >= 0].long()
        k = key[ids].repeat_interleave(rep, 1).float()
        v = value[ids].repeat_interleave(rep, 1).float()
        p = (torch.einsum("hd,shd->hs", q.float(), k) * scale).softmax(-1)
        y = torch.einsum("hs,shd->hd", p, v)
        out.append((y * torch.sigmoid(g.float())).to(query.dtype))
    return torch.stack(out)


def quantize_kv(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """INT8 group-64 with FP16 scales (the paged KV format of every model here)."""
    g = x.float().reshape(*x.shape[:-1], -1, 64)
    scale = (g.abs().amax(-1) / 127).clamp_min(2 ** -24).half()
    codes = (g / scale.float()[..., None]).round().clamp(-127, 127).to(torch.int8)
    return codes.reshape_as(x), scale


def dequantize_kv(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return (codes.float().reshape(*codes.shape[:-1], -1, 64) * scale.float()[..., None]).flatten(-2)
