"""Vectorised PyTorch E8P encoder/decoder (any device).

Same search as :func:`orinfer_b200.quant.e8p.encode_nearest`, batched over
vectors and basis rows; used to quantise whole matrices quickly on CPU and as
the oracle of the CUDA encoder kernel (which replaces the reference's
kernels/cuda/model/e8p_encode.py:61).
"""

from __future__ import annotations

import functools

import numpy as np
import torch

from . import e8p

_COORD_BIT = [0, 4, 1, 5, 2, 6, 3, 7]


@functools.lru_cache(maxsize=8)
def _tables(device_str: str):
    dev = torch.device(device_str)
    tab = torch.from_numpy(np.array(e8p.basis())).to(dev)
    return tab, tab.float().abs(), tab < 0, torch.tensor(_COORD_BIT, device=dev)


def decode_t(codes: torch.Tensor) -> torch.Tensor:
    """int32 codes [...] (low 16 bits used) -> int8 [..., 8]."""
    tab, _, _, bits = _tables(str(codes.device))
    c = codes.to(torch.int64) & 0xFFFF
    low = c & 0xFF
    par = torch.zeros_like(low)
    for b in range(8):
        par ^= (low >> b) & 1
    flips = low ^ par
    neg = (flips[..., None] >> bits) & 1
    vec = tab[(c >> 8)].to(torch.int64)
    return (vec * (1 - 2 * neg) + (1 - 2 * par)[..., None]).to(torch.int8)


def encode_nearest_t(x: torch.Tensor, chunk: int = 32768) -> torch.Tensor:
    """float [V, 8] -> int32 codes [V] (exhaustive nearest codeword)."""
    tab, mag, tneg, bits = _tables(str(x.device))
    out = torch.empty(x.shape[0], dtype=torch.int32, device=x.device)
    for lo in range(0, x.shape[0], chunk):
        xs = x[lo:lo + chunk].float()
        best_d = torch.full((xs.shape[0],), float("inf"), device=x.device)
        best_c = torch.zeros(xs.shape[0], dtype=torch.int64, device=x.device)
        for p in (0, 1):
            t = xs - float(1 - 2 * p)
            want = t < 0
            a = t.abs()
            flip = want[:, None, :] ^ tneg[None]                    # [v,256,8]
            dist = (a * a).sum(1)[:, None] - 2.0 * (a @ mag.t()) + (mag * mag).sum(1)[None]
            odd = (flip.sum(2) & 1).bool()
            tog = a[:, None, :] * mag[None]                         # toggle cost / 4
            tmin, targ = tog.min(2)
            dist = dist + torch.where(odd, 4.0 * tmin, torch.zeros_like(tmin))
            d, pick = dist.min(1)
            rows = torch.arange(xs.shape[0], device=x.device)
            fl = flip[rows, pick]
            need = odd[rows, pick]
            tcoord = targ[rows, pick]
            fl = fl ^ (need[:, None] & (torch.arange(8, device=x.device)[None] == tcoord[:, None]))
            low = (fl.to(torch.int64) << bits[None]).sum(1) ^ p
            code = (pick << 8) | low
            better = d < best_d
            best_d = torch.where(better, d, best_d)
            best_c = torch.where(better, code, best_c)
        out[lo:lo + chunk] = best_c.to(torch.int32)
    return out


def rotate_t(w: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
    from ..ref.ops_ref import hadamard_rotate
    return hadamard_rotate(w, signs)


def _scale16(v: torch.Tensor) -> torch.Tensor:
    return torch.clamp(v, min=2.0 ** -24).to(torch.float16).float()


def fit_q4_t(weight: torch.Tensor, signs: torch.Tensor, refine: int = 0):
    """[N,K] -> (int32 codes [K/128, N, 16], fp16 scale [N]); all rows at once."""
    w = rotate_t(weight.float(), signs)
    n, k = w.shape
    enc = lambda m: encode_nearest_t(m.reshape(-1, 8)).reshape(n, k // 8)
    dec = lambda c: decode_t(c).reshape(n, k).float()
    s = _scale16(w.pow(2).mean(1).sqrt() / 16.0)[:, None]
    c0 = enc(w / (4.0 * s)); q0 = dec(c0)
    c1 = enc(w / s - 4.0 * q0); q1 = dec(c1)
    for _ in range(refine):
        q = 4.0 * q0 + q1
        s = _scale16((w * q).sum(1) / (q * q).sum(1).clamp(min=1e-30))[:, None]
        c0 = enc((w / s - q1) / 4.0); q0 = dec(c0)
        c1 = enc(w / s - 4.0 * q0); q1 = dec(c1)
    packed = (c0.to(torch.int64) | (c1.to(torch.int64) << 16))
    packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32)
    kmaj = packed.reshape(n, k // 128, 16).permute(1, 0, 2).contiguous()
    return kmaj, s[:, 0].to(torch.float16)


def fit_q2_t(weight: torch.Tensor, signs: torch.Tensor, refine: int = 1):
    """[N,K] -> (int16 codes [K/128, N, 16], fp16 scale [N])."""
    w = rotate_t(weight.float(), signs)
    n, k = w.shape
    enc = lambda m: encode_nearest_t(m.reshape(-1, 8)).reshape(n, k // 8)
    dec = lambda c: decode_t(c).reshape(n, k).float()
    s = _scale16(w.pow(2).mean(1).sqrt() / 4.0)[:, None]
    c = enc(w / s); q = dec(c)
    for _ in range(refine):
        s = _scale16((w * q).sum(1) / (q * q).sum(1).clamp(min=1e-30))[:, None]
        c = enc(w / s); q = dec(c)
    c16 = torch.where(c >= 2 ** 15, c - 2 ** 16, c).to(torch.int16)
    kmaj = c16.reshape(n, k // 128, 16).permute(1, 0, 2).contiguous()
    return kmaj, s[:, 0].to(torch.float16)
