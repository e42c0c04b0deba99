"""Device-side E8P encoder entry points (K14: csrc/kernels/e8p_encode.cu)."""

from __future__ import annotations

import torch


def available() -> bool:
    from . import native
    return native.loaded() and native.has("orinfer_e8p_encode")


def encode_e8p(weight: torch.Tensor, signs: torch.Tensor, fmt: str, refine: int = 0):
    """fp32 [N,K] CUDA weights -> (codes [K/128,N,16], fp16 scale [N]) with the CUDA
    nearest-codeword kernel doing the search."""
    from . import native
    from ..quant import e8p_torch
    w = e8p_torch.rotate_t(weight.float(), signs)
    n, k = w.shape

    def enc(m):
        return native.e8p_encode(m.reshape(-1, 8).contiguous()).reshape(n, k // 8)

    dec = lambda c: e8p_torch.decode_t(c).reshape(n, k).float()
    sc = e8p_torch._scale16
    if fmt == "q4":
        s = sc(w.pow(2).mean(1).sqrt() / 16.0)[:, None]
        c0 = enc(w / (4.0 * s)); q0 = dec(c0)
        c1 = enc(w / s - 4.0 * q0); q1 = dec(c1)
        for _ in range(refine):
            q = 4.0 * q0 + q1
            s = sc((w * q).sum(1) / (q * q).sum(1).clamp(min=1e-30))[:, None]
            c0 = enc((w / s - q1) / 4.0); q0 = dec(c0)
            c1 = enc(w / s - 4.0 * q0); q1 = dec(c1)
        packed = c0.to(torch.int64) | (c1.to(torch.int64) << 16)
        packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32)
        return packed.reshape(n, k // 128, 16).permute(1, 0, 2).contiguous(), s[:, 0].half()
    s = sc(w.pow(2).mean(1).sqrt() / 4.0)[:, None]
    c = enc(w / s); q = dec(c)
    for _ in range(max(refine, 1)):
        s = sc((w * q).sum(1) / (q * q).sum(1).clamp(min=1e-30))[:, None]
        c = enc(w / s); q = dec(c)
    c16 = torch.where(c >= 2 ** 15, c - 2 ** 16, c).to(torch.int16)
    return c16.reshape(n, k // 128, 16).permute(1, 0, 2).contiguous(), s[:, 0].half()
