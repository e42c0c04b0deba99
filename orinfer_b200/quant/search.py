"""Weight-MSE search over two-stage E8P codes: exact top-8 coarse candidates and the
"beam-8" refinement of an existing Q4 encoding.

Nearest rounding picks the coarse code first and the residual code second, so a coarse
codeword that is slightly farther from the target can still win once its residual is
rounded.  The beam search looks at the eight nearest coarse codewords of every 8-vector,
rounds the residual of each, and keeps the pair with the smallest total error, unless the
incumbent pair is already better.  Scales are refitted by least squares between passes and
the best (codes, scale) seen per row is what is returned, so the result is never worse than
the input encoding in weight MSE.

PyTorch on any device; the exhaustive distance table ([vectors, 65536]) is built in
chunks.  Role of python/orinfer_build/quantization/e8p_q4_gpu.py:67-159 (``refine``) and of
the top-8 encoder kernels/cuda/model/e8p_encode.py:237.
"""

from __future__ import annotations

import functools

import numpy as np
import torch

from . import e8p
from .e8p_torch import decode_t, encode_nearest_t, rotate_t

BEAM = 8


@functools.lru_cache(maxsize=4)
def codebook(device_str: str) -> torch.Tensor:
    """All 65536 codewords as float32 [65536, 8] (2 MiB)."""
    codes = torch.arange(65536, dtype=torch.int32, device=torch.device(device_str))
    return decode_t(codes).float()


def nearest_top8(x: torch.Tensor, chunk: int = 512) -> torch.Tensor:
    """float [V, 8] -> int32 [V, 8]: the eight nearest codewords of each vector, nearest
    first (exhaustive over the 65536 codewords, hence exact)."""
    book = codebook(str(x.device))
    norms = (book * book).sum(1)
    out = torch.empty(x.shape[0], BEAM, dtype=torch.int32, device=x.device)
    for lo in range(0, x.shape[0], chunk):
        xs = x[lo:lo + chunk].float()
        dist = norms[None, :] - 2.0 * (xs @ book.t())          # + |x|^2, constant per row
        idx = torch.topk(dist, BEAM, dim=1, largest=False, sorted=True).indices
        out[lo:lo + chunk] = idx.to(torch.int32)
    return out


def _scale16(v: torch.Tensor) -> torch.Tensor:
    s = torch.clamp(v, min=2.0 ** -24).to(torch.float16)
    if not bool(torch.isfinite(s).all()):
        raise ValueError("scale not representable in FP16")
    return s


def refine_q4(weight, q4: e8p.Q4Weight, *, iterations: int = 8, beam_passes: int = 2,
              device: str = "cpu") -> e8p.Q4Weight:
    """Improves ``q4`` (an encoding of ``weight`` [N, K]) in weight MSE.

    ``iterations`` alternating passes (refit scale, re-round coarse given residual, re-round
    residual), then ``beam_passes`` top-8 passes.  Callers bound memory by passing row
    chunks."""
    if not isinstance(iterations, int) or not 0 <= iterations <= 8:
        raise ValueError("iterations must be in 0..8")
    dev = torch.device(device)
    raw = torch.as_tensor(np.asarray(weight, np.float32), device=dev)
    n, k = q4.shape
    if raw.shape != (n, k) or not bool(torch.isfinite(raw).all()):
        raise ValueError("weight and encoding shapes differ")
    signs = torch.as_tensor(q4.signs.astype(np.float32), device=dev)
    w = rotate_t(raw, signs)
    target = w.reshape(n, k // 8, 8)
    packed = torch.as_tensor(q4.packed.astype(np.int64), device=dev)
    first, second = packed & 0xFFFF, packed >> 16
    scale = torch.as_tensor(q4.scales, device=dev)
    grid = lambda c: decode_t(c.to(torch.int32)).float()
    q0, q1 = grid(first), grid(second)

    def loss_of(sc, a, b):
        return (w - sc.float()[:, None] * (4 * a + b).reshape(n, k)).square().sum(1)

    best = {"loss": loss_of(scale, q0, q1), "first": first.clone(), "second": second.clone(),
            "scale": scale.clone()}

    def keep():
        cur = loss_of(scale, q0, q1)
        better = cur < best["loss"]
        best["first"] = torch.where(better[:, None], first, best["first"])
        best["second"] = torch.where(better[:, None], second, best["second"])
        best["scale"] = torch.where(better, scale, best["scale"])
        best["loss"] = torch.minimum(best["loss"], cur)

    def refit():
        q = (4 * q0 + q1).reshape(n, k)
        return _scale16((w * q).sum(1) / q.square().sum(1).clamp_min(1e-30))

    def nearest(values):
        ids = encode_nearest_t(values.reshape(-1, 8)).to(torch.int64).reshape(n, k // 8)
        return ids, grid(ids)

    for _ in range(iterations):
        scale = refit()
        keep()
        normal = target / scale.float()[:, None, None]
        first, q0 = nearest((normal - q1) / 4)
        second, q1 = nearest(normal - 4 * q0)
        keep()
    first, second, scale = best["first"].clone(), best["second"].clone(), best["scale"].clone()
    q0, q1 = grid(first), grid(second)
    for _ in range(beam_passes):
        normal = target / scale.float()[:, None, None]
        cand = nearest_top8((normal / 4).reshape(-1, 8)).to(torch.int64).reshape(n, k // 8, BEAM)
        resid = normal[:, :, None, :] - 4 * grid(cand)                    # [n, k/8, 8, 8]
        rcode = encode_nearest_t(resid.reshape(-1, 8)).to(torch.int64).reshape(n, k // 8, BEAM)
        err = (resid - grid(rcode)).square().sum(-1)
        pick = err.argmin(-1, keepdim=True)
        c0 = cand.gather(-1, pick).squeeze(-1)
        c1 = rcode.gather(-1, pick).squeeze(-1)
        incumbent = (normal - 4 * q0 - q1).square().sum(-1)
        better = err.gather(-1, pick).squeeze(-1) < incumbent
        first, second = torch.where(better, c0, first), torch.where(better, c1, second)
        q0, q1 = grid(first), grid(second)
        keep()
        scale = refit()
        keep()
    out = (best["first"] | (best["second"] << 16)).cpu().numpy().astype(np.uint32)
    return e8p.Q4Weight(out, best["scale"].cpu().numpy().astype(np.float16), q4.signs.copy())
