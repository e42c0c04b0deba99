"""Whole-model reference forward in plain PyTorch (CPU or any device).

Two arithmetic modes over the same :class:`ModelWeights`:

* ``fp32``      - the original dense fp32 weights, no quantisation anywhere.
* ``quantized`` - op for op what the CUDA engine computes (A8 activations,
  integer GEMM, FP16 boundaries, INT8 KV), built from ``ops_ref``.

The reference has no CPU inference path (its CPU code is oracles only); this
module is the build's own oracle for logits and the timed CPU baseline.
Program order follows python/orinfer_build/models/qwen35/build.py:802-1116.
"""

from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..config import ModelConfig
from ..models.weights import LayerWeights, ModelWeights, QLinear
from . import ops_ref as R


class RefKV:
    """Per-request INT8 KV for the reference path: lists of per-layer tensors."""

    def __init__(self, layers: int):
        self.k: List[Optional[torch.Tensor]] = [None] * layers
        self.v: List[Optional[torch.Tensor]] = [None] * layers
        self.length = 0

    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor):
        self.k[layer] = k if self.k[layer] is None else torch.cat([self.k[layer], k], 0)
        self.v[layer] = v if self.v[layer] is None else torch.cat([self.v[layer], v], 0)


def _linear_q(lin: QLinear, y_f16: torch.Tensor, out_f32: bool = False) -> torch.Tensor:
    """Quantised projection of an f16-valued activation (rotation inside)."""
    z = R.hadamard_rotate(y_f16, lin.signs) if lin.signs is not None else y_f16
    q, s = R.a8(z)
    return R.qgemm(q, s, lin.integers(), lin.scale, out_f32)


def _linear_fp(lin: QLinear, x: torch.Tensor) -> torch.Tensor:
    return x @ lin.dense.to(x.device).t()


def _norm_fp(v, w, eps, zc):
    r = torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)
    return v * r * (w.float() + (1.0 if zc else 0.0))


def _rope_fp(x, cos, sin):
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


def attention_layer(cfg: ModelConfig, lw: LayerWeights, y: torch.Tensor, positions: torch.Tensor,
                    kv: RefKV, layer: int, quantized: bool) -> torch.Tensor:
    """y: normed input [T, H] for ONE request; returns mixer output [T, QH*D]."""
    t = y.shape[0]
    d, qh, kvh = cfg.head_dim, cfg.q_heads, cfg.kv_heads
    cos, sin = R.rope_tables(positions, d, cfg.rope_theta, cfg.rotary_dim)
    proj = _linear_q(lw.qkv, y) if quantized else _linear_fp(lw.qkv, y)
    qw = cfg.q_dim
    gate = None
    if cfg.gated_attention:
        qg = proj[:, :qw].reshape(t, qh, 2 * d)
        q, gate = qg[..., :d], qg[..., d:]
    else:
        q = proj[:, :qw].reshape(t, qh, d)
    k = proj[:, qw:qw + cfg.kv_dim].reshape(t, kvh, d)
    v = proj[:, qw + cfg.kv_dim:].reshape(t, kvh, d)
    offset = int(positions[0])
    if quantized:
        qn = R.qk_norm_rope(q, lw.q_norm if cfg.qk_norm else None, cos, sin, cfg.eps,
                            cfg.zero_centered_norm)
        kn = R.qk_norm_rope(k, lw.k_norm if cfg.qk_norm else None, cos, sin, cfg.eps,
                            cfg.zero_centered_norm)
        kq, ks = R.kv_quant(kn)
        vq, vs = R.kv_quant(R.f16(v))
        kv.append(layer, R.kv_dequant(kq, ks), R.kv_dequant(vq, vs))
        out = R.causal_gqa(qn, kv.k[layer], kv.v[layer], offset, gate)
    else:
        if cfg.qk_norm:
            q = _norm_fp(q, lw.q_norm, cfg.eps, cfg.zero_centered_norm)
            k = _norm_fp(k, lw.k_norm, cfg.eps, cfg.zero_centered_norm)
        q, k = _rope_fp(q, cos, sin), _rope_fp(k, cos, sin)
        kv.append(layer, k, v)
        kk = kv.k[layer].repeat_interleave(qh // kvh, 1)
        vv = kv.v[layer].repeat_interleave(qh // kvh, 1)
        s = torch.einsum("qhd,khd->hqk", q, kk) / math.sqrt(d)
        tk = kk.shape[0]
        mask = torch.arange(tk)[None, :] > (offset + torch.arange(t))[:, None]
        p = torch.softmax(s.masked_fill(mask[None].to(s.device), float("-inf")), -1)
        o = torch.einsum("hqk,khd->qhd", p, vv)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        out = o.reshape(t, qh * d)
    return out


def dense_ffn(lw: LayerWeights, y: torch.Tensor, quantized: bool) -> torch.Tensor:
    if quantized:
        gu = _linear_q(lw.gate_up, y)
        f = gu.shape[-1] // 2
        return _linear_q(lw.down, R.silu_mul(gu[:, :f], gu[:, f:]))
    gu = _linear_fp(lw.gate_up, y)
    f = gu.shape[-1] // 2
    return _linear_fp(lw.down, torch.nn.functional.silu(gu[:, :f]) * gu[:, f:])


def moe_ffn(cfg: ModelConfig, lw: LayerWeights, y: torch.Tensor, quantized: bool) -> torch.Tensor:
    """softmax -> top-k (ties to the lower expert id) -> optional renormalise ->
    sum_k p_k * expert_k(y) (+ sigmoid(shared gate) * shared(y))
    (kernels/cuda/model/moe.py:413 router_topk, :498-557 moe_combine)."""
    logits = (y.float() @ lw.router.float().t())
    e = cfg.experts
    probs = torch.softmax(logits[:, :e], -1)
    # stable descending sort gives the lower id on ties
    order = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, :cfg.top_k]
    w = torch.gather(probs, 1, order)
    if cfg.renormalize:
        w = w / w.sum(-1, keepdim=True)
    out = torch.zeros(y.shape[0], cfg.hidden)
    for tok in range(y.shape[0]):
        for j in range(cfg.top_k):
            ex = int(order[tok, j])
            if not lw.expert_gate_up.owns(ex):        # another rank's expert
                continue
            gu_l, dn_l = lw.expert_gate_up.expert(ex), lw.expert_down.expert(ex)
            row = y[tok:tok + 1]
            if quantized:
                gu = _linear_q(gu_l, row)
                f = gu.shape[-1] // 2
                o = _linear_q(dn_l, R.silu_mul(gu[:, :f], gu[:, f:]))
            else:
                gu = _linear_fp(gu_l, row)
                f = gu.shape[-1] // 2
                o = _linear_fp(dn_l, torch.nn.functional.silu(gu[:, :f]) * gu[:, f:])
            out[tok] += w[tok, j] * o[0]
    if lw.shared_gate_up is not None and getattr(lw, "_add_shared", True):
        sh = LayerWeights("attn", lw.in_norm, lw.post_norm, gate_up=lw.shared_gate_up,
                          down=lw.shared_down)
        out = out + torch.sigmoid(logits[:, e:e + 1]) * dense_ffn(sh, y, quantized)
    return R.f16(out) if quantized else out


def forward_request(weights: ModelWeights, ids: torch.Tensor, start: int, kv: RefKV,
                    quantized: bool, return_hidden: bool = False):
    """Run tokens ``ids`` (positions start..start+T-1) of one request; returns
    fp32 logits [T, V] for every row (and the final-norm hidden when asked)."""
    cfg = weights.config
    t = ids.shape[0]
    positions = torch.arange(start, start + t)
    if quantized:
        x = R.embed_w8(ids, weights.embed_q, weights.embed_s)
    else:
        x = weights.embed_dense[ids.long()]
    resid = torch.zeros(t, cfg.hidden)
    zc = cfg.zero_centered_norm
    for i, lw in enumerate(weights.layers):
        if lw.kind != "attn":
            from .gdn_ref import gdn_layer
            resid = resid + x
            y = R.rms_norm(resid, lw.in_norm, cfg.eps, zc) if quantized else \
                _norm_fp(resid, lw.in_norm, cfg.eps, zc)
            mix = gdn_layer(cfg, lw, y, kv, i, quantized)
            x = _linear_q(lw.gdn_out, mix) if quantized else _linear_fp(lw.gdn_out, mix)
        else:
            resid = resid + x
            y = R.rms_norm(resid, lw.in_norm, cfg.eps, zc) if quantized else \
                _norm_fp(resid, lw.in_norm, cfg.eps, zc)
            mix = attention_layer(cfg, lw, y, positions, kv, i, quantized)
            x = _linear_q(lw.o, mix) if quantized else _linear_fp(lw.o, mix)
        resid = resid + x
        y = R.rms_norm(resid, lw.post_norm, cfg.eps, zc) if quantized else \
            _norm_fp(resid, lw.post_norm, cfg.eps, zc)
        x = moe_ffn(cfg, lw, y, quantized) if cfg.experts else dense_ffn(lw, y, quantized)
    resid = resid + x
    kv.length = start + t
    if quantized:
        h = R.rms_norm(resid, weights.final_norm, cfg.eps, zc)
        logits = _linear_q(weights.head, h, out_f32=True)
    else:
        h = _norm_fp(resid, weights.final_norm, cfg.eps, zc)
        logits = _linear_fp(weights.head, h)
    return (logits, h) if return_hidden else logits


def generate_greedy(weights: ModelWeights, prompt: torch.Tensor, new_tokens: int,
                    quantized: bool = True):
    """Prefill then greedy decode; returns (tokens, logits of every sampled position)."""
    kv = RefKV(weights.config.layers)
    logits = forward_request(weights, prompt, 0, kv, quantized)[-1:]
    out, trace = [], []
    for _ in range(new_tokens):
        tok = int(R.argmax_lowest(logits)[0])
        out.append(tok)
        trace.append(logits[0].clone())
        logits = forward_request(weights, torch.tensor([tok]), kv.length, kv, quantized)
    return out, torch.stack(trace)
