"""A Flash-Next class decoder as an fp32 PyTorch oracle model: hyper-connection residual streams,
a conditional-memory (PLE) block fed by n-gram addressed host rows, groups of gated-delta-rule
layers closed by a query-selected sparse attention layer, and a routed expert FFN with a shared
expert.  It exists to pin the family's semantics (chunking, state carry, sparse selection) on
the CPU; the CUDA runner serves the hybrid GDN / MoE part of this family, the three extra
blocks have no device kernels yet.

Block order per layer (reference: crates/orinfer-models/src/flash_next/plan.rs, hc.rs,
python/orinfer_build/models/flash_next/reference/teacher.py): streams -> [PLE at its layers]
-> hc_read -> mixer (GDN with a sigmoid-gated norm, or QSA attention) -> hc_write -> hc_read
-> experts -> hc_write; the head reads the mean of the streams.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..ref import flash_next_ref as FN
from ..ref import gdn_ref as G


@dataclass
class FlashNextConfig:
    vocab: int = 256
    hidden: int = 64
    streams: int = 4
    hc_rank: int = 16
    layers: int = 4
    attention_period: int = 4          # every 4th layer is QSA attention, the others GDN
    q_heads: int = 4
    kv_heads: int = 2
    head_dim: int = 128                # QSA index width is 128; rotary covers 64 channels
    gdn_k_heads: int = 2
    gdn_v_heads: int = 4
    gdn_head_dim: int = 32
    experts: int = 8
    top_k: int = 2
    expert_ffn: int = 32
    shared_ffn: int = 32
    ple_layers: tuple = (0,)
    ple_features: int = 24
    top_groups: int = FN.TOP_GROUPS
    eps: float = 1e-6

    def is_attention(self, layer: int) -> bool:
        return (layer + 1) % self.attention_period == 0


def _w(gen, *shape, scale=None):
    scale = scale if scale is not None else shape[-1] ** -0.5
    return torch.randn(*shape, generator=gen) * scale


def random_weights(cfg: FlashNextConfig, seed: int = 0) -> dict:
    gen = torch.Generator().manual_seed(seed)
    s, h = cfg.streams, cfg.hidden

    def hc():
        return {"norm": torch.zeros(s * h), "down": _w(gen, cfg.hc_rank, s * h),
                "up": _w(gen, s * h, cfg.hc_rank), "inject": _w(gen, s, s * h)}

    layers = []
    for i in range(cfg.layers):
        lw = {"hc_mix": hc(), "hc_ffn": hc(),
              "router": _w(gen, cfg.experts, h), "shared_gate": _w(gen, 1, h),
              "gate_up": _w(gen, cfg.experts, 2 * cfg.expert_ffn, h),
              "down": _w(gen, cfg.experts, h, cfg.expert_ffn),
              "shared_gate_up": _w(gen, 2 * cfg.shared_ffn, h),
              "shared_down": _w(gen, h, cfg.shared_ffn)}
        if cfg.is_attention(i):
            d = cfg.head_dim
            lw.update(q=_w(gen, cfg.q_heads * d, h), gate=_w(gen, cfg.q_heads * d, h),
                      k=_w(gen, cfg.kv_heads * d, h), v=_w(gen, cfg.kv_heads * d, h),
                      index=_w(gen, 5 * FN.INDEX_DIM, h), index_q_norm=torch.zeros(FN.INDEX_DIM),
                      index_k_norm=torch.zeros(FN.INDEX_DIM), o=_w(gen, h, cfg.q_heads * d))
        else:
            dk, dv = cfg.gdn_k_heads * cfg.gdn_head_dim, cfg.gdn_v_heads * cfg.gdn_head_dim
            lw.update(qkvz=_w(gen, 2 * dk + 2 * dv, h), ab=_w(gen, 2 * cfg.gdn_v_heads, h),
                      conv=_w(gen, 2 * dk + dv, 4, scale=0.5), a_log=torch.zeros(cfg.gdn_v_heads),
                      dt_bias=torch.zeros(cfg.gdn_v_heads), norm=torch.ones(cfg.gdn_head_dim),
                      o=_w(gen, h, dv))
        if i in cfg.ple_layers:
            lw["ple"] = {"key": _w(gen, s * h, cfg.ple_features),
                         "value": _w(gen, h, cfg.ple_features),
                         "norm_key": torch.zeros(s * h), "norm_query": torch.zeros(s * h),
                         "norm_conv": torch.zeros(s * h), "conv": _w(gen, s * h, 4, scale=0.5)}
        layers.append(lw)
    return {"embed": _w(gen, cfg.vocab, h, scale=1.0), "layers": layers,
            "final_norm": torch.zeros(h), "head": _w(gen, cfg.vocab, h)}


@dataclass
class FlashNextState:
    """Everything request-private: committed tokens (the n-gram hasher reads its last three),
    per-layer recurrent state, convolution histories and caches."""
    tokens: List[int] = field(default_factory=list)
    layer: Dict[int, dict] = field(default_factory=dict)


class FlashNextOracle:
    def __init__(self, cfg: FlashNextConfig, weights: dict, memory=None):
        """``memory``: ``core.host_rows.ConditionalMemory`` whose hashed layers are the model's
        PLE layers, in order; None feeds zero features."""
        self.cfg, self.w, self.memory = cfg, weights, memory

    # ------------------------------------------------------------------ blocks
    def _features(self, st: FlashNextState, tokens: List[int], slot: int) -> torch.Tensor:
        t = len(tokens)
        if self.memory is None:
            return torch.zeros(t, self.cfg.ple_features)
        rows, valid = self.memory.lookup(st.tokens, tokens)        # [T, layers, 3*heads, dim]
        feats = torch.from_numpy(rows[:, slot]).reshape(t, -1)
        if feats.shape[1] != self.cfg.ple_features:
            raise ValueError("memory rows do not add up to the PLE feature width")
        return feats

    def _gdn(self, lw, y, ls):
        c = self.cfg
        hk, hv, d = c.gdn_k_heads, c.gdn_v_heads, c.gdn_head_dim
        dk, dv = hk * d, hv * d
        t = y.shape[0]
        proj = F.linear(y, lw["qkvz"])
        conv_dim = 2 * dk + dv
        hist = ls.get("hist", torch.zeros(3, conv_dim))
        state = ls.get("state", torch.zeros(hv, d, d))
        yc, ls["hist"] = G.conv_silu_l2(proj[:, :conv_dim], hist, lw["conv"], dk, d)
        g, beta = G.gates(F.linear(y, lw["ab"]), lw["a_log"], lw["dt_bias"])
        o, ls["state"] = G.recurrence(yc[:, :dk].reshape(t, hk, d),
                                      yc[:, dk:2 * dk].reshape(t, hk, d),
                                      yc[:, 2 * dk:].reshape(t, hv, d), g, beta, state)
        z = proj[:, conv_dim:].reshape(t, hv, d)
        return F.linear(G.gated_norm(o, z, lw["norm"], c.eps, sigmoid_gate=True), lw["o"])

    def _attention(self, lw, y, ls, first: int):
        c = self.cfg
        t, d = y.shape[0], c.head_dim
        pos = torch.arange(first, first + t)
        q = FN.qsa_rope(F.linear(y, lw["q"]).reshape(t, c.q_heads, d), pos)
        k = FN.qsa_rope(F.linear(y, lw["k"]).reshape(t, c.kv_heads, d), pos)
        v = F.linear(y, lw["v"]).reshape(t, c.kv_heads, d)
        gate = F.linear(y, lw["gate"]).reshape(t, c.q_heads, d)
        idx = F.linear(y, lw["index"]).reshape(t, 5, FN.INDEX_DIM)
        for name, new in (("k", k), ("v", v), ("idx", idx)):
            ls[name] = new if name not in ls else torch.cat([ls[name], new])
        # index keys are pooled over complete groups of the whole context
        iq = FN.qsa_rope(FN.rms(idx[:, :4], lw["index_q_norm"]), pos)
        _, group_keys = FN.qsa_index(ls["idx"], lw["index_q_norm"], lw["index_k_norm"])
        sel = FN.qsa_select(iq, group_keys, pos.tolist(), top=c.top_groups)
        out = FN.qsa_attention(q, ls["k"], ls["v"], gate, sel)
        return F.linear(out.reshape(t, -1), lw["o"])

    def _experts(self, lw, y):
        c = self.cfg
        prob = F.linear(y, lw["router"]).softmax(-1)
        top_p, top_i = prob.topk(c.top_k, dim=-1)
        top_p = top_p / top_p.sum(-1, keepdim=True)
        out = torch.zeros_like(y)
        for slot in range(c.top_k):
            for e in top_i[:, slot].unique().tolist():
                rows = (top_i[:, slot] == e).nonzero().flatten()
                gu = F.linear(y[rows], lw["gate_up"][e])
                act = F.silu(gu[:, :c.expert_ffn]) * gu[:, c.expert_ffn:]
                out[rows] += top_p[rows, slot, None] * F.linear(act, lw["down"][e])
        gu = F.linear(y, lw["shared_gate_up"])
        shared = F.linear(F.silu(gu[:, :c.shared_ffn]) * gu[:, c.shared_ffn:], lw["shared_down"])
        return out + torch.sigmoid(F.linear(y, lw["shared_gate"])) * shared

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, tokens: List[int], state: Optional[FlashNextState] = None):
        """Run ``tokens`` after what ``state`` has committed; returns (logits [T, vocab],
        state).  Any split of a prompt into calls gives the same logits."""
        c = self.cfg
        st = state or FlashNextState()
        first = len(st.tokens)
        t = len(tokens)
        x = self.w["embed"][torch.tensor(tokens)][:, None, :].repeat(1, c.streams, 1)
        ple_slot = 0
        for i, lw in enumerate(self.w["layers"]):
            ls = st.layer.setdefault(i, {})
            if "ple" in lw:
                x, ls["ple_hist"] = FN.ple(x, self._features(st, tokens, ple_slot), lw["ple"],
                                           history=ls.get("ple_hist"))
                ple_slot += 1
            y, gate = FN.hc_read(x, lw["hc_mix"])
            mixed = self._attention(lw, y, ls, first) if c.is_attention(i) else self._gdn(lw, y, ls)
            x = FN.hc_write(x, mixed, gate)
            y, gate = FN.hc_read(x, lw["hc_ffn"])
            x = FN.hc_write(x, self._experts(lw, y), gate)
        final = FN.rms(x.mean(1), self.w["final_norm"], c.eps)
        st.tokens = st.tokens + list(tokens)
        return F.linear(final, self.w["head"]), st

    def generate(self, prompt: List[int], max_new: int, chunk: int = 64) -> List[int]:
        st, logits = None, None
        for lo in range(0, len(prompt), chunk):
            logits, st = self.forward(prompt[lo:lo + chunk], st)
        out = []
        for _ in range(max_new):
            tok = int(logits[-1].argmax())
            out.append(tok)
            logits, st = self.forward([tok], st)
        return out
