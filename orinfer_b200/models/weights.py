"""Weight containers and random initialisation in the checkpoint formats.

A projection is stored either as two-stage E8P codes (``q4``: U32
``[K/128, N, 16]`` + FP16 row scale), single-stage codes (``q2``: U16, same
tiling) or plain INT8 rows (``w8``: ``[N, K]`` + FP16 row scale), the layouts
the reference's runtime consumes (python/orinfer_build/models/qwen35/storage.py:38-86;
crates/orinfer-models/src/qwen3_5/rows.rs:343-365).  One rotation sign vector
exists per input width K and is shared by every projection of that width.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from ..config import ModelConfig
from ..quant import e8p


@dataclass
class QLinear:
    fmt: str                          # "q4" | "q2" | "w8"
    n: int
    k: int
    codes: torch.Tensor               # q4: int32 [K/128,N,16]; q2: int16 [K/128,N,16]; w8: int8 [N,K]
    scale: torch.Tensor               # fp16 [N]
    signs: Optional[torch.Tensor]     # int8 [K] when the input is rotated
    dense: Optional[torch.Tensor] = None   # original fp32 weights (kept for tiny models only)
    # uint8 [N, K/2]: the scalar level-table nibbles these W8 codes were expanded from
    # (quant/row_q4.py); a checkpoint then stores the nibbles, 4 bits per weight, not the codes
    rowq4: Optional[torch.Tensor] = None

    def integers(self) -> torch.Tensor:
        """INT8 [N, K] integer weights in the (rotated) basis the GEMM multiplies."""
        if self.fmt == "w8":
            return self.codes
        c = self.codes.cpu().numpy()
        if self.fmt == "q4":
            rows = c.view(np.uint32).transpose(1, 0, 2).reshape(self.n, self.k // 8)
            return torch.from_numpy(e8p.decode_q4(rows)).to(self.codes.device)
        rows = c.view(np.uint16).transpose(1, 0, 2).reshape(self.n, self.k // 8)
        return torch.from_numpy(e8p.decode_q2(rows)).to(self.codes.device)

    def to(self, device) -> "QLinear":
        mv = lambda t: None if t is None else t.to(device)
        return QLinear(self.fmt, self.n, self.k, mv(self.codes), mv(self.scale), mv(self.signs),
                       self.dense, self.rowq4)

    def nbytes(self) -> int:
        return self.codes.numel() * self.codes.element_size() + self.scale.numel() * 2


def quantize_linear(weight: torch.Tensor, fmt: str, signs: Optional[torch.Tensor],
                    keep_dense: bool = False, fast: bool = True) -> QLinear:
    """Quantise fp32 ``[N, K]`` weights.  CUDA tensors use the device encoder
    (one pass, rms-derived scale); CPU tensors use the exhaustive numpy fit."""
    n, k = weight.shape
    dense = weight.detach().float().cpu() if keep_dense else None
    if fmt == "w8":
        w = weight.float()
        if signs is not None:
            from ..ref.ops_ref import hadamard_rotate
            w = hadamard_rotate(w, signs.to(w.device))
        amax = w.abs().amax(1)
        scale = torch.where(amax > 0, torch.clamp(amax / 127.0, min=2.0 ** -24),
                            torch.ones_like(amax)).to(torch.float16)
        q = torch.clamp(torch.round(w / scale.float()[:, None]), -127, 127).to(torch.int8)
        return QLinear("w8", n, k, q.contiguous(), scale, signs, dense)
    if signs is None:
        raise ValueError("E8P formats need rotation signs")
    from ..quant import e8p_torch
    if weight.is_cuda:
        from ..ops import quantize as devq
        if devq.available():
            codes, scale = devq.encode_e8p(weight, signs, fmt, refine=0 if fast else 1)
            return QLinear(fmt, n, k, codes, scale, signs, dense)
    if fmt == "q4":
        codes, scale = e8p_torch.fit_q4_t(weight, signs, refine=0 if fast else 2)
    elif fmt == "q2":
        codes, scale = e8p_torch.fit_q2_t(weight, signs, refine=1 if fast else 2)
    else:
        raise ValueError(f"unknown format {fmt}")
    return QLinear(fmt, n, k, codes, scale, signs, dense)


@dataclass
class ExpertBank:
    """Stacked expert projections: codes carry a leading expert axis."""
    fmt: str
    experts: int
    n: int
    k: int
    codes: torch.Tensor               # [E, K/128, N, 16] (q4 int32 / q2 int16) or [E, N, K] int8
    scale: torch.Tensor               # fp16 [E, N]
    signs: Optional[torch.Tensor]
    dense: Optional[torch.Tensor] = None
    base: int = 0                     # global id of local expert 0 (expert parallelism)

    def expert(self, e: int) -> QLinear:
        """Projection of GLOBAL expert ``e`` (must be one of this bank's experts)."""
        e -= self.base
        return QLinear(self.fmt, self.n, self.k, self.codes[e], self.scale[e], self.signs,
                       None if self.dense is None else self.dense[e])

    def owns(self, e: int) -> bool:
        return self.base <= e < self.base + self.experts

    def to(self, device) -> "ExpertBank":
        mv = lambda t: None if t is None else t.to(device)
        return ExpertBank(self.fmt, self.experts, self.n, self.k, mv(self.codes), mv(self.scale),
                          mv(self.signs), self.dense, self.base)


@dataclass
class LayerWeights:
    kind: str                                     # "attn" | "gdn"
    in_norm: torch.Tensor
    post_norm: torch.Tensor
    # attention
    qkv: Optional[QLinear] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    o: Optional[QLinear] = None
    # gated delta rule
    gdn_qkvz: Optional[QLinear] = None            # rows: q | k | v | z
    gdn_ab: Optional[torch.Tensor] = None         # fp16 [2*HV, H]
    gdn_conv: Optional[torch.Tensor] = None       # fp16 [conv_dim, 4]
    gdn_a_log: Optional[torch.Tensor] = None      # fp32 [HV]
    gdn_dt_bias: Optional[torch.Tensor] = None    # fp32 [HV]
    gdn_norm: Optional[torch.Tensor] = None       # fp16 [head_dim]
    gdn_out: Optional[QLinear] = None
    # dense FFN
    gate_up: Optional[QLinear] = None
    down: Optional[QLinear] = None
    # MoE FFN
    router: Optional[torch.Tensor] = None         # fp16 [E(+1 shared gate), H]
    expert_gate_up: Optional[ExpertBank] = None
    expert_down: Optional[ExpertBank] = None
    shared_gate_up: Optional[QLinear] = None
    shared_down: Optional[QLinear] = None
    shared_owner: int = -1                        # rank adding the shared expert (-1: every rank)

    def to(self, device) -> "LayerWeights":
        out = {}
        for name, val in self.__dict__.items():
            out[name] = val.to(device) if hasattr(val, "to") and not isinstance(val, str) else val
        return LayerWeights(**out)


@dataclass
class ModelWeights:
    config: ModelConfig
    embed_q: torch.Tensor             # int8 [V, H]
    embed_s: torch.Tensor             # fp16 [V]
    layers: List[LayerWeights]
    final_norm: torch.Tensor
    head: QLinear
    signs: Dict[int, torch.Tensor] = field(default_factory=dict)
    mtp: Optional["MtpWeights"] = None
    embed_dense: Optional[torch.Tensor] = None

    def to(self, device) -> "ModelWeights":
        return ModelWeights(self.config, self.embed_q.to(device), self.embed_s.to(device),
                            [l.to(device) for l in self.layers], self.final_norm.to(device),
                            self.head.to(device), {k: v.to(device) for k, v in self.signs.items()},
                            None if self.mtp is None else self.mtp.to(device), self.embed_dense)

    def nbytes(self) -> int:
        total = self.embed_q.numel()
        for l in self.layers:
            for v in l.__dict__.values():
                if isinstance(v, QLinear):
                    total += v.nbytes()
                elif isinstance(v, ExpertBank):
                    total += v.codes.numel() * v.codes.element_size()
        return total


@dataclass
class MtpWeights:
    """Draft head: concat(norm_e(embed), norm_h(hidden)) -> fc -> one decoder layer -> shared head
    (kernels/cuda/model/speculation.py:31 mtp_norm_concat)."""
    norm_e: torch.Tensor
    norm_h: torch.Tensor
    fc: QLinear                       # [H, 2H] w8
    layer: LayerWeights
    final_norm: torch.Tensor

    def to(self, device) -> "MtpWeights":
        return MtpWeights(self.norm_e.to(device), self.norm_h.to(device), self.fc.to(device),
                          self.layer.to(device), self.final_norm.to(device))


class _Init:
    def __init__(self, cfg: ModelConfig, seed: int, device, keep_dense: bool):
        self.cfg, self.device, self.keep = cfg, torch.device(device), keep_dense
        self.gen = torch.Generator(device=self.device)
        self.gen.manual_seed(seed)
        self.signs: Dict[int, torch.Tensor] = {}

    def sign(self, k: int) -> torch.Tensor:
        if k not in self.signs:
            self.signs[k] = torch.from_numpy(e8p.random_signs(k, seed=k)).to(self.device)
        return self.signs[k]

    def normal(self, *shape) -> torch.Tensor:
        return torch.randn(*shape, generator=self.gen, device=self.device,
                           dtype=torch.float32) * 0.02

    def linear(self, n: int, k: int, fmt: str, rotate: bool = True) -> QLinear:
        signs = self.sign(k) if (rotate or fmt != "w8") else None
        return quantize_linear(self.normal(n, k), fmt, signs, self.keep)

    def bank(self, e: int, n: int, k: int, fmt: str) -> ExpertBank:
        parts = [self.linear(n, k, fmt) for _ in range(e)]
        dense = torch.stack([p.dense for p in parts]) if self.keep else None
        return ExpertBank(fmt, e, n, k, torch.stack([p.codes for p in parts]),
                          torch.stack([p.scale for p in parts]), self.sign(k), dense)

    def ones(self, n: int) -> torch.Tensor:
        return torch.ones(n, dtype=torch.float16, device=self.device)

    def layer(self, index: int, full_attention: bool) -> LayerWeights:
        c = self.cfg
        lw = LayerWeights("attn" if full_attention else "gdn", self.ones(c.hidden),
                          self.ones(c.hidden))
        if full_attention:
            lw.qkv = self.linear(c.q_dim + 2 * c.kv_dim, c.hidden, c.attn_format)
            lw.q_norm, lw.k_norm = self.ones(c.head_dim), self.ones(c.head_dim)
            lw.o = self.linear(c.hidden, c.q_heads * c.head_dim, c.attn_format)
        else:
            dk, dv = c.gdn_k_heads * c.gdn_head_dim, c.gdn_v_heads * c.gdn_head_dim
            lw.gdn_qkvz = self.linear(2 * dk + 2 * dv, c.hidden, c.attn_format)
            lw.gdn_ab = self.normal(2 * c.gdn_v_heads, c.hidden).to(torch.float16)
            lw.gdn_conv = (torch.randn(2 * dk + dv, c.gdn_conv, generator=self.gen,
                                       device=self.device) * 0.3).to(torch.float16)
            lw.gdn_a_log = torch.zeros(c.gdn_v_heads, device=self.device)
            lw.gdn_dt_bias = torch.zeros(c.gdn_v_heads, device=self.device)
            lw.gdn_norm = self.ones(c.gdn_head_dim)
            lw.gdn_out = self.linear(c.hidden, dv, c.attn_format)
        if c.experts:
            rows = c.experts + (1 if c.shared_expert_ffn else 0)
            lw.router = self.normal(rows, c.hidden).to(torch.float16)
            lw.expert_gate_up = self.bank(c.experts, 2 * c.expert_ffn, c.hidden, c.expert_format)
            lw.expert_down = self.bank(c.experts, c.hidden, c.expert_ffn, c.expert_format)
            if c.shared_expert_ffn:
                lw.shared_gate_up = self.linear(2 * c.shared_expert_ffn, c.hidden, c.proj_format)
                lw.shared_down = self.linear(c.hidden, c.shared_expert_ffn, c.proj_format)
        else:
            lw.gate_up = self.linear(2 * c.ffn, c.hidden, c.proj_format)
            lw.down = self.linear(c.hidden, c.ffn, c.proj_format)
        return lw


def random_model(cfg: ModelConfig, seed: int = 0, device="cpu",
                 keep_dense: bool = False) -> ModelWeights:
    """Random-init N(0, 0.02) weights quantised to the configured formats."""
    init = _Init(cfg, seed, device, keep_dense)
    emb = init.normal(cfg.vocab, cfg.hidden)
    emb_l = quantize_linear(emb, "w8", None, keep_dense)
    layers = [init.layer(i, cfg.is_full_attention(i)) for i in range(cfg.layers)]
    if cfg.tied_embeddings:
        head = QLinear("w8", cfg.vocab, cfg.hidden, emb_l.codes, emb_l.scale, None, emb_l.dense)
    else:
        head = init.linear(cfg.vocab, cfg.hidden, cfg.head_format, rotate=False)
    mtp = None
    if cfg.mtp_layers:
        mtp = MtpWeights(init.ones(cfg.hidden), init.ones(cfg.hidden),
                         init.linear(cfg.hidden, 2 * cfg.hidden, "w8", rotate=False),
                         _mtp_layer(init), init.ones(cfg.hidden))
    return ModelWeights(cfg, emb_l.codes, emb_l.scale, layers, init.ones(cfg.hidden), head,
                        init.signs, mtp, emb_l.dense)


def _mtp_layer(init: _Init) -> LayerWeights:
    """The draft layer is a dense full-attention decoder layer in W8
    (python/orinfer_build/models/qwen35/mtp.py: one W8 layer + shared head)."""
    c = init.cfg
    if c.draft_layer == "model":           # a full-attention layer shaped like the model's own
        return init.layer(c.layers, True)
    lw = LayerWeights("attn", init.ones(c.hidden), init.ones(c.hidden))
    qd = c.q_heads * c.head_dim
    lw.qkv = init.linear(qd + 2 * c.kv_dim, c.hidden, "w8", rotate=False)
    lw.q_norm, lw.k_norm = init.ones(c.head_dim), init.ones(c.head_dim)
    lw.o = init.linear(c.hidden, qd, "w8", rotate=False)
    f = c.ffn or max(c.expert_ffn * 4, 512)
    lw.gate_up = init.linear(2 * f, c.hidden, "w8", rotate=False)
    lw.down = init.linear(c.hidden, f, "w8", rotate=False)
    return lw
