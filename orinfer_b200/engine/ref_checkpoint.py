"""Reader for quantised checkpoints in the layout the reference's toolchain publishes.

Such a directory keeps the Hugging Face tensor names and shards and replaces every
quantised projection ``<name>`` by

* ``<name>.packed``  U32 ``[N, K/8]`` (``orin.layout.* = e8p-q4-row-u32``: coarse code in the
  low half-word, residual in the high one) or ``<name>.int8`` I8 ``[N, K]``, and
* ``<name>.scale``   F16 ``[N]``;

``model.safetensors.index.json`` maps tensors to shards, ``quantization.safetensors`` holds
one rotation sign vector per input width (``orinfer.rotation.k<K>.signs``) and the lattice
basis, and ``config.json`` carries ``quantization_config`` (``orinfer_e8p_q4_int8``,
coefficients ``[4, 1]``, ``signed-block128`` rotation)
(python/orinfer_build/quantization/qwen_e8p.py:386-474).  Projections are stored one by one;
the runtime fuses q|k|v and gate|up by concatenating rows, which is exact because scales
are per output row, and turns ``[N, K/8]`` rows into the k-block-major tiling the kernels
stream (``[K/128, N, 16]``), the same re-tiling the reference's own runtime build does
(python/orinfer_build/models/qwen35/storage.py:38-86).

Covered: the text decoder of dense, mixture-of-experts and hybrid (gated-delta-rule)
Qwen-style models.  A lattice-coded embedding table is decoded, rotated back and kept as
W8 rows for the gather kernel (the tied head keeps the lattice codes); vision / audio
towers and draft heads of such a checkpoint are not read.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional

import torch
from safetensors import safe_open

from ..config import ModelConfig
from ..models.weights import ExpertBank, LayerWeights, ModelWeights, QLinear, quantize_linear
from ..quant import e8p
from ..quant.convert import config_from_hf, rotary_permutation
from .checkpoint import CheckpointError

METHOD = "orinfer_e8p_q4_int8"
ROW_LAYOUT = "e8p-q4-row-u32"
PREFIXES = ("model.language_model.", "language_model.", "model.")


def is_reference_layout(directory) -> bool:
    cfg = Path(directory) / "config.json"
    if not cfg.exists():
        return False
    try:
        q = json.loads(cfg.read_text()).get("quantization_config") or {}
    except ValueError:
        return False
    return q.get("quant_method") == METHOD


class _Shards:
    """Name -> tensor through ``model.safetensors.index.json`` (or every shard found)."""

    def __init__(self, directory: Path):
        self.dir = directory
        index = directory / "model.safetensors.index.json"
        self.where: Dict[str, str] = {}
        if index.exists():
            self.where = dict(json.loads(index.read_text())["weight_map"])
        else:
            for f in sorted(directory.glob("*.safetensors")):
                with safe_open(str(f), "pt") as h:
                    for k in h.keys():
                        self.where.setdefault(k, f.name)
        self.layouts: Dict[str, str] = {}
        for f in sorted(set(self.where.values())):
            with safe_open(str(directory / f), "pt") as h:
                for k, v in (h.metadata() or {}).items():
                    if k.startswith("orin.layout."):
                        self.layouts[k[len("orin.layout."):]] = v

    def has(self, name: str) -> bool:
        return name in self.where

    def get(self, name: str) -> torch.Tensor:
        f = self.where.get(name)
        if f is None:
            raise CheckpointError(f"tensor `{name}` is missing from the checkpoint")
        with safe_open(str(self.dir / f), "pt") as h:
            return h.get_tensor(name)


def _retile(rows_u32: torch.Tensor) -> torch.Tensor:
    """U32 [N, K/8] row codes -> int32 [K/128, N, 16] k-block-major tiling."""
    n, words = rows_u32.shape
    if words % 16:
        raise CheckpointError("packed rows must cover whole 128-channel blocks")
    t = rows_u32.view(torch.int32).reshape(n, words // 16, 16).permute(1, 0, 2)
    return t.contiguous()


class _Reader:
    def __init__(self, directory: Path):
        self.src = _Shards(directory)
        self.signs: Dict[int, torch.Tensor] = {}
        qpath = directory / "quantization.safetensors"
        if not qpath.exists():
            raise CheckpointError("quantization.safetensors is missing")
        with safe_open(str(qpath), "pt") as h:
            for key in h.keys():
                if key.startswith("orinfer.rotation.k") and key.endswith(".signs"):
                    k = int(key[len("orinfer.rotation.k"):-len(".signs")])
                    self.signs[k] = h.get_tensor(key).to(torch.int8).contiguous()
                elif key == "orinfer.e8p_q4.basis":
                    basis = h.get_tensor(key).to(torch.int8)
                    if not torch.equal(basis, torch.from_numpy(e8p.basis().copy())):
                        raise CheckpointError("the checkpoint's lattice basis differs from "
                                              "the one the kernels decode")
        self.prefix = next((p for p in PREFIXES
                            if self.src.has(p + "norm.weight")
                            or self.src.has(p + "embed_tokens.weight")
                            or self.src.has(p + "embed_tokens.weight.packed")), None)
        if self.prefix is None:
            raise CheckpointError("cannot find the text decoder's tensors")

    def sign(self, k: int) -> torch.Tensor:
        if k not in self.signs:
            raise CheckpointError(f"no rotation signs for input width {k}")
        return self.signs[k]

    def plain(self, name: str) -> torch.Tensor:
        return self.src.get(name).float()

    def f16(self, name: str, index: Optional[torch.Tensor] = None) -> torch.Tensor:
        t = self.plain(name)
        if index is not None:
            t = t[index]
        return t.to(torch.float16).contiguous()

    def rows(self, name: str):
        """One stored projection as (format, row-major codes [N, ...], scales [N])."""
        if self.src.has(name + ".packed"):
            lay = self.src.layouts.get(name + ".packed", ROW_LAYOUT)
            if lay != ROW_LAYOUT:
                raise CheckpointError(f"{name}.packed has layout {lay}, expected {ROW_LAYOUT}")
            codes = self.src.get(name + ".packed")
            if codes.dtype not in (torch.uint32, torch.int32):
                raise CheckpointError(f"{name}.packed must be U32")
            return "q4", codes.view(torch.int32), self.src.get(name + ".scale").to(torch.float16)
        if self.src.has(name + ".int8"):
            return "w8", self.src.get(name + ".int8").to(torch.int8), \
                self.src.get(name + ".scale").to(torch.float16)
        raise CheckpointError(f"projection `{name}` is neither packed nor int8 in the checkpoint")

    def linear(self, names: List[str], perms: Optional[List[Optional[torch.Tensor]]] = None,
               rotated_w8: bool = False) -> QLinear:
        """Row concatenation of stored projections (optionally with their rows reordered)."""
        fmts, codes, scales = [], [], []
        for i, name in enumerate(names):
            fmt, c, s = self.rows(name)
            if perms is not None and perms[i] is not None:
                c, s = c.index_select(0, perms[i]), s.index_select(0, perms[i])
            fmts.append(fmt)
            codes.append(c)
            scales.append(s)
        if len(set(fmts)) != 1:
            raise CheckpointError(f"{names} mix weight formats and cannot be fused")
        rows, scale = torch.cat(codes), torch.cat(scales).contiguous()
        n = rows.shape[0]
        if fmts[0] == "q4":
            k = rows.shape[1] * 8
            return QLinear("q4", n, k, _retile(rows), scale, self.sign(k))
        k = rows.shape[1]
        return QLinear("w8", n, k, rows.contiguous(), scale, self.sign(k) if rotated_w8 else None)


def load_reference_model(directory, device="cpu", name: Optional[str] = None) -> ModelWeights:
    """Loads the text decoder of a checkpoint in the reference's published layout."""
    directory = Path(directory)
    hf = json.loads((directory / "config.json").read_text())
    q = hf.get("quantization_config") or {}
    if q.get("quant_method") != METHOD:
        raise CheckpointError("not a checkpoint of the reference's quantiser")
    if list(q.get("coefficients", [4, 1])) != [4, 1] or \
            q.get("rotation", "signed-block128") != "signed-block128" or \
            q.get("layout", "u32-low-coarse-high-residual") != "u32-low-coarse-high-residual":
        raise CheckpointError("unsupported codec parameters in quantization_config")
    text = dict(hf.get("text_config") or hf)
    text.setdefault("architectures", hf.get("architectures", []))
    text.setdefault("model_type", hf.get("model_type", ""))
    cfg: ModelConfig = config_from_hf(text, name or directory.name)
    protected = set(q.get("rotated_w8_layers") or [])
    rd = _Reader(directory)
    P = rd.prefix
    layers: List[LayerWeights] = []
    d = cfg.head_dim
    perm = rotary_permutation(cfg.head_dim, cfg.rotary_dim)
    for i in range(cfg.layers):
        p = f"{P}layers.{i}."
        rot = i in protected
        full = cfg.is_full_attention(i)
        lw = LayerWeights("attn" if full else "gdn", rd.f16(p + "input_layernorm.weight"),
                          rd.f16(p + "post_attention_layernorm.weight"))
        if full:
            qh, kvh = cfg.q_heads, cfg.kv_heads
            head = torch.arange(d)
            if cfg.gated_attention:                # per head: d query rows, then d gate rows
                q_idx = torch.cat([torch.cat([h * 2 * d + perm, h * 2 * d + d + head])
                                   for h in range(qh)])
            else:
                q_idx = torch.cat([h * d + perm for h in range(qh)])
            k_idx = torch.cat([h * d + perm for h in range(kvh)])
            lw.qkv = rd.linear([p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight",
                                p + "self_attn.v_proj.weight"], [q_idx, k_idx, None], rot)
            if cfg.qk_norm:
                lw.q_norm = rd.f16(p + "self_attn.q_norm.weight", perm)
                lw.k_norm = rd.f16(p + "self_attn.k_norm.weight", perm)
            lw.o = rd.linear([p + "self_attn.o_proj.weight"], None, rot)
        else:
            hk, hv, gd = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
            rep = hv // hk
            per = 2 * gd + 2 * rep * gd            # source rows per key head: q | k | v.. | z..
            ar = torch.arange
            idx = torch.cat(
                [torch.cat([h * per + ar(0, gd) for h in range(hk)]),
                 torch.cat([h * per + ar(gd, 2 * gd) for h in range(hk)]),
                 torch.cat([h * per + ar(2 * gd, 2 * gd + rep * gd) for h in range(hk)]),
                 torch.cat([h * per + ar(2 * gd + rep * gd, per) for h in range(hk)])])
            lw.gdn_qkvz = rd.linear([p + "linear_attn.in_proj_qkvz.weight"], [idx], rot)
            ba = rd.plain(p + "linear_attn.in_proj_ba.weight").reshape(hk, 2 * rep, -1)
            lw.gdn_ab = torch.cat([ba[:, rep:].reshape(hv, -1),
                                   ba[:, :rep].reshape(hv, -1)]).to(torch.float16).contiguous()
            lw.gdn_conv = rd.plain(p + "linear_attn.conv1d.weight")[:, 0, :] \
                .to(torch.float16).contiguous()
            lw.gdn_a_log = rd.plain(p + "linear_attn.A_log").contiguous()
            lw.gdn_dt_bias = rd.plain(p + "linear_attn.dt_bias").contiguous()
            lw.gdn_norm = rd.f16(p + "linear_attn.norm.weight")
            lw.gdn_out = rd.linear([p + "linear_attn.out_proj.weight"], None, rot)
        if cfg.experts:
            router = rd.plain(p + "mlp.gate.weight")
            if cfg.shared_expert_ffn:
                router = torch.cat([router, rd.plain(p + "mlp.shared_expert_gate.weight")])
                lw.shared_gate_up = rd.linear([p + "mlp.shared_expert.gate_proj.weight",
                                               p + "mlp.shared_expert.up_proj.weight"], None, rot)
                lw.shared_down = rd.linear([p + "mlp.shared_expert.down_proj.weight"], None, rot)
            lw.router = router.to(torch.float16).contiguous()
            lw.expert_gate_up = _bank(rd, p + "mlp.experts.gate_up_proj", cfg.experts)
            lw.expert_down = _bank(rd, p + "mlp.experts.down_proj", cfg.experts)
        else:
            lw.gate_up = rd.linear([p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"], None,
                                   rot)
            lw.down = rd.linear([p + "mlp.down_proj.weight"], None, rot)
        layers.append(lw)
    emb_name = P + "embed_tokens.weight"
    head: Optional[QLinear] = None
    if rd.src.has(emb_name + ".packed"):
        coded = rd.linear([emb_name])              # lattice-coded table, rotated input basis
        from ..ref.ops_ref import hadamard_rotate
        ints = coded.integers().float() * coded.scale.float()[:, None]
        dense = hadamard_rotate(ints, coded.signs)   # the signed block transform is its own inverse
        emb = quantize_linear(dense, "w8", None)
        if cfg.tied_embeddings:
            head = coded
    else:
        emb = quantize_linear(rd.plain(emb_name), "w8", None)
    if head is None:
        if cfg.tied_embeddings:
            head = QLinear("w8", cfg.vocab, cfg.hidden, emb.codes, emb.scale, None)
        elif rd.src.has("lm_head.weight.packed") or rd.src.has("lm_head.weight.int8"):
            head = rd.linear(["lm_head.weight"])
        else:
            head = quantize_linear(rd.plain("lm_head.weight"), cfg.head_format, None)
    weights = ModelWeights(cfg, emb.codes, emb.scale, layers, rd.f16(P + "norm.weight"), head,
                           dict(rd.signs))
    return weights.to(device)


def _bank(rd: _Reader, name: str, experts: int) -> ExpertBank:
    """Stacked expert projections stored as one 3-D tensor ``[E, N, K/8]`` (+ ``[E, N]``)."""
    fmt, codes, scale = rd.rows(name)
    if codes.dim() != 3 or codes.shape[0] != experts:
        raise CheckpointError(f"{name}: expected a bank of {experts} experts")
    n = codes.shape[1]
    if fmt == "q4":
        k = codes.shape[2] * 8
        tiled = torch.stack([_retile(codes[e]) for e in range(experts)])
        return ExpertBank("q4", experts, n, k, tiled, scale.contiguous(), rd.sign(k))
    k = codes.shape[2]
    return ExpertBank("w8", experts, n, k, codes.contiguous(), scale.contiguous(), None)
