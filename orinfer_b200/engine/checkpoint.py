"""Checkpoint I/O of this engine's own model directory, plus dispatch to the reader of
directories published by the reference's quantiser.

Own format: ``model.safetensors`` (one file), ``config.json`` (geometry) and
``cache/model.json`` - the descriptor with the architecture, compute policy, per-tensor
SHA-256 digests and frontend-asset hashes (the role of crates/orinfer-engine/src/loader.rs:16-35).
Tensors are stored already fused and tiled for the kernels, under this engine's own names
(``layers.N.qkv`` ...): ``<name>.packed`` int32 ``[K/128, N, 16]`` + ``<name>.scale`` FP16
``[N]`` for E8P Q4 (the reference's runtime tiling ``e8p-q4-k128-u32``), ``<name>.packed16``
for Q2, ``<name>.int8`` INT8 ``[N, K]`` for W8, ``orinfer.rotation.k{K}.signs`` and
``orinfer.e8p_q4.basis``; the codes themselves are bit-identical to the reference's codec.

A directory written by the reference's quantiser keeps Hugging Face tensor names, one
projection per tensor in row-major ``[N, K/8]`` U32, shards with an index and a separate
``quantization.safetensors`` (python/orinfer_build/quantization/qwen_e8p.py:386-474);
``load_model`` recognises it by its ``quantization_config`` and hands it to
``ref_checkpoint.load_reference_model``.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np
import torch
from safetensors import safe_open
from safetensors.torch import save_file

from ..config import ModelConfig
from ..models.weights import ExpertBank, LayerWeights, ModelWeights, MtpWeights, QLinear
from ..quant import e8p

SCHEMA = 1
QUANT_METADATA = {"quant_method": "orinfer_e8p_q4_int8", "codec": "orinfer-e8p-q4-v1",
                  "coefficients": "4,1", "layout": "u32-low-coarse-high-residual",
                  "rotation": "signed-block128", "scale": "fp16-output-row"}


class CheckpointError(ValueError):
    pass


def _put_linear(out: Dict[str, torch.Tensor], name: str, lin: QLinear) -> None:
    if lin.fmt == "w8" and lin.rowq4 is not None:
        out[f"{name}.rowq4"] = lin.rowq4                 # 4-bit level-table rows, expanded on load
    elif lin.fmt == "w8":
        out[f"{name}.int8"] = lin.codes
    elif lin.fmt == "q4":
        out[f"{name}.packed"] = lin.codes
    else:
        out[f"{name}.packed16"] = lin.codes
    out[f"{name}.scale"] = lin.scale
    if lin.fmt == "w8" and lin.signs is not None:
        out[f"{name}.rotated"] = torch.ones(1, dtype=torch.int8)


def _get_linear(t: Dict[str, torch.Tensor], name: str, signs: Dict[int, torch.Tensor]) -> QLinear:
    scale = t[f"{name}.scale"]
    if f"{name}.rowq4" in t:
        # scalar level-table rows (quant/row_q4.py): the INT8 levels are what the W8 kernels
        # multiply, so the rows are expanded once here
        from ..quant.row_q4 import RowQ4Weight
        packed = t[f"{name}.rowq4"]
        n, k = packed.shape[0], 2 * packed.shape[1]
        if k not in signs:
            raise CheckpointError(f"{name}: no rotation signs for K={k}")
        ints = RowQ4Weight(packed.cpu().numpy(), scale.cpu().numpy(),
                           signs[k].cpu().numpy().astype(np.int8)).integers()
        return QLinear("w8", n, k, torch.from_numpy(ints).to(packed.device), scale, signs[k],
                       None, packed)
    if f"{name}.int8" in t:
        codes = t[f"{name}.int8"]
        n, k = codes.shape
        return QLinear("w8", n, k, codes, scale, signs.get(k) if f"{name}.rotated" in t else None)
    if f"{name}.packed" in t:
        codes = t[f"{name}.packed"]
        fmt = "q4"
    elif f"{name}.packed16" in t:
        codes = t[f"{name}.packed16"]
        fmt = "q2"
    else:
        raise CheckpointError(f"missing tensor for projection {name}")
    kb, n, sixteen = codes.shape
    if sixteen != 16:
        raise CheckpointError(f"{name}: expected [K/128, N, 16] codes")
    k = kb * 128
    if k not in signs:
        raise CheckpointError(f"{name}: no rotation signs for K={k}")
    return QLinear(fmt, n, k, codes, scale, signs[k])


_LAYER_LINEARS = ["qkv", "o", "gdn_qkvz", "gdn_out", "gate_up", "down", "shared_gate_up",
                  "shared_down"]
_LAYER_TENSORS = ["in_norm", "post_norm", "q_norm", "k_norm", "gdn_ab", "gdn_conv", "gdn_a_log",
                  "gdn_dt_bias", "gdn_norm", "router"]


def _layer_tensors(prefix: str, lw: LayerWeights) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for f in _LAYER_TENSORS:
        v = getattr(lw, f)
        if v is not None:
            out[f"{prefix}.{f}"] = v
    for f in _LAYER_LINEARS:
        v = getattr(lw, f)
        if v is not None:
            _put_linear(out, f"{prefix}.{f}", v)
    for f in ("expert_gate_up", "expert_down"):
        bank = getattr(lw, f)
        if bank is not None:
            key = {"w8": "int8", "q4": "packed", "q2": "packed16"}[bank.fmt]
            out[f"{prefix}.{f}.{key}"] = bank.codes
            out[f"{prefix}.{f}.scale"] = bank.scale
    return out


def _load_layer(t, prefix: str, kind: str, signs) -> LayerWeights:
    lw = LayerWeights(kind, t[f"{prefix}.in_norm"], t[f"{prefix}.post_norm"])
    for f in _LAYER_TENSORS[2:]:
        if f"{prefix}.{f}" in t:
            setattr(lw, f, t[f"{prefix}.{f}"])
    for f in _LAYER_LINEARS:
        if f"{prefix}.{f}.scale" in t:
            setattr(lw, f, _get_linear(t, f"{prefix}.{f}", signs))
    for f in ("expert_gate_up", "expert_down"):
        if f"{prefix}.{f}.scale" in t:
            for key, fmt in (("int8", "w8"), ("packed", "q4"), ("packed16", "q2")):
                if f"{prefix}.{f}.{key}" in t:
                    codes = t[f"{prefix}.{f}.{key}"]
                    e = codes.shape[0]
                    if fmt == "w8":
                        n, k = codes.shape[1:]
                    else:
                        n, k = codes.shape[2], codes.shape[1] * 128
                    setattr(lw, f, ExpertBank(fmt, e, n, k, codes, t[f"{prefix}.{f}.scale"],
                                              signs.get(k)))
    return lw


def save_model(weights: ModelWeights, directory, name: Optional[str] = None) -> Path:
    directory = Path(directory)
    (directory / "cache").mkdir(parents=True, exist_ok=True)
    cfg = weights.config
    t: Dict[str, torch.Tensor] = {
        "embed.int8": weights.embed_q, "embed.scale": weights.embed_s,
        "final_norm": weights.final_norm,
        "orinfer.e8p_q4.basis": torch.from_numpy(np.array(e8p.basis())),
    }
    for k, s in weights.signs.items():
        t[f"orinfer.rotation.k{k}.signs"] = s
    if not cfg.tied_embeddings:
        _put_linear(t, "head", weights.head)
    for i, lw in enumerate(weights.layers):
        t.update(_layer_tensors(f"layers.{i}", lw))
    if weights.mtp is not None:
        m = weights.mtp
        t["mtp.norm_e"], t["mtp.norm_h"], t["mtp.final_norm"] = m.norm_e, m.norm_h, m.final_norm
        _put_linear(t, "mtp.fc", m.fc)
        t.update(_layer_tensors("mtp.layer", m.layer))
    t = {k: v.detach().cpu().contiguous() for k, v in t.items()}
    save_file(t, str(directory / "model.safetensors"), metadata=dict(QUANT_METADATA))
    (directory / "config.json").write_text(cfg.to_json())
    digests = {k: hashlib.sha256(v.numpy().tobytes()).hexdigest() for k, v in t.items()}
    assets = {f: hashlib.sha256((directory / f).read_bytes()).hexdigest()
              for f in ("tokenizer.json", "chat_template.jinja", "generation_config.json")
              if (directory / f).exists()}
    descriptor = {"schema": SCHEMA, "architecture": f"orinfer_b200.{cfg.arch}",
                  "name": name or cfg.name, "compute_policy": "int8_quality",
                  "target": "sm_100a", "quantization_config": QUANT_METADATA,
                  "tensors": digests, "frontend_assets": assets,
                  "buffer_scopes": ["Weights", "Sequence", "Workspace"]}
    (directory / "cache" / "model.json").write_text(json.dumps(descriptor, indent=1,
                                                               sort_keys=True))
    return directory


def read_descriptor(directory) -> dict:
    p = Path(directory) / "cache" / "model.json"
    if not p.exists():
        raise CheckpointError(f"{p} is missing")
    d = json.loads(p.read_text())
    if d.get("schema") != SCHEMA:
        raise CheckpointError("unsupported descriptor schema")
    if d.get("target") != "sm_100a":
        raise CheckpointError(f"descriptor target {d.get('target')!r} is not sm_100a")
    return d


def load_model(directory, device="cpu", verify: bool = False,
               workers: Optional[int] = None) -> ModelWeights:
    """Reads the checkpoint with the C++ parallel reader (``workers`` threads, pinned staging
    when the target is a GPU, per-tensor SHA-256 when ``verify``) and uploads it."""
    from .weight_io import WeightReadError, read_tensors
    directory = Path(directory)
    from .ref_checkpoint import is_reference_layout, load_reference_model
    if is_reference_layout(directory):           # published by the reference's own quantiser
        return load_reference_model(directory, device)
    desc = read_descriptor(directory)
    cfg = ModelConfig.from_json((directory / "config.json").read_text())
    from .. import contracts
    try:                                      # architecture -> family, policy and target checks
        contracts.create(desc["architecture"], desc.get("compute_policy", contracts.COMPUTE_POLICY),
                         cfg)
        contracts.parse_target(desc.get("target", contracts.TARGET))
    except contracts.ContractError as e:
        raise CheckpointError(str(e)) from e
    to_gpu = torch.device(device).type == "cuda"
    try:
        t, meta = read_tensors(directory / "model.safetensors", workers=workers, device=device,
                               digests=desc["tensors"] if verify else None)
    except WeightReadError as e:
        raise CheckpointError(str(e)) from e
    for key in ("codec", "layout", "rotation"):
        if meta.get(key) != QUANT_METADATA[key]:
            raise CheckpointError(f"quantisation contract mismatch on {key}")
    if verify and set(desc["tensors"]) - set(t):
        raise CheckpointError(f"tensors missing: {sorted(set(desc['tensors']) - set(t))[:3]}")
    if not np.array_equal(t["orinfer.e8p_q4.basis"].cpu().numpy(), np.array(e8p.basis())):
        raise CheckpointError("E8P basis in the checkpoint differs from the codec's")
    t = {k: v.to(device, non_blocking=to_gpu) for k, v in t.items()}
    if to_gpu:
        torch.cuda.synchronize()
    signs = {int(k.split(".k")[1].split(".")[0]): v for k, v in t.items()
             if k.startswith("orinfer.rotation.")}
    layers = [_load_layer(t, f"layers.{i}", "attn" if cfg.is_full_attention(i) else "gdn", signs)
              for i in range(cfg.layers)]
    if cfg.tied_embeddings:
        head = QLinear("w8", cfg.vocab, cfg.hidden, t["embed.int8"], t["embed.scale"], None)
    else:
        head = _get_linear(t, "head", signs)
    mtp = None
    if "mtp.norm_e" in t:
        mtp = MtpWeights(t["mtp.norm_e"], t["mtp.norm_h"], _get_linear(t, "mtp.fc", signs),
                         _load_layer(t, "mtp.layer", "attn", signs), t["mtp.final_norm"])
    return ModelWeights(cfg, t["embed.int8"], t["embed.scale"], layers, t["final_norm"], head,
                        signs, mtp)


def validate_model(directory) -> dict:
    """CPU-only validation: descriptor, quantisation contract, every tensor digest,
    shapes against the geometry (crates/orinfer-engine/src/model.rs:114-154)."""
    directory = Path(directory)
    desc = read_descriptor(directory)
    weights = load_model(directory, "cpu", verify=True)
    cfg = weights.config
    problems: List[str] = []
    for i, lw in enumerate(weights.layers):
        for f in _LAYER_LINEARS:
            lin = getattr(lw, f)
            if lin is not None and lin.k % 128:
                problems.append(f"layers.{i}.{f}: K={lin.k} is not a multiple of 128")
            if lin is not None and lin.scale.shape[0] != lin.n:
                problems.append(f"layers.{i}.{f}: scale length differs from N")
    for f, digest in desc.get("frontend_assets", {}).items():
        p = directory / f
        if not p.exists() or hashlib.sha256(p.read_bytes()).hexdigest() != digest:
            problems.append(f"frontend asset {f} does not match the descriptor")
    if problems:
        raise CheckpointError("; ".join(problems))
    return {"model": desc["name"], "architecture": desc["architecture"], "layers": cfg.layers,
            "tensors": len(desc["tensors"]), "weight_bytes": weights.nbytes(), "ok": True}
