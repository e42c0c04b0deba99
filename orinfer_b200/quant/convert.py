"""Convert a Hugging Face Qwen3-style checkpoint (dense or MoE, bf16 / fp16 / fp32 safetensors)
into this engine's quantised model directory.

Projections are fused the way the runner multiplies them (``q|k|v`` rows, ``gate|up`` rows),
rotated by the signed block-128 Hadamard transform and quantised to the configured formats
(two-stage E8P Q4 by default, W8 for embeddings and the head); norms, the router and the
tokenizer assets are carried over.  The job is resumable: every finished layer is written to
its own file under ``<output>/.convert`` and recorded in ``progress.json`` (with the identity
of the source, so a different source never resumes someone else's work); a rerun skips what is
recorded and intact.  The final step assembles ``model.safetensors``, ``config.json`` and
``cache/model.json``.  Counterpart of the reference's offline converter
(python/orinfer_build/quantization/qwen_e8p.py:1-7: per-shard resumable jobs with
``progress.json``; models/qwen35/storage.py:38-86: K-major repack of fused projections).

    python -m orinfer_b200.quant.convert /path/to/Qwen3-4B /path/to/out --device cuda
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
from pathlib import Path
from typing import Callable, Dict, List, Optional

import torch
from safetensors import safe_open
from safetensors.torch import load_file, save_file

from ..config import ModelConfig
from ..models.weights import ExpertBank, LayerWeights, ModelWeights, QLinear, quantize_linear
from . import e8p

ASSETS = ("tokenizer.json", "tokenizer_config.json", "chat_template.jinja",
          "generation_config.json", "vocab.json", "merges.txt")


class ConvertError(ValueError):
    pass


def config_from_hf(hf: dict, name: Optional[str] = None) -> ModelConfig:
    arch = (hf.get("architectures") or [""])[0]
    if arch not in ("Qwen3ForCausalLM", "Qwen3MoeForCausalLM"):
        raise ConvertError(f"unsupported architecture `{arch}` (Qwen3 dense and MoE are converted)")
    if hf.get("attention_bias"):
        raise ConvertError("attention projections with bias are not supported")
    heads = hf["num_attention_heads"]
    # older configs carry `rope_theta` (+ `rope_scaling`), newer ones a `rope_parameters` object
    rope = dict(hf.get("rope_parameters") or hf.get("rope_scaling") or {})
    kind = rope.get("rope_type") or rope.get("type") or "default"
    if kind != "default":
        raise ConvertError(f"rotary scaling `{kind}` is not supported (plain RoPE only)")
    theta = hf.get("rope_theta") or rope.get("rope_theta") or 1e6
    common = dict(
        name=name or hf.get("_name_or_path") or arch, layers=hf["num_hidden_layers"],
        hidden=hf["hidden_size"], q_heads=heads, kv_heads=hf.get("num_key_value_heads", heads),
        head_dim=hf.get("head_dim") or hf["hidden_size"] // heads, vocab=hf["vocab_size"],
        eps=hf.get("rms_norm_eps", 1e-6), rope_theta=float(theta),
        tied_embeddings=bool(hf.get("tie_word_embeddings", False)),
        max_context=int(hf.get("max_position_embeddings", 32768)))
    if arch == "Qwen3MoeForCausalLM":
        if hf.get("mlp_only_layers") or hf.get("decoder_sparse_step", 1) != 1:
            raise ConvertError("mixed dense / sparse layer stacks are not supported")
        experts = hf.get("num_experts") or hf.get("num_local_experts")
        if not experts:
            raise ConvertError("the configuration does not say how many experts there are")
        return ModelConfig(arch="moe", ffn=0, experts=experts,
                           top_k=hf["num_experts_per_tok"], expert_ffn=hf["moe_intermediate_size"],
                           renormalize=bool(hf.get("norm_topk_prob", True)), **common)
    return ModelConfig(arch="dense", ffn=hf["intermediate_size"], **common)


class _Source:
    """Name -> tensor over all safetensors shards of a directory, opened lazily."""

    def __init__(self, directory: Path):
        self.files = sorted(directory.glob("*.safetensors"))
        if not self.files:
            raise ConvertError(f"no safetensors files in {directory}")
        self.where: Dict[str, Path] = {}
        for f in self.files:
            with safe_open(str(f), "pt") as h:
                for k in h.keys():
                    self.where[k] = f

    def identity(self, config_text: str) -> str:
        h = hashlib.sha256(config_text.encode())
        for f in self.files:
            h.update(f"{f.name}:{f.stat().st_size}".encode())
        return h.hexdigest()

    def get(self, name: str) -> torch.Tensor:
        f = self.where.get(name)
        if f is None:
            raise ConvertError(f"tensor `{name}` is missing from the source checkpoint")
        with safe_open(str(f), "pt") as h:
            return h.get_tensor(name).float()


def _atomic_json(path: Path, obj) -> None:
    tmp = path.with_suffix(path.suffix + ".tmp")
    tmp.write_text(json.dumps(obj, indent=1))
    os.replace(tmp, path)


def convert(source, output, device: str = "cpu", fast: bool = True, name: Optional[str] = None,
            on_layer: Optional[Callable[[int, bool], None]] = None,
            formats: Optional[Dict[str, str]] = None) -> Path:
    """Returns the model directory.  ``on_layer(i, resumed)`` is called after layer ``i`` is on
    disk (freshly quantised or found in the progress record).  ``formats`` overrides the
    weight formats of the geometry (``attn_format``, ``proj_format``, ``expert_format``,
    ``head_format``: ``q4`` | ``q2`` | ``w8``)."""
    from ..engine.checkpoint import _layer_tensors, _load_layer, save_model
    source, output = Path(source), Path(output)
    config_text = (source / "config.json").read_text()
    cfg = config_from_hf(json.loads(config_text), name)
    if formats:
        import dataclasses
        unknown = set(formats) - {"attn_format", "proj_format", "expert_format", "head_format"}
        if unknown or any(v not in ("q4", "q2", "w8") for v in formats.values()):
            raise ConvertError("formats maps attn / proj / expert / head_format to q4, q2 or w8")
        cfg = dataclasses.replace(cfg, **formats)
    src = _Source(source)
    work = output / ".convert"
    work.mkdir(parents=True, exist_ok=True)
    identity = src.identity(config_text + f"|{cfg.attn_format}|{cfg.proj_format}"
                            f"|{cfg.expert_format}|{cfg.head_format}|{fast}")
    record_path = work / "progress.json"
    record = {"source": identity, "done": {}}
    if record_path.exists():
        old = json.loads(record_path.read_text())
        if old.get("source") == identity:
            record = old
    dev = torch.device(device)
    signs: Dict[int, torch.Tensor] = {}

    def sign(k: int) -> torch.Tensor:
        if k not in signs:
            signs[k] = torch.from_numpy(e8p.random_signs(k, seed=k))
        return signs[k]

    def lin(weight: torch.Tensor, fmt: str) -> QLinear:
        s = sign(weight.shape[1])
        q = quantize_linear(weight.to(dev), fmt, s.to(dev), fast=fast)
        return QLinear(q.fmt, q.n, q.k, q.codes.cpu(), q.scale.cpu(), s)

    def f16(t: torch.Tensor) -> torch.Tensor:
        return t.to(torch.float16).contiguous()

    for i in range(cfg.layers):
        key, path = f"layer.{i}", work / f"layer_{i:05d}.safetensors"
        done = record["done"].get(key)
        if done and path.exists() and path.stat().st_size == done:
            if on_layer:
                on_layer(i, True)
            continue
        p = f"model.layers.{i}."
        lw = LayerWeights("attn", f16(src.get(p + "input_layernorm.weight")),
                          f16(src.get(p + "post_attention_layernorm.weight")))
        lw.qkv = lin(torch.cat([src.get(p + f"self_attn.{x}_proj.weight") for x in "qkv"]),
                     cfg.attn_format)
        lw.q_norm = f16(src.get(p + "self_attn.q_norm.weight"))
        lw.k_norm = f16(src.get(p + "self_attn.k_norm.weight"))
        lw.o = lin(src.get(p + "self_attn.o_proj.weight"), cfg.attn_format)
        if cfg.experts:
            lw.router = f16(src.get(p + "mlp.gate.weight"))
            gu, dn = [], []
            fused = p + "mlp.experts.gate_up_proj" in src.where     # [E, 2F, H] / [E, H, F]
            if fused:
                all_gu, all_dn = src.get(p + "mlp.experts.gate_up_proj"), \
                    src.get(p + "mlp.experts.down_proj")
            for e in range(cfg.experts):
                q = p + f"mlp.experts.{e}."
                if fused:
                    gu.append(lin(all_gu[e], cfg.expert_format))
                    dn.append(lin(all_dn[e], cfg.expert_format))
                    continue
                gu.append(lin(torch.cat([src.get(q + "gate_proj.weight"),
                                         src.get(q + "up_proj.weight")]), cfg.expert_format))
                dn.append(lin(src.get(q + "down_proj.weight"), cfg.expert_format))
            for bank_name, parts in (("expert_gate_up", gu), ("expert_down", dn)):
                setattr(lw, bank_name, ExpertBank(
                    parts[0].fmt, cfg.experts, parts[0].n, parts[0].k,
                    torch.stack([x.codes for x in parts]), torch.stack([x.scale for x in parts]),
                    parts[0].signs))
        else:
            lw.gate_up = lin(torch.cat([src.get(p + "mlp.gate_proj.weight"),
                                        src.get(p + "mlp.up_proj.weight")]), cfg.proj_format)
            lw.down = lin(src.get(p + "mlp.down_proj.weight"), cfg.proj_format)
        tensors = {k: v.detach().cpu().contiguous()
                   for k, v in _layer_tensors(f"layers.{i}", lw).items()}
        tmp = path.with_suffix(".tmp")
        save_file(tensors, str(tmp))
        os.replace(tmp, path)
        record["done"][key] = path.stat().st_size
        _atomic_json(record_path, record)
        if on_layer:
            on_layer(i, False)

    # ---- assemble -----------------------------------------------------------------------
    for k in {cfg.hidden, cfg.q_heads * cfg.head_dim, cfg.ffn or cfg.expert_ffn}:
        sign(k)
    layers: List[LayerWeights] = []
    for i in range(cfg.layers):
        t = load_file(str(work / f"layer_{i:05d}.safetensors"))
        layers.append(_load_layer(t, f"layers.{i}", "attn", signs))
    emb = quantize_linear(src.get("model.embed_tokens.weight"), "w8", None)
    if cfg.tied_embeddings:
        head = QLinear("w8", cfg.vocab, cfg.hidden, emb.codes, emb.scale, None)
    else:
        hq = quantize_linear(src.get("lm_head.weight").to(dev), cfg.head_format, None, fast=fast)
        head = QLinear(hq.fmt, hq.n, hq.k, hq.codes.cpu(), hq.scale.cpu(), None)
    weights = ModelWeights(cfg, emb.codes, emb.scale, layers, f16(src.get("model.norm.weight")),
                           head, signs)
    for asset in ASSETS:
        if (source / asset).exists():
            shutil.copyfile(source / asset, output / asset)
    save_model(weights, output, cfg.name)
    shutil.rmtree(work)
    return output


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("source")
    ap.add_argument("output")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--exhaustive", action="store_true", help="slower search, lower error")
    ap.add_argument("--name", default=None)
    ap.add_argument("--format", action="append", default=[], metavar="KEY=FMT",
                    help="e.g. --format attn_format=w8 (q4 | q2 | w8)")
    a = ap.parse_args(argv)
    try:
        out = convert(a.source, a.output, a.device, fast=not a.exhaustive, name=a.name,
                      formats=dict(x.split("=", 1) for x in a.format) or None,
                      on_layer=lambda i, resumed: print(
                          f"layer {i} {'kept' if resumed else 'quantised'}", flush=True))
    except ConvertError as e:
        print(str(e))
        return 2
    print(json.dumps({"model": str(out)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
