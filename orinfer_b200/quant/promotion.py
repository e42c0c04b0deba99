"""Precision promotion: re-encode the projections of selected decoder layers as rotated W8
from the original weights, keeping every other tensor of an already converted model as it is.

A few layers (typically the first and last ones) are far more sensitive to 4-bit weights
than the rest; promoting just those recovers most of the quality gap for a small size cost.
The promoted matrices stay in the rotated input basis (same signs), so the runtime runs them
through the W8A8 kernels with the activation preparation it already does.

    python -m orinfer_b200.quant.promotion SOURCE_DIR MODEL_DIR OUTPUT_DIR --layers 0,1,35

What is promoted per layer: the attention projections that read the hidden state (q, k, v:
the fused ``qkv``; the GDN input projection of a linear-attention layer) and the dense FFN
(``gate_up``, ``down``); the attention output projection and routed experts keep their
format, as in python/orinfer_build/quantization/promotion.py:41-55.  The report lists the
relative squared error of every promoted matrix in the rotated basis (``:96-123``).
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import shutil
from pathlib import Path
from typing import Dict, Iterable, List, Optional

import torch

from ..models.weights import LayerWeights, QLinear, quantize_linear
from .convert import ASSETS, ConvertError, _Source, build_layer, config_from_hf

PROMOTED = ("qkv", "gdn_qkvz", "gate_up", "down", "shared_gate_up", "shared_down")


def _relative_error(lin: QLinear, weight: torch.Tensor) -> float:
    from ..ref.ops_ref import hadamard_rotate
    ref = hadamard_rotate(weight.float(), lin.signs) if lin.signs is not None else weight.float()
    got = lin.codes.float() * lin.scale.float()[:, None]
    return float((got - ref).square().sum() / ref.square().sum().clamp_min(1e-30))


def promote(source, model_dir, output, layers: Iterable[int], device: str = "cpu") -> dict:
    """Writes a copy of ``model_dir`` to ``output`` with ``layers`` promoted; returns the
    report ``{"layers": [...], "matrices": {name: relative_mse}, "bytes_before", "bytes_after"}``."""
    from ..engine.checkpoint import load_model, read_descriptor, save_model
    source, model_dir, output = Path(source), Path(model_dir), Path(output)
    layers = sorted(set(int(i) for i in layers))
    weights = load_model(model_dir, "cpu", verify=True)
    cfg = weights.config
    src_cfg = config_from_hf(json.loads((source / "config.json").read_text()), cfg.name)
    same = ("hidden", "layers", "q_heads", "kv_heads", "head_dim", "ffn", "experts", "vocab")
    if any(getattr(cfg, f) != getattr(src_cfg, f) for f in same):
        raise ConvertError("the source weights are not those of the converted model")
    if not layers or layers[0] < 0 or layers[-1] >= cfg.layers:
        raise ConvertError(f"layers must be within 0..{cfg.layers - 1}")
    src = _Source(source)
    dev = torch.device(device)
    report: Dict[str, float] = {}
    errors: Dict[int, float] = {}

    def lin(weight: torch.Tensor, fmt: str) -> QLinear:
        signs = weights.signs[weight.shape[1]]
        q = quantize_linear(weight.to(dev), fmt, signs.to(dev))
        out = QLinear(q.fmt, q.n, q.k, q.codes.cpu(), q.scale.cpu(), signs)
        errors[id(out)] = _relative_error(out, weight)
        return out

    before = sum(_layer_bytes(lw) for lw in weights.layers)
    w8 = dataclasses.replace(src_cfg, attn_format="w8", proj_format="w8")
    for i in layers:
        fresh = build_layer(w8, src, i, lin)
        old = weights.layers[i]
        for field in PROMOTED:
            new_lin: Optional[QLinear] = getattr(fresh, field, None)
            if new_lin is None or getattr(old, field, None) is None:
                continue
            setattr(old, field, new_lin)
            report[f"layers.{i}.{field}"] = errors[id(new_lin)]
    after = sum(_layer_bytes(lw) for lw in weights.layers)
    output.mkdir(parents=True, exist_ok=True)
    for asset in ASSETS:
        if (model_dir / asset).exists():
            shutil.copyfile(model_dir / asset, output / asset)
    save_model(weights, output, read_descriptor(model_dir).get("name", cfg.name))
    result = {"layers": layers, "precision": "rotated-w8", "matrices": report,
              "bytes_before": before, "bytes_after": after}
    (output / "promotion.json").write_text(json.dumps(result, indent=1, sort_keys=True))
    return result


def _layer_bytes(lw: LayerWeights) -> int:
    total = 0
    for field in dataclasses.fields(lw):
        v = getattr(lw, field.name)
        if isinstance(v, QLinear):
            total += v.codes.numel() * v.codes.element_size() + v.scale.numel() * 2
        elif hasattr(v, "codes") and hasattr(v, "scale"):
            total += v.codes.numel() * v.codes.element_size() + v.scale.numel() * 2
    return total


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="orinfer_b200.quant.promotion", description=__doc__)
    ap.add_argument("source")
    ap.add_argument("model_dir")
    ap.add_argument("output")
    ap.add_argument("--layers", required=True, help="comma-separated layer numbers")
    ap.add_argument("--device", default="cpu")
    args = ap.parse_args(argv)
    rep = promote(args.source, args.model_dir, args.output,
                  [int(x) for x in args.layers.split(",") if x], args.device)
    for name, err in sorted(rep["matrices"].items()):
        print(f"PROMOTED {name} relative_mse {err:.3e}")
    print(f"COMPLETE {rep['bytes_before']} -> {rep['bytes_after']} layer bytes")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
