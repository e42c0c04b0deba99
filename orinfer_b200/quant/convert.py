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
    plain = ("LlamaForCausalLM", "MistralForCausalLM")       # same decoder without head norms
    if arch not in ("Qwen3ForCausalLM", "Qwen3MoeForCausalLM", "Qwen3NextForCausalLM") + plain:
        raise ConvertError(f"unsupported architecture `{arch}` (Qwen3 dense, MoE and the hybrid "
                           "gated-delta-rule family, Llama and Mistral are converted)")
    if hf.get("mlp_bias") or hf.get("sliding_window"):
        raise ConvertError("MLP biases and sliding-window attention are not supported")
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
    if arch == "Qwen3NextForCausalLM":
        period = hf.get("full_attention_interval") or 4
        types = hf.get("layer_types")
        want = ["full_attention" if i % period == period - 1 else "linear_attention"
                for i in range(hf["num_hidden_layers"])]
        if types is not None and list(types) != want:
            raise ConvertError("layer_types must repeat (period - 1) linear layers and one "
                               "full-attention layer")
        if hf.get("linear_key_head_dim") != hf.get("linear_value_head_dim"):
            raise ConvertError("key and value head sizes of the linear layers must be equal")
        if hf.get("mlp_only_layers") or hf.get("decoder_sparse_step", 1) != 1:
            raise ConvertError("mixed dense / sparse layer stacks are not supported")
        factor = hf.get("partial_rotary_factor") or rope.get("partial_rotary_factor") or 1.0
        rotary = int(common["head_dim"] * factor)
        return ModelConfig(
            arch="hybrid", ffn=0, gdn_period=period, gdn_k_heads=hf["linear_num_key_heads"],
            gdn_v_heads=hf["linear_num_value_heads"], gdn_head_dim=hf["linear_key_head_dim"],
            gdn_conv=hf.get("linear_conv_kernel_dim", 4),
            experts=hf.get("num_experts") or hf.get("num_local_experts"),
            top_k=hf["num_experts_per_tok"], expert_ffn=hf["moe_intermediate_size"],
            shared_expert_ffn=hf.get("shared_expert_intermediate_size", 0),
            renormalize=bool(hf.get("norm_topk_prob", True)), gated_attention=True,
            zero_centered_norm=True, rotary_dim=0 if rotary == common["head_dim"] else rotary,
            **common)
    if arch == "Qwen3MoeForCausalLM":
        if hf.get("mlp_only_layers") or hf.get("decoder_sparse_step", 1) != 1:
            raise ConvertError("mixed dense / sparse layer stacks are not supported")
        experts = hf.get("num_experts") or hf.get("num_local_experts")
        if not experts:
            raise ConvertError("the configuration does not say how many experts there are")
        return ModelConfig(arch="moe", ffn=0, experts=experts,
                           top_k=hf["num_experts_per_tok"], expert_ffn=hf["moe_intermediate_size"],
                           renormalize=bool(hf.get("norm_topk_prob", True)), **common)
    return ModelConfig(arch="dense", ffn=hf["intermediate_size"], qk_norm=arch not in plain,
                       **common)


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


def rotary_permutation(head_dim: int, rotary_dim: int) -> torch.Tensor:
    """Channel order that turns "rotate the first ``rotary_dim`` channels in pairs
    ``(i, i + rotary_dim / 2)``" into this engine's pairing ``(i, i + head_dim / 2)``:
    ``new[j] = old[perm[j]]``.  Applied alike to q rows, k rows and their head-norm weights it
    leaves every attention score unchanged."""
    if not rotary_dim or rotary_dim == head_dim:
        return torch.arange(head_dim)
    half, r2 = head_dim // 2, rotary_dim // 2
    rest = torch.arange(rotary_dim, head_dim)
    fill = half - r2
    return torch.cat([torch.arange(0, r2), rest[:fill], torch.arange(r2, rotary_dim), rest[fill:]])


def _atomic_json(path: Path, obj) -> None:
    tmp = path.with_suffix(path.suffix + ".tmp")
    tmp.write_text(json.dumps(obj, indent=1))
    os.replace(tmp, path)


def _f16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float16).contiguous()


DRAFT_PREFIX = "mtp."


def has_draft_head(src: "_Source") -> bool:
    return DRAFT_PREFIX + "fc.weight" in src.where


def build_draft_head(cfg: ModelConfig, src: "_Source", lin):
    """The checkpoint's draft head (``mtp.*`` tensors of the Qwen3-Next / Qwen3.5 families):
    norms of the token embedding and of the target's hidden state, the [H, 2H] projection of
    their concatenation (embedding half first), one full-attention decoder layer shaped like
    the model's own, and the norm before the shared vocabulary head."""
    from ..models.weights import MtpWeights
    p = DRAFT_PREFIX
    layer = build_layer(cfg, src, 0, lin, prefix=p + "layers.0.", full=True)
    fc = quantize_linear(src.get(p + "fc.weight"), "w8", None)
    fc = QLinear(fc.fmt, fc.n, fc.k, fc.codes.cpu(), fc.scale.cpu(), None)
    return MtpWeights(_f16(src.get(p + "pre_fc_norm_embedding.weight")),
                      _f16(src.get(p + "pre_fc_norm_hidden.weight")), fc, layer,
                      _f16(src.get(p + "norm.weight")))


def build_layer(cfg: ModelConfig, src: "_Source", i: int, lin, prefix: Optional[str] = None,
                full: Optional[bool] = None) -> LayerWeights:
    """Assembles decoder layer ``i`` from the source tensors; ``lin(weight, fmt)`` quantises
    one projection.  Formats come from ``cfg`` (``attn_format`` / ``proj_format`` /
    ``expert_format``).  ``prefix`` / ``full``: a layer that lives elsewhere in the checkpoint
    (the draft head's)."""
    f16 = _f16
    p = prefix or f"model.layers.{i}."
    full = cfg.is_full_attention(i) if full is None else full
    lw = LayerWeights("attn" if full else "gdn", f16(src.get(p + "input_layernorm.weight")),
                      f16(src.get(p + "post_attention_layernorm.weight")))
    if full:
        d, perm = cfg.head_dim, rotary_permutation(cfg.head_dim, cfg.rotary_dim)
        q = src.get(p + "self_attn.q_proj.weight")
        k = src.get(p + "self_attn.k_proj.weight").reshape(cfg.kv_heads, d, -1)[:, perm]
        if cfg.gated_attention:                # per head: d query rows, then d gate rows
            q = q.reshape(cfg.q_heads, 2, d, -1)
            q = torch.cat([q[:, 0][:, perm], q[:, 1]], dim=1)
        else:
            q = q.reshape(cfg.q_heads, d, -1)[:, perm]
        lw.qkv = lin(torch.cat([q.reshape(-1, cfg.hidden), k.reshape(-1, cfg.hidden),
                                src.get(p + "self_attn.v_proj.weight")]), cfg.attn_format)
        if cfg.qk_norm:
            lw.q_norm = f16(src.get(p + "self_attn.q_norm.weight")[perm])
            lw.k_norm = f16(src.get(p + "self_attn.k_norm.weight")[perm])
        lw.o = lin(src.get(p + "self_attn.o_proj.weight"), cfg.attn_format)
    else:
        hk, hv, gd = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
        rep = hv // hk
        # source rows are grouped per key head: q | k | v of its value heads | z of them
        w = src.get(p + "linear_attn.in_proj_qkvz.weight").reshape(hk, 2 * gd + 2 * rep * gd, -1)
        parts = torch.split(w, [gd, gd, rep * gd, rep * gd], dim=1)
        lw.gdn_qkvz = lin(torch.cat([x.reshape(-1, cfg.hidden) for x in parts]),
                          cfg.attn_format)
        ba = src.get(p + "linear_attn.in_proj_ba.weight").reshape(hk, 2 * rep, -1)
        lw.gdn_ab = f16(torch.cat([ba[:, rep:].reshape(hv, -1), ba[:, :rep].reshape(hv, -1)]))
        lw.gdn_conv = f16(src.get(p + "linear_attn.conv1d.weight")[:, 0, :])
        lw.gdn_a_log = src.get(p + "linear_attn.A_log").float().contiguous()
        lw.gdn_dt_bias = src.get(p + "linear_attn.dt_bias").float().contiguous()
        lw.gdn_norm = f16(src.get(p + "linear_attn.norm.weight"))
        lw.gdn_out = lin(src.get(p + "linear_attn.out_proj.weight"), cfg.attn_format)
    if cfg.experts:
        router = src.get(p + "mlp.gate.weight")
        if cfg.shared_expert_ffn:
            router = torch.cat([router, src.get(p + "mlp.shared_expert_gate.weight")])
            lw.shared_gate_up = lin(torch.cat([
                src.get(p + "mlp.shared_expert.gate_proj.weight"),
                src.get(p + "mlp.shared_expert.up_proj.weight")]), cfg.proj_format)
            lw.shared_down = lin(src.get(p + "mlp.shared_expert.down_proj.weight"),
                                 cfg.proj_format)
        lw.router = f16(router)
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
    return lw


def beam_refine(lin: QLinear, weight: torch.Tensor, device: str = "cpu", rows: int = 128) -> QLinear:
    """Re-searches the codes of a Q4 projection with the beam-8 refinement (``search.py``),
    ``rows`` output rows at a time; other formats pass through."""
    if lin.fmt != "q4":
        return lin
    from . import search
    n, k = lin.n, lin.k
    packed = lin.codes.cpu().permute(1, 0, 2).reshape(n, k // 8).numpy().view("uint32")
    scales = lin.scale.cpu().numpy().copy()
    out = packed.copy()
    signs = lin.signs.cpu().numpy().astype("int8")
    for lo in range(0, n, rows):
        cur = e8p.Q4Weight(packed[lo:lo + rows], scales[lo:lo + rows], signs)
        new = search.refine_q4(weight[lo:lo + rows].float().cpu().numpy(), cur, device=device)
        out[lo:lo + rows], scales[lo:lo + rows] = new.packed, new.scales
    codes = torch.from_numpy(out.view("int32")).reshape(n, k // 128, 16).permute(1, 0, 2)
    return QLinear("q4", n, k, codes.contiguous(), torch.from_numpy(scales), lin.signs, lin.dense)


def convert(source, output, device: str = "cpu", fast: bool = True, name: Optional[str] = None,
            on_layer: Optional[Callable[[int, bool], None]] = None,
            formats: Optional[Dict[str, str]] = None, search: str = "nearest") -> Path:
    """Returns the model directory.  ``on_layer(i, resumed)`` is called after layer ``i`` is on
    disk (freshly quantised or found in the progress record).  ``formats`` overrides the
    weight formats of the geometry (``attn_format``, ``proj_format``, ``expert_format``,
    ``head_format``: ``q4`` | ``q2`` | ``w8``; ``attn_format`` and ``proj_format`` also take
    ``rq4``: scalar level-table rows of ``quant/row_q4.py``, stored as 4-bit nibbles and run as
    8-bit weights).  ``search="beam8"`` re-searches every Q4
    projection with the top-8 coarse-candidate refinement (slower, lower weight error)."""
    if search not in ("nearest", "beam8"):
        raise ConvertError("search is nearest or beam8")
    from ..engine.checkpoint import _layer_tensors, _load_layer, save_model
    source, output = Path(source), Path(output)
    config_text = (source / "config.json").read_text()
    cfg = config_from_hf(json.loads(config_text), name)
    if formats:
        import dataclasses
        unknown = set(formats) - {"attn_format", "proj_format", "expert_format", "head_format"}
        if unknown or any(v not in ("q4", "q2", "w8", "rq4") for v in formats.values()):
            raise ConvertError("formats maps attn / proj / expert / head_format to q4, q2, w8 "
                               "or rq4")
        if any(v == "rq4" for k, v in formats.items() if k in ("expert_format", "head_format")):
            raise ConvertError("rq4 (scalar level-table rows) serves attn_format and proj_format")
        # rq4 rows run as W8 (their levels are INT8 values); only the stored form differs, so
        # the saved geometry says w8 and the layer builder is told rq4
        build_cfg = dataclasses.replace(cfg, **formats)
        cfg = dataclasses.replace(cfg, **{k: ("w8" if v == "rq4" else v)
                                          for k, v in formats.items()})
    else:
        build_cfg = cfg
    src = _Source(source)
    if has_draft_head(src):
        import dataclasses
        cfg = dataclasses.replace(cfg, mtp_layers=1, draft_layer="model")
        build_cfg = dataclasses.replace(build_cfg, mtp_layers=1, draft_layer="model")
    work = output / ".convert"
    work.mkdir(parents=True, exist_ok=True)
    identity = src.identity(config_text + f"|{build_cfg.attn_format}|{build_cfg.proj_format}"
                            f"|{cfg.expert_format}|{cfg.head_format}|{fast}"
                            + ("" if search == "nearest" else f"|{search}"))
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
        if fmt == "rq4":
            from . import row_q4
            q = row_q4.fit(weight.float().cpu().numpy(), s.cpu().numpy().astype("int8"))
            codes, scale = row_q4.expand_to_w8(q)
            return QLinear("w8", weight.shape[0], weight.shape[1], torch.from_numpy(codes),
                           torch.from_numpy(scale), s, None, torch.from_numpy(q.packed))
        q = quantize_linear(weight.to(dev), fmt, s.to(dev), fast=fast)
        q = QLinear(q.fmt, q.n, q.k, q.codes.cpu(), q.scale.cpu(), s)
        return beam_refine(q, weight, device) if search == "beam8" else q

    f16 = _f16

    for i in range(cfg.layers):
        key, path = f"layer.{i}", work / f"layer_{i:05d}.safetensors"
        done = record["done"].get(key)
        if done and path.exists() and path.stat().st_size == done:
            if on_layer:
                on_layer(i, True)
            continue
        lw = build_layer(build_cfg, src, i, lin)
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
    for k in {cfg.hidden, cfg.q_heads * cfg.head_dim, cfg.ffn or cfg.expert_ffn,
              cfg.shared_expert_ffn or cfg.hidden, (cfg.gdn_v_heads * cfg.gdn_head_dim) or cfg.hidden}:
        sign(k)
    layers: List[LayerWeights] = []
    for i in range(cfg.layers):
        t = load_file(str(work / f"layer_{i:05d}.safetensors"))
        layers.append(_load_layer(t, f"layers.{i}",
                                  "attn" if cfg.is_full_attention(i) else "gdn", signs))
    emb = quantize_linear(src.get("model.embed_tokens.weight"), "w8", None)
    if cfg.tied_embeddings:
        head = QLinear("w8", cfg.vocab, cfg.hidden, emb.codes, emb.scale, None)
    else:
        hq = quantize_linear(src.get("lm_head.weight").to(dev), cfg.head_format, None, fast=fast)
        head = QLinear(hq.fmt, hq.n, hq.k, hq.codes.cpu(), hq.scale.cpu(), None)
    mtp = None
    if cfg.mtp_layers:
        from ..models.weights import MtpWeights
        dpath = work / "draft.safetensors"
        done = record["done"].get("draft")
        if not (done and dpath.exists() and dpath.stat().st_size == done):
            m = build_draft_head(build_cfg, src, lin)
            t = {"norm_e": m.norm_e, "norm_h": m.norm_h, "final_norm": m.final_norm,
                 "fc.int8": m.fc.codes, "fc.scale": m.fc.scale}
            t.update(_layer_tensors("layer", m.layer))
            tmp = dpath.with_suffix(".tmp")
            save_file({k: v.detach().cpu().contiguous() for k, v in t.items()}, str(tmp))
            os.replace(tmp, dpath)
            record["done"]["draft"] = dpath.stat().st_size
            _atomic_json(record_path, record)
        t = load_file(str(dpath))
        fc = QLinear("w8", t["fc.int8"].shape[0], t["fc.int8"].shape[1], t["fc.int8"],
                     t["fc.scale"], None)
        mtp = MtpWeights(t["norm_e"], t["norm_h"], fc, _load_layer(t, "layer", "attn", signs),
                         t["final_norm"])
    weights = ModelWeights(cfg, emb.codes, emb.scale, layers, f16(src.get("model.norm.weight")),
                           head, signs, mtp)
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
    ap.add_argument("--search", default="nearest", choices=["nearest", "beam8"],
                    help="beam8: top-8 coarse candidates per vector (Q4 projections)")
    ap.add_argument("--format", action="append", default=[], metavar="KEY=FMT",
                    help="e.g. --format attn_format=w8 (q4 | q2 | w8; attn / proj also rq4)")
    a = ap.parse_args(argv)
    try:
        out = convert(a.source, a.output, a.device, fast=not a.exhaustive, name=a.name, search=a.search,
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
