"""Validate a serving plan before anything is allocated.

``validate_plan`` checks the geometry of a model against the options it is to be served with
(context, pages, rows, ranks) and against the device it is to run on, and returns the memory
plan: bytes of weights, KV pages, workspaces and host tables.  It raises ``PlanError`` with
the offending quantity in the message, so a model that cannot be served fails with a sentence
rather than with an allocator error half way through start-up.  With a checkpoint descriptor
(``cache/model.json``) it also checks that every projection the geometry needs is listed with
its codes and scales and, when ``exhaustive``, that every digest is well formed.

The command line calls it before it constructs an engine (``serve``, ``generate``,
``run-model`` ...); ``orinfer plan-model [--tp N] [--max-context T] [--device-gib G]`` prints
the result or the reason a plan is refused.  Role of the reference's plan validation
(crates/orinfer-model-sdk/src/model.rs:399-827: dimensions, buffer and tensor identities,
weight accounting, KV allocation contract, all before allocation).
"""

from __future__ import annotations

import dataclasses
import re
from typing import Dict, Optional

from ..config import LoadOptions, ModelConfig, SchedulerOptions

PAGE_TOKENS = 128
INT32_MAX = 2 ** 31 - 1
FORMAT_BITS = {"q4": 4.0, "q2": 2.0, "w8": 8.0}
_SHA256 = re.compile(r"^[0-9a-f]{64}$")


class PlanError(ValueError):
    """The model cannot be served with these options on this device."""


@dataclasses.dataclass(frozen=True)
class MemoryPlan:
    weight_parameters: int
    weight_bytes: int             # this rank's share
    kv_bytes_per_page: int
    kv_pages: int
    kv_bytes: int
    workspace_bytes: int
    table_bytes: int
    total_bytes: int
    device_bytes: Optional[int]
    max_context: int
    max_rows: int
    world: int

    def as_dict(self) -> Dict[str, int]:
        return dataclasses.asdict(self)


def _linear_bytes(n: int, k: int, fmt: str) -> int:
    """Codes plus one FP16 scale per output row."""
    return int(n * k * FORMAT_BITS[fmt] / 8) + 2 * n


def weight_shapes(cfg: ModelConfig) -> Dict[str, tuple]:
    """(rows, columns, format) of every quantised projection of one rank-less model, keyed by
    the checkpoint's tensor stem; norms and small FP16 / FP32 tensors are accounted apart."""
    out: Dict[str, tuple] = {}
    h = cfg.hidden
    for i in range(cfg.layers):
        p = f"layers.{i}."
        if cfg.is_full_attention(i):
            q_rows = cfg.q_heads * cfg.head_dim * (2 if cfg.gated_attention else 1)
            out[p + "qkv"] = (q_rows + 2 * cfg.kv_heads * cfg.head_dim, h, cfg.attn_format)
            out[p + "o"] = (h, cfg.q_heads * cfg.head_dim, cfg.attn_format)
        else:
            dk, dv = cfg.gdn_k_heads * cfg.gdn_head_dim, cfg.gdn_v_heads * cfg.gdn_head_dim
            out[p + "gdn_qkvz"] = (2 * dk + 2 * dv, h, cfg.attn_format)
            out[p + "gdn_out"] = (h, dv, cfg.attn_format)
        if cfg.experts:
            out[p + "expert_gate_up"] = (cfg.experts * 2 * cfg.expert_ffn, h, cfg.expert_format)
            out[p + "expert_down"] = (cfg.experts * h, cfg.expert_ffn, cfg.expert_format)
            if cfg.shared_expert_ffn:
                out[p + "shared_gate_up"] = (2 * cfg.shared_expert_ffn, h, cfg.proj_format)
                out[p + "shared_down"] = (h, cfg.shared_expert_ffn, cfg.proj_format)
        else:
            out[p + "gate_up"] = (2 * cfg.ffn, h, cfg.proj_format)
            out[p + "down"] = (h, cfg.ffn, cfg.proj_format)
    if cfg.mtp_layers:
        # the draft head: its [H, 2H] input projection and one full-attention layer, shaped
        # like the model's own layers or (the presets) a dense W8 layer
        p = "mtp.layer."
        out["mtp.fc"] = (h, 2 * h, "w8")
        own = cfg.draft_layer == "model"
        gated = 2 if own and cfg.gated_attention else 1
        attn_fmt = cfg.attn_format if own else "w8"
        out[p + "qkv"] = (cfg.q_heads * cfg.head_dim * gated + 2 * cfg.kv_heads * cfg.head_dim,
                          h, attn_fmt)
        out[p + "o"] = (h, cfg.q_heads * cfg.head_dim, attn_fmt)
        if own and cfg.experts:
            out[p + "expert_gate_up"] = (cfg.experts * 2 * cfg.expert_ffn, h, cfg.expert_format)
            out[p + "expert_down"] = (cfg.experts * h, cfg.expert_ffn, cfg.expert_format)
            if cfg.shared_expert_ffn:
                out[p + "shared_gate_up"] = (2 * cfg.shared_expert_ffn, h, cfg.proj_format)
                out[p + "shared_down"] = (h, cfg.shared_expert_ffn, cfg.proj_format)
        else:
            f = cfg.ffn or max(cfg.expert_ffn * 4, 512)
            fmt = cfg.proj_format if own else "w8"
            out[p + "gate_up"] = (2 * f, h, fmt)
            out[p + "down"] = (h, f, fmt)
    out["embed"] = (cfg.vocab, h, "w8")
    if not cfg.tied_embeddings:
        out["head"] = (cfg.vocab, h, cfg.head_format)
    return out


def _check_dimensions(cfg: ModelConfig, world: int, max_context: int, max_rows: int,
                      sched: SchedulerOptions) -> None:
    if cfg.layers <= 0 or cfg.hidden <= 0 or cfg.vocab <= 0 or cfg.vocab > INT32_MAX:
        raise PlanError(f"invalid model dimensions (layers {cfg.layers}, hidden {cfg.hidden}, "
                        f"vocab {cfg.vocab})")
    for name in ("attn_format", "proj_format", "expert_format", "head_format"):
        if getattr(cfg, name) not in FORMAT_BITS:
            raise PlanError(f"{name} {getattr(cfg, name)!r} is not one of q4, q2, w8")
    if max_context <= 0 or max_context > INT32_MAX:
        raise PlanError(f"max_context {max_context} is outside 1..2^31-1")
    if max_context > cfg.max_context:
        raise PlanError(f"max_context {max_context} exceeds the model's {cfg.max_context}")
    if sched.prefill_chunk <= 0 or sched.max_active <= 0:
        raise PlanError("prefill_chunk and max_active must be positive")
    if max_rows < min(sched.prefill_chunk, max_context) or max_rows < sched.max_active:
        raise PlanError(f"max_rows {max_rows} cannot hold a prefill chunk of "
                        f"{sched.prefill_chunk} rows or {sched.max_active} decode rows")
    if cfg.experts and not 0 < cfg.top_k <= cfg.experts:
        raise PlanError(f"top_k {cfg.top_k} is outside 1..{cfg.experts}")
    if world < 1:
        raise PlanError("world must be at least 1")
    if world > 1:
        # the sharding rules themselves decide (uneven 128-wide FFN and vocabulary blocks are
        # fine; heads must split evenly)
        from ..parallel.tp import layout
        try:
            for rank in range(world):
                lay = layout(cfg, rank, world)
                if cfg.ffn and lay.ffn[1] <= lay.ffn[0]:
                    raise ValueError(f"rank {rank} would get no FFN channels")
                if lay.vocab[1] <= lay.vocab[0]:
                    raise ValueError(f"rank {rank} would get no vocabulary rows")
        except ValueError as e:
            raise PlanError(f"{world} ranks: {e}") from e
        if cfg.experts and cfg.experts % world:
            raise PlanError(f"{cfg.experts} experts do not split over {world} ranks")
        for what, heads in (("GDN key", cfg.gdn_k_heads), ("GDN value", cfg.gdn_v_heads)):
            if heads % world:
                raise PlanError(f"{heads} {what} heads do not split over {world} ranks")
        if cfg.gdn_v_heads and (cfg.gdn_v_heads // world * cfg.gdn_head_dim) % 128:
            raise PlanError(f"GDN value heads per rank must cover a multiple of 128 channels")


def _check_descriptor(cfg: ModelConfig, descriptor: dict, exhaustive: bool) -> None:
    """``descriptor["tensors"]`` maps tensor names to SHA-256 digests.  Every projection the
    geometry needs must be there with its codes (whatever their format: promoted layers carry
    8-bit codes in a 4-bit model) and its scales; a digest must look like one."""
    tensors = descriptor.get("tensors")
    if not isinstance(tensors, dict) or not tensors:
        raise PlanError("descriptor lists no tensors")
    if descriptor.get("target", "sm_100a") != "sm_100a":
        raise PlanError(f"descriptor targets {descriptor.get('target')!r}, not sm_100a")
    if exhaustive:
        for name, digest in tensors.items():
            if not _SHA256.match(str(digest)):
                raise PlanError(f"tensor {name}: malformed hash")
    for stem in weight_shapes(cfg):
        if stem == "head" and cfg.tied_embeddings:
            continue
        if stem + ".scale" not in tensors:
            raise PlanError(f"descriptor has no scales for {stem}")
        if not any(stem + suffix in tensors for suffix in (".int8", ".packed", ".packed16", ".rowq4")):
            raise PlanError(f"descriptor has no weight codes for {stem}")
    for name in ("final_norm", "orinfer.e8p_q4.basis"):
        if name not in tensors:
            raise PlanError(f"descriptor has no tensor {name}")


def validate_plan(cfg: ModelConfig, load: LoadOptions, sched: SchedulerOptions, *,
                  max_context: Optional[int] = None, kv_pages: Optional[int] = None,
                  max_rows: Optional[int] = None, world: int = 1,
                  device_bytes: Optional[int] = None, descriptor: Optional[dict] = None,
                  exhaustive: bool = False, headroom: float = 0.94) -> MemoryPlan:
    max_context = max_context or min(cfg.max_context, 32768)
    max_rows = max_rows or max(sched.prefill_chunk + sched.max_active, 256)
    _check_dimensions(cfg, world, max_context, max_rows, sched)
    if descriptor is not None:
        _check_descriptor(cfg, descriptor, exhaustive)

    shapes = weight_shapes(cfg)
    params = sum(n * k for n, k, _ in shapes.values())
    sharded = sum(_linear_bytes(n, k, f) for s, (n, k, f) in shapes.items() if s != "embed")
    replicated = _linear_bytes(*shapes["embed"])
    small = cfg.layers * (4 * cfg.hidden * 2) + cfg.hidden * 2       # norms
    if cfg.experts:
        small += cfg.layers * (cfg.experts + 1) * cfg.hidden * 2     # router rows
    weight_bytes = sharded // world + replicated + small

    from ..models.runner import KVPool
    per_page = KVPool.bytes_per_page(cfg, cfg.mtp_layers)
    if world > 1:
        per_page = per_page // min(world, max(cfg.kv_heads, 1)) if cfg.kv_heads else per_page
    pages_per_request = (max_context + PAGE_TOKENS - 1) // PAGE_TOKENS
    if kv_pages is not None:
        if kv_pages < pages_per_request + 1:
            raise PlanError(f"{kv_pages} KV pages cannot hold one request of {max_context} "
                            f"tokens ({pages_per_request} pages) beside the padding page")
        pages = kv_pages
    else:
        pages = pages_per_request + 1
    kv_bytes = per_page * pages
    widest = max(cfg.hidden, (cfg.ffn or cfg.expert_ffn * max(cfg.top_k, 1)) * 2 // world,
                 (cfg.q_heads * cfg.head_dim * 3) // world)
    workspace = max_rows * (cfg.hidden * (4 + 2 + 2 + 1) + widest * 3)
    head_rows = min(max_rows, sched.max_active + 64)
    workspace += head_rows * (cfg.vocab // world) * 4
    tables = (sched.max_active + 1) * pages_per_request * 4 * 2
    total = weight_bytes + kv_bytes + workspace + tables
    if device_bytes is not None and total > device_bytes * headroom:
        gib = lambda b: f"{b / 2 ** 30:.1f} GiB"
        raise PlanError(
            f"the plan needs {gib(total)} per device (weights {gib(weight_bytes)}, KV "
            f"{gib(kv_bytes)} for {pages} pages, workspaces {gib(workspace)}) and the device "
            f"has {gib(device_bytes)}; lower max_context, kv_pages or max_rows, or use more ranks")
    return MemoryPlan(params, weight_bytes, per_page, pages, kv_bytes, workspace, tables, total,
                      device_bytes, max_context, max_rows, world)
