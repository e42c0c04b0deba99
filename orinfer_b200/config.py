"""Typed configuration: model geometry, load options, scheduler options.

Mirrors the reference's contracts: ``GraphMode`` / ``ExecutionPhase``
(crates/orinfer-model-sdk/src/device.rs:37-60), ``LoadOptions``
(crates/orinfer-engine/src/execution.rs:13-69) and the scheduler ``Options``
defaults and limits (crates/orinfer-engine/src/scheduler.rs:10-33).
The only supported device target is ``sm_100a``.
"""

from __future__ import annotations

import dataclasses
import enum
import json
from dataclasses import dataclass, field
from typing import Optional

TARGET = "sm_100a"
PAGE_TOKENS = 128          # tokens per KV page
KV_GROUP = 64              # channels per INT8-KV scale group
MAX_MTP_DRAFTS = 31
MAX_ACTIVE_LIMIT = 128


class GraphMode(str, enum.Enum):
    OFF = "off"
    DECODE_ONLY = "decode_only"
    FULL = "full"

    def uses_graph(self, phase: "Phase") -> bool:
        if self is GraphMode.OFF:
            return False
        if self is GraphMode.FULL:
            return True
        return phase is Phase.DECODE


class Phase(str, enum.Enum):
    PREFILL = "prefill"
    DECODE = "decode"
    VISION = "vision"


class Policy(str, enum.Enum):
    LATENCY = "latency"
    THROUGHPUT = "throughput"


@dataclass(frozen=True)
class ModelConfig:
    """Decoder geometry.  ``arch`` selects the layer recipe:

    * ``dense``  - Qwen3-style: RMSNorm, q/k head norm, NeoX RoPE, GQA, SwiGLU.
    * ``moe``    - the same attention with a top-k routed SwiGLU expert FFN.
    * ``hybrid`` - groups of ``gdn_period`` layers, the last one gated GQA, the
      others gated-delta-rule linear attention; MoE FFN with a shared expert.
    """

    name: str = "tiny"
    arch: str = "dense"
    layers: int = 2
    hidden: int = 256
    q_heads: int = 4
    kv_heads: int = 2
    head_dim: int = 64
    ffn: int = 512
    vocab: int = 1024
    eps: float = 1e-6
    rope_theta: float = 1e6
    rotary_dim: int = 0            # channels of a head that rotate (0 = all of them)
    tied_embeddings: bool = True
    zero_centered_norm: bool = False
    qk_norm: bool = True
    gated_attention: bool = False
    # projections: "q4" (two-stage E8P), "w8", "q2"
    proj_format: str = "q4"
    attn_format: str = "q4"
    head_format: str = "w8"
    embed_format: str = "w8"
    # MoE
    experts: int = 0
    top_k: int = 0
    expert_ffn: int = 0
    shared_expert_ffn: int = 0
    expert_format: str = "q4"
    renormalize: bool = True
    # hybrid linear attention
    gdn_period: int = 0            # 4 => 3 GDN + 1 full attention per group
    gdn_k_heads: int = 0
    gdn_v_heads: int = 0
    gdn_head_dim: int = 128
    gdn_conv: int = 4
    # MTP draft head (number of extra decoder layers, 0 = none)
    mtp_layers: int = 0
    # shape of the draft layer: "dense" = plain attention + dense FFN in W8 whatever the model
    # is; "model" = the shape of the model's own full-attention layers (gated attention where
    # the model has it, routed experts where the model has them), which is what checkpoints
    # of the expert and hybrid families carry
    draft_layer: str = "dense"
    max_context: int = 32768
    # Encoder families (embedding models): every token attends to the whole input.  Such a
    # model serves /v1/embeddings through ``Engine.encode``; it does not generate.
    bidirectional: bool = False
    pooling: str = "mean"          # "mean" | "last" | "first"

    def __post_init__(self):
        if self.pooling not in ("mean", "last", "first"):
            raise ValueError("pooling must be mean, last or first")
        if self.bidirectional and self.arch == "hybrid":
            raise ValueError("recurrent (gated-delta-rule) layers cannot run bidirectionally")
        if self.q_heads % max(self.kv_heads, 1):
            raise ValueError("q_heads must be a multiple of kv_heads")
        for dim in (self.hidden, self.ffn or 128, self.expert_ffn or 128,
                    self.q_heads * self.head_dim):
            if dim % 128:
                raise ValueError(f"dimension {dim} must be a multiple of 128 (block rotation)")
        if self.head_dim % KV_GROUP:
            raise ValueError("head_dim must be a multiple of 64 (INT8-KV scale groups)")

    @property
    def q_dim(self) -> int:
        return self.q_heads * self.head_dim * (2 if self.gated_attention else 1)

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim

    def is_full_attention(self, layer: int) -> bool:
        if self.arch != "hybrid" or self.gdn_period <= 1:
            return True
        return layer % self.gdn_period == self.gdn_period - 1

    def kv_bytes_per_token(self) -> int:
        """INT8 K+V plus FP16 group scales over all full-attention layers."""
        full = sum(self.is_full_attention(i) for i in range(self.layers)) + self.mtp_layers
        per = 2 * self.kv_dim + 2 * 2 * (self.kv_dim // KV_GROUP)
        return full * per

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self), sort_keys=True)

    @classmethod
    def from_json(cls, text: str) -> "ModelConfig":
        return cls(**json.loads(text))


# Named geometries of the benchmark configurations.
PRESETS = {
    "tiny": ModelConfig(),
    "tiny-embed": ModelConfig(name="tiny-embed", bidirectional=True, pooling="mean"),
    "tiny-moe": ModelConfig(name="tiny-moe", arch="moe", experts=8, top_k=2, expert_ffn=128,
                            ffn=0),
    "tiny-hybrid": ModelConfig(name="tiny-hybrid", arch="hybrid", layers=4, gdn_period=4,
                               gdn_k_heads=2, gdn_v_heads=4, gdn_head_dim=64, experts=8, top_k=2,
                               expert_ffn=128, shared_expert_ffn=128, ffn=0, gated_attention=True,
                               expert_format="q2"),
    # mid-size geometry for multi-GPU tests: splits over 2, 4 and 8 ranks, and is large
    # enough that split-K, tail-peeled and sequence-parallel GEMM launches all occur
    "mid-dense": ModelConfig(name="mid-dense", layers=4, hidden=1024, q_heads=16, kv_heads=8,
                             head_dim=64, ffn=4096, vocab=8192),
    "qwen3.5-4b-class": ModelConfig(
        name="qwen3.5-4b-class", layers=36, hidden=2560, q_heads=32, kv_heads=8, head_dim=128,
        ffn=9728, vocab=151936, tied_embeddings=True, mtp_layers=1),
    "27b-class": ModelConfig(
        name="27b-class", layers=64, hidden=5120, q_heads=40, kv_heads=8, head_dim=128,
        ffn=20480, vocab=151936, tied_embeddings=False, mtp_layers=1),
    "35b-a3b-class": ModelConfig(
        name="35b-a3b-class", arch="moe", layers=48, hidden=2048, q_heads=32, kv_heads=4,
        head_dim=128, ffn=0, vocab=151936, tied_embeddings=False, experts=128, top_k=8,
        expert_ffn=768, attn_format="w8", expert_format="q4"),
    "80b-a3b-class": ModelConfig(
        name="80b-a3b-class", arch="hybrid", layers=48, hidden=2048, q_heads=16, kv_heads=2,
        head_dim=256, ffn=0, vocab=151936, tied_embeddings=False, experts=512, top_k=10,
        expert_ffn=512, shared_expert_ffn=512, expert_format="q2", gdn_period=4,
        gdn_k_heads=16, gdn_v_heads=32, gdn_head_dim=128, gated_attention=True, mtp_layers=1),
}


@dataclass
class LoadOptions:
    cuda_graph: GraphMode = GraphMode.DECODE_ONLY
    verify_weights: bool = False
    load_workers: int = 0                 # 0 = auto (<= 4), hard limit 32
    prefix_cache_bytes: int = 4096 << 20
    kv_offload_bytes: int = 0
    mtp_drafts: Optional[int] = None      # None = auto, else 0..31
    prompt_lookup: bool = False
    resident_experts: int = 0
    tp: int = 1
    ep: int = 1

    def validate(self) -> None:
        if self.mtp_drafts is not None and not 0 <= self.mtp_drafts <= MAX_MTP_DRAFTS:
            raise ValueError(f"mtp_drafts must be within 0..{MAX_MTP_DRAFTS}")
        if not 0 <= self.load_workers <= 32:
            raise ValueError("load_workers must be within 0..32")


@dataclass
class SchedulerOptions:
    policy: Policy = Policy.LATENCY
    max_active: int = 32
    max_batch_tokens: int = 128
    max_speculative_tokens: int = 0
    prefill_budget_ms: float = 200.0
    target_tpot_ms: float = 400.0
    memory_reserve_bytes: int = 1 << 30
    prefill_chunk: int = 4096
    # Layered prefill: a prefill packet of at least ``layered_min_rows`` rows that runs while
    # requests are decoding is paused at ``prefill_stages - 1`` layer boundaries; the decoders
    # take a step at each pause (only the hidden rows and the FP32 residual stay live).
    prefill_stages: int = 1
    layered_min_rows: int = 1024

    def validate(self) -> None:
        if not 1 <= self.prefill_stages <= 16:
            raise ValueError("prefill_stages must be within 1..16")
        if not 1 <= self.max_active <= MAX_ACTIVE_LIMIT:
            raise ValueError("max_active must be within 1..128")
        if not 1 <= self.max_batch_tokens <= 1 << 20:
            raise ValueError("max_batch_tokens out of range")
        if self.prefill_budget_ms <= 0 or self.target_tpot_ms <= 0:
            raise ValueError("time budgets must be positive")
