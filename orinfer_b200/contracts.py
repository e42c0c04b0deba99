"""Device, memory and model-family contracts shared by the engine, the loader and the tools.

Counterparts of the reference's SDK contracts (crates/orinfer-model-sdk/src/device.rs:9-196:
``Backend``, ``Target``, ``DeviceOwner`` generation tags, ``MemoryRange`` checked extents;
operators/gdn.rs:4-31 GDN execution policy; embedding.rs / reranking.rs / encoder_rows.rs
pooled-encoder specs; crates/orinfer-models/src/registry.rs:7-47 architecture -> factory with the
single compute policy ``int8_quality``).  There is one target here: ``sm_100a``.
"""

from __future__ import annotations

import enum
import itertools
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

TARGET = "sm_100a"
COMPUTE_POLICY = "int8_quality"


class ContractError(ValueError):
    pass


def parse_target(text: str) -> str:
    """The only execution target of this build; anything else is refused by name."""
    if text != TARGET:
        raise ContractError(f"unsupported target `{text}`: this build runs on {TARGET} only")
    return TARGET


class Dtype(str, enum.Enum):
    U8 = "u8"
    I8 = "i8"
    U16 = "u16"
    F16 = "f16"
    BF16 = "bf16"
    I32 = "i32"
    U32 = "u32"
    F32 = "f32"
    U64 = "u64"

    @property
    def bytes(self) -> int:
        return {"u8": 1, "i8": 1, "u16": 2, "f16": 2, "bf16": 2, "i32": 4, "u32": 4, "f32": 4,
                "u64": 8}[self.value]


_GENERATION = itertools.count(1)


@dataclass(frozen=True)
class DeviceOwner:
    """Who owns a device allocation: the ordinal alone cannot tell a restarted worker, or two
    sessions on one GPU, apart, so every owner gets a process-unique generation."""
    ordinal: int
    generation: int

    @classmethod
    def new(cls, ordinal: int) -> "DeviceOwner":
        return cls(int(ordinal), next(_GENERATION))

    def require(self, other: "DeviceOwner") -> None:
        if self != other:
            raise ContractError("device allocation belongs to a different device or session")


@dataclass(frozen=True)
class MemoryRange:
    """``[offset, offset + length)`` inside an allocation of ``capacity`` bytes; every
    constructor checks the extent, so holders of a range never re-check."""
    offset: int
    length: int
    capacity: int

    def __post_init__(self):
        if min(self.offset, self.length, self.capacity) < 0 or \
                self.offset + self.length > self.capacity or self.capacity >= 1 << 62:
            raise ContractError(f"memory range {self.offset}+{self.length} exceeds its "
                                f"allocation of {self.capacity} bytes")

    @property
    def end(self) -> int:
        return self.offset + self.length

    def slice(self, offset: int, length: int) -> "MemoryRange":
        if offset < 0 or length < 0 or offset + length > self.length:
            raise ContractError("sub-range outside its parent range")
        return MemoryRange(self.offset + offset, length, self.capacity)

    def rows(self, row_bytes: int, first: int, count: int) -> "MemoryRange":
        if row_bytes <= 0:
            raise ContractError("row size must be positive")
        return self.slice(first * row_bytes, count * row_bytes)

    def overlaps(self, other: "MemoryRange") -> bool:
        return self.length > 0 and other.length > 0 and \
            self.offset < other.end and other.offset < self.end

    def aligned(self, alignment: int) -> bool:
        return self.offset % alignment == 0


def disjoint(ranges: Sequence[MemoryRange]) -> bool:
    ordered = sorted((r for r in ranges if r.length), key=lambda r: r.offset)
    return all(a.end <= b.offset for a, b in zip(ordered, ordered[1:]))


# ------------------------------------------------------------------ GDN execution policy
class GdnPrefill(str, enum.Enum):
    SEQUENTIAL = "sequential"        # token-by-token scan (what the kernels here implement)
    CHUNKED = "chunked"              # chunkwise WY form


@dataclass(frozen=True)
class GdnDecode:
    """Dense: the state is rewritten every step.  Deferred: up to ``capacity`` rank-one updates
    are logged and applied in one pass."""
    deferred_capacity: int = 0

    def __post_init__(self):
        if not 0 <= self.deferred_capacity <= 64:
            raise ContractError("deferred GDN update capacity must be within 0..64")

    @property
    def dense(self) -> bool:
        return self.deferred_capacity == 0


@dataclass(frozen=True)
class GdnPolicy:
    prefill: GdnPrefill = GdnPrefill.SEQUENTIAL
    decode: GdnDecode = GdnDecode()

    def validate_supported(self) -> None:
        if self.prefill is not GdnPrefill.SEQUENTIAL or not self.decode.dense:
            raise ContractError("this build implements sequential prefill and dense decode for "
                                "gated-delta-rule layers")


# ------------------------------------------------------------------ speculation contract
@dataclass(frozen=True)
class MtpSpec:
    """What speculative decoding may do for a model.

    ``verification_widths``: row counts of one request's verification (verified token plus
    drafts) that the engine may choose from, ascending; ``batch_verification_tokens``: most
    rows of a verification packet over all requests; ``batch_draft_profiles``: request counts
    the draft head runs in one batched pass, ascending (a batch is padded up to the next
    profile and split when it exceeds the last); ``commit_always``: recurrent layers need a
    commit pass even when every draft was accepted; ``hidden_ring``: the draft head consumes
    the target's hidden rows of every prefill chunk before the ring is reused.
    (crates/orinfer-model-sdk/src/mtp.rs:20-70,280-300 of the reference.)"""
    max_drafts: int = 3
    verification_widths: Tuple[int, ...] = (2, 3, 4)
    batch_verification_tokens: int = 512
    batch_draft_profiles: Tuple[int, ...] = (1, 2, 4, 8, 16, 32, 64, 128)
    commit_always: bool = False
    hidden_ring: bool = True

    def __post_init__(self):
        if not 0 <= self.max_drafts <= 31:
            raise ContractError("max_drafts must be within 0..31")
        w = self.verification_widths
        if any(a >= b for a, b in zip(w, w[1:])) or any(not 2 <= x <= 32 for x in w):
            raise ContractError("verification widths must ascend within 2..32")
        if w and w[-1] > self.max_drafts + 1 and self.max_drafts:
            raise ContractError("a verification width exceeds max_drafts + 1")
        p = self.batch_draft_profiles
        if not p or p[0] < 1 or any(a >= b for a, b in zip(p, p[1:])):
            raise ContractError("batch draft profiles must be positive and strictly ascending")
        if self.batch_verification_tokens < (w[-1] if w else 1):
            raise ContractError("batch_verification_tokens cannot hold one request's round")

    @staticmethod
    def for_config(cfg, max_drafts: int, max_active: int, max_rows: int) -> "MtpSpec":
        """The contract the engine derives for a geometry and its serving options."""
        drafts = max(0, min(int(max_drafts), 31))
        widths = tuple(range(2, drafts + 2))
        profiles = tuple(b for b in (1, 2, 4, 8, 16, 32, 64, 128) if b < max_active) + (max_active,)
        return MtpSpec(max_drafts=drafts, verification_widths=widths,
                       batch_verification_tokens=max(max_rows, widths[-1] if widths else 1),
                       batch_draft_profiles=profiles,
                       commit_always=getattr(cfg, "arch", "") == "hybrid")

    def draft_capacity(self, requests: int) -> int:
        """Profile that holds ``requests`` draft rows, or the largest one when none does (the
        caller then drafts in several passes)."""
        for p in self.batch_draft_profiles:
            if p >= requests:
                return p
        return self.batch_draft_profiles[-1]

    def width_allowed(self, width: int, requests: int) -> bool:
        return (width in self.verification_widths
                and width * requests <= self.batch_verification_tokens)


# ------------------------------------------------------------------ pooled-encoder specs
@dataclass(frozen=True)
class EmbeddingSpec:
    dimensions: int
    max_tokens: int = 32768
    max_items: int = 128
    query_prefix: str = "query: "
    document_prefix: str = "passage: "
    normalize: bool = True

    def output_dimensions(self, requested: Optional[int]) -> int:
        if requested is None:
            return self.dimensions
        if not isinstance(requested, int) or not 1 <= requested <= self.dimensions:
            raise ContractError("`dimensions` is outside 1..hidden size")
        return requested


@dataclass(frozen=True)
class RerankSpec:
    yes_token: int
    no_token: int
    max_documents: int = 128
    max_tokens: int = 32768

    def score(self, logits) -> float:
        """Unsaturated relevance: the yes logit minus the no logit."""
        return float(logits[self.yes_token] - logits[self.no_token])


def encoder_rows(lengths: Sequence[int], capacity: int) -> List[Tuple[int, int]]:
    """Pack independent encoder inputs into one packet: (first row, rows) per input, in
    order, refusing a packet beyond ``capacity`` rows or an empty input."""
    out, at = [], 0
    for n in lengths:
        if n <= 0:
            raise ContractError("empty encoder input")
        out.append((at, n))
        at += n
    if at > capacity:
        raise ContractError(f"encoder packet of {at} rows exceeds its capacity of {capacity}")
    return out


# ------------------------------------------------------------------ model registry
_REGISTRY: Dict[str, Callable] = {}


def register(architecture: str, factory: Callable) -> None:
    if architecture in _REGISTRY:
        raise ContractError(f"architecture `{architecture}` is registered twice")
    _REGISTRY[architecture] = factory


def architectures() -> List[str]:
    return sorted(_REGISTRY)


def create(architecture: str, compute_policy: str, *args, **kw):
    """Build the model family registered for ``architecture``; the only compute policy is
    ``int8_quality`` (INT8 tensor-core products with exact INT32 accumulation)."""
    if compute_policy != COMPUTE_POLICY:
        raise ContractError(f"unsupported compute policy `{compute_policy}`")
    factory = _REGISTRY.get(architecture)
    if factory is None:
        raise ContractError(f"unknown architecture `{architecture}`; known: "
                            + ", ".join(architectures()))
    return factory(*args, **kw)


for _arch in ("dense", "moe", "hybrid"):
    register(f"orinfer_b200.{_arch}", lambda cfg, _a=_arch: cfg if cfg.arch == _a else
             (_ for _ in ()).throw(ContractError(
                 f"config.json describes `{cfg.arch}`, the descriptor says `{_a}`")))
