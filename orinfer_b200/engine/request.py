"""Per-request state of the continuous engine.

Mirrors the fields of the reference's ``RequestCore``
(crates/orinfer-engine/src/model/request.rs:10-38): input, history (= input then
generated), limit, sampling options, prefill cursor, generated count, timing
marks; ``finished = generated == limit or released or stop token``.
"""

from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional

from ..core.sampling import SamplingOptions


class Phase(enum.Enum):
    WAITING = 0
    PREFILL = 1
    DECODE = 2
    FINISHED = 3


@dataclass
class MediaSpan:
    """Encoder features bound to the placeholder run ``[start, end)`` of a prompt."""
    start: int
    end: int
    features: object                          # tensor [end - start, hidden]
    digest: int                               # content hash (prefix-cache identity)


@dataclass
class Request:
    rid: int
    prompt: List[int]
    max_new: int
    sampling: SamplingOptions = field(default_factory=lambda: SamplingOptions(temperature=0.0))
    stop_ids: tuple = ()
    ignore_eos: bool = False
    want_logprobs: bool = False
    cache_prompt: bool = True
    constraint: Optional[object] = None       # grammar / thinking-budget decoder (host)
    on_token: Optional[Callable] = None
    media: List[MediaSpan] = field(default_factory=list)
    rope_positions: Optional[object] = None   # int32 [3, len(prompt)] when media shift RoPE
    rope_delta: int = 0                       # rotary position of token i >= len(prompt): i + delta
    # runtime
    phase: Phase = Phase.WAITING
    slot: int = -1                            # row of the device page table
    pages: List[int] = field(default_factory=list)
    offset: int = 0                           # tokens whose KV is in the cache
    cached_tokens: int = 0                    # prefix-cache hit length
    snapshots: dict = field(default_factory=dict)   # position -> recurrent state copy (hybrid)
    generated: List[int] = field(default_factory=list)
    logprobs: List[object] = field(default_factory=list)
    pending: int = -1                         # sampled token not yet fed to the model
    finish_reason: Optional[str] = None
    cancelled: bool = False
    arrived: float = field(default_factory=time.monotonic)
    first_token_at: Optional[float] = None
    finished_at: Optional[float] = None
    last_prefill_at: Optional[float] = None
    error: Optional[str] = None

    @property
    def history(self) -> List[int]:
        return self.prompt + self.generated

    @property
    def remaining_prefill(self) -> int:
        return len(self.prompt) - self.offset

    @property
    def finished(self) -> bool:
        return self.phase is Phase.FINISHED

    def page_media(self, page_tokens: int, pages: int) -> Optional[List[int]]:
        """Per page, a hash of the media whose spans overlap it (0 = none); None without
        media.  The prefix cache keys pages by (tokens, this value), so equal placeholder
        runs of different images never share KV."""
        if not self.media:
            return None
        out = [0] * pages
        for m in self.media:
            for pg in range(m.start // page_tokens, min(pages, (m.end - 1) // page_tokens + 1)):
                out[pg] = (out[pg] * 0x9E3779B97F4A7C15 + m.digest + 1) & 0xFFFFFFFFFFFFFFFF
        return out

    def context_needed(self) -> int:
        return len(self.prompt) + self.max_new
