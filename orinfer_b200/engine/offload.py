"""Host tier of the prefix cache: evicted KV pages move to pinned host memory and come back
on a later hit.

A page's record is every cached layer's INT8 K and V rows plus their FP16 group scales for
the 128 tokens of the page, held in one slot of a pinned slab per cached tensor, so a save or
a restore is one contiguous device<->host copy per layer tensor on the engine's stream.  The radix tree keeps the
node indexed while its page lives here (``RadixPrefixCache.set_host``); when the slab is
full the tree drops its least useful host-only leaves.  Plays the role of the reference's
host KV tier (crates/orinfer-engine/src/backend/kv/host.rs:5-375,
runtime/requests/prefix.rs offload / restore).
"""

from __future__ import annotations

from typing import List, Optional

import torch

from ..models.runner import KVPool


class HostKvStore:
    def __init__(self, kv: KVPool, capacity_bytes: int):
        self.kv = kv
        self._parts = [*kv.k, *kv.v, *kv.ks, *kv.vs]      # each [pages, 128, kv heads, ...]
        self.page_bytes = sum(p[0].numel() * p.element_size() for p in self._parts)
        self.slots = max(int(capacity_bytes // self.page_bytes), 0)
        self._cuda = kv.k[0].is_cuda
        self._slabs = []
        for p in self._parts:
            t = torch.empty((self.slots,) + tuple(p[0].shape), dtype=p.dtype)
            self._slabs.append(t.pin_memory() if self._cuda and self.slots else t)
        self._free: List[int] = list(range(self.slots - 1, -1, -1))
        self.saved = self.restored = 0

    @property
    def available(self) -> int:
        return len(self._free)

    def save(self, page: int) -> Optional[int]:
        """Copies device page ``page`` out; returns its handle, or None when full."""
        if not self._free:
            return None
        h = self._free.pop()
        for slab, part in zip(self._slabs, self._parts):
            slab[h].copy_(part[page], non_blocking=True)
        self.saved += 1
        return h

    def load(self, handle: int, page: int) -> None:
        """Copies the record ``handle`` into device page ``page`` (the handle stays valid)."""
        for slab, part in zip(self._slabs, self._parts):
            part[page].copy_(slab[handle], non_blocking=True)
        self.restored += 1

    def free(self, handle: int) -> None:
        self._free.append(handle)

    def sync(self) -> None:
        if self._cuda:
            torch.cuda.current_stream().synchronize()
