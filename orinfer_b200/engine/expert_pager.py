"""Bounded expert residency: ``resident`` of a layer's experts live in device memory, the rest
in pinned host memory, and a packet's routed experts are paged in before its expert GEMMs.

Per MoE layer the device holds two slot banks (gate_up and down) of ``resident`` experts and a
remap table ``expert id -> slot`` (-1 = not resident).  After the router has chosen the
experts of a packet:

1. the distinct expert ids are read back (one small synchronising copy: the launch sequence of
   the layer depends on them, which is why CUDA graphs are off while paging);
2. missing experts are copied host -> device into victim slots (free slot first, then the
   least recently used *probationary* expert, then the least recently used *protected* one;
   an expert is promoted to protected at its second use: segmented LRU), never evicting an
   expert the same packet needs;
3. the router's ids are rewritten to slot ids, so dispatch, the grouped GEMMs and the combine
   run unchanged on the slot banks.

A packet can touch at most ``rows x top_k`` experts, so the engine bounds packets to
``resident // top_k`` rows; ``page_in`` refuses a packet that needs more experts than slots.
Counterpart of the reference's ``--resident-experts N`` pager (per-layer SLRU over VMM pages,
SSD -> GPU on the route histogram, graphs forced off:
crates/orinfer-engine/src/backend/cuda/experts.rs:1-335).  Here the cold tier is pinned host
memory: a B200 node has no need to page from SSD for the models in scope.
"""

from __future__ import annotations

import dataclasses
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import torch

from ..models.weights import ExpertBank


class ExpertCapacityError(RuntimeError):
    """A packet routed to more distinct experts than there are resident slots."""


@dataclass
class PagerStatistics:
    lookups: int = 0          # (layer, packet) page-in calls
    hits: int = 0             # needed experts found resident
    misses: int = 0           # experts copied in
    evictions: int = 0
    bytes_in: int = 0

    def as_dict(self) -> dict:
        d = dataclasses.asdict(self)
        total = self.hits + self.misses
        d["hit_rate"] = self.hits / total if total else 0.0
        return d


def _pin(t: torch.Tensor) -> torch.Tensor:
    t = t.detach().to("cpu").contiguous()
    if torch.cuda.is_available():
        try:
            return t.pin_memory()
        except RuntimeError:
            return t
    return t


class _LayerResidency:
    """Slot banks, remap table and SLRU bookkeeping of one layer."""

    def __init__(self, up: ExpertBank, down: ExpertBank, resident: int, device):
        self.host = (self._host_bank(up), self._host_bank(down))
        self.experts, self.resident = up.experts, resident
        self.slots = tuple(self._slot_bank(b, resident, device) for b in self.host)
        self.slot_of: List[int] = [-1] * up.experts
        self.in_slot: List[int] = [-1] * resident
        self.free: List[int] = list(range(resident - 1, -1, -1))
        self.probation: "OrderedDict[int, None]" = OrderedDict()
        self.protected: "OrderedDict[int, None]" = OrderedDict()
        self.protected_cap = max(resident * 2 // 3, 1)
        self.remap_host = torch.full((up.experts,), -1, dtype=torch.int32)
        if torch.device(device).type == "cuda":
            self.remap_host = _pin(self.remap_host)
        self.remap = self.remap_host.to(device)
        self.histogram = [0] * up.experts
        self.bytes_per_expert = sum(b.codes[0].numel() * b.codes.element_size()
                                    + b.scale[0].numel() * b.scale.element_size()
                                    for b in self.host)

    @staticmethod
    def _host_bank(b: ExpertBank) -> ExpertBank:
        return ExpertBank(b.fmt, b.experts, b.n, b.k, _pin(b.codes), _pin(b.scale), b.signs,
                          None, b.base)

    @staticmethod
    def _slot_bank(b: ExpertBank, resident: int, device) -> ExpertBank:
        codes = torch.zeros((resident,) + tuple(b.codes.shape[1:]), dtype=b.codes.dtype,
                            device=device)
        scale = torch.zeros((resident,) + tuple(b.scale.shape[1:]), dtype=b.scale.dtype,
                            device=device)
        signs = None if b.signs is None else b.signs.to(device)
        return ExpertBank(b.fmt, resident, b.n, b.k, codes, scale, signs, None, 0)

    def _touch(self, e: int) -> None:
        if e in self.protected:
            self.protected.move_to_end(e)
            return
        if e in self.probation:                       # second use: promote
            del self.probation[e]
            self.protected[e] = None
            while len(self.protected) > self.protected_cap:
                old, _ = self.protected.popitem(last=False)
                self.probation[old] = None            # demoted, most recent of probation
            return
        self.probation[e] = None

    def _victim(self, keep: set) -> Tuple[int, int]:
        """-> (slot, evicted expert or -1)."""
        if self.free:
            return self.free.pop(), -1
        for seg in (self.probation, self.protected):
            for e in seg:
                if e not in keep:
                    del seg[e]
                    slot = self.slot_of[e]
                    self.slot_of[e] = -1
                    self.remap_host[e] = -1
                    return slot, e
        raise ExpertCapacityError("no evictable expert slot")

    def page_in(self, needed: Sequence[int], stats: PagerStatistics) -> None:
        if len(needed) > self.resident:
            raise ExpertCapacityError(
                f"packet routes to {len(needed)} experts of one layer but only {self.resident} "
                "are resident: lower the packet size or raise resident_experts")
        keep = set(needed)
        changed = False
        for e in needed:
            self.histogram[e] += 1
            if self.slot_of[e] >= 0:
                stats.hits += 1
                self._touch(e)
                continue
            slot, evicted = self._victim(keep)
            if evicted >= 0:
                stats.evictions += 1
            for host, dev in zip(self.host, self.slots):
                dev.codes[slot].copy_(host.codes[e], non_blocking=True)
                dev.scale[slot].copy_(host.scale[e], non_blocking=True)
            self.slot_of[e], self.in_slot[slot] = slot, e
            self.remap_host[e] = slot
            self._touch(e)
            stats.misses += 1
            stats.bytes_in += self.bytes_per_expert
            changed = True
        if changed:
            self.remap.copy_(self.remap_host, non_blocking=True)


class ExpertPager:
    def __init__(self, banks: Dict[int, Tuple[ExpertBank, ExpertBank]], resident: int, device):
        """``banks``: key (any hashable per layer) -> (gate_up bank, down bank) holding ALL of
        the layer's experts; they are moved to pinned host memory."""
        if resident < 1:
            raise ValueError("resident_experts must be positive")
        self.device = device
        self.stats = PagerStatistics()
        self.layers = {key: _LayerResidency(up, down, min(resident, up.experts), device)
                       for key, (up, down) in banks.items()}

    def resident_slots(self, key) -> int:
        return self.layers[key].resident

    def page_in(self, key, ids: torch.Tensor, rows: int):
        """``ids``: int32 [>= rows, top_k] expert ids from the router.  Makes every expert of the
        first ``rows`` rows resident and returns (gate_up slot bank, down slot bank, slot ids
        int32 [rows, top_k])."""
        layer = self.layers[key]
        live = ids[:rows]
        needed = torch.unique(live).cpu().tolist()            # synchronises
        self.stats.lookups += 1
        layer.page_in([int(e) for e in needed], self.stats)
        slot_ids = layer.remap.index_select(0, live.reshape(-1).long()).view(rows, -1)
        return layer.slots[0], layer.slots[1], slot_ids.contiguous()

    def route_histogram(self, key) -> List[int]:
        return list(self.layers[key].histogram)

    def device_bytes(self) -> int:
        return sum(l.bytes_per_expert * l.resident for l in self.layers.values())
