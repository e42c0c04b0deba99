"""Python face of the C++ radix prefix cache (``csrc/core/prefix_cache.cpp``)."""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_int, c_int32, c_int64, c_uint32, c_uint64, c_void_p
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np

from ._lib import lib


@dataclass
class PrefixStatistics:
    lookups: int = 0
    hit_tokens: int = 0
    miss_tokens: int = 0
    inserted: int = 0
    evicted: int = 0
    offloaded: int = 0
    restored: int = 0
    device_pages: int = 0
    host_pages: int = 0
    nodes: int = 0

    @property
    def hit_rate(self) -> float:
        total = self.hit_tokens + self.miss_tokens
        return self.hit_tokens / total if total else 0.0


class RadixPrefixCache:
    def __init__(self, page_tokens: int = 128):
        l = lib()
        l.orinfer_prefix_create.restype = c_void_p
        l.orinfer_prefix_create.argtypes = [c_int]
        l.orinfer_prefix_destroy.argtypes = [c_void_p]
        l.orinfer_prefix_match.argtypes = [c_void_p, POINTER(c_uint32), c_int, POINTER(c_uint64),
                                           c_int, c_int, POINTER(c_int32), POINTER(c_int32), c_int]
        l.orinfer_prefix_insert.argtypes = [c_void_p, POINTER(c_uint32), c_int, POINTER(c_uint64),
                                            POINTER(c_int32), c_int, POINTER(c_int32),
                                            POINTER(c_int32)]
        l.orinfer_prefix_release.argtypes = [c_void_p, POINTER(c_int32), c_int]
        l.orinfer_prefix_abandon.argtypes = [c_void_p, POINTER(c_int32), c_int]
        l.orinfer_prefix_evict.argtypes = [c_void_p, c_int, c_int, POINTER(c_int32),
                                           POINTER(c_int32)]
        l.orinfer_prefix_set_host.argtypes = [c_void_p, c_int32, c_int64]
        l.orinfer_prefix_host_handle.argtypes = [c_void_p, c_int32]
        l.orinfer_prefix_host_handle.restype = c_int64
        l.orinfer_prefix_restore.argtypes = [c_void_p, c_int32, c_int32]
        l.orinfer_prefix_drop_host.argtypes = [c_void_p, c_int, POINTER(c_int64)]
        l.orinfer_prefix_stats.argtypes = [c_void_p, POINTER(c_uint64)]
        self._l = l
        self.page_tokens = page_tokens
        self._h = c_void_p(l.orinfer_prefix_create(page_tokens))

    def __del__(self):
        if getattr(self, "_h", None):
            self._l.orinfer_prefix_destroy(self._h)
            self._h = None

    @staticmethod
    def _u32(tokens) -> np.ndarray:
        return np.ascontiguousarray(tokens, dtype=np.uint32)

    def match(self, tokens: Sequence[int], limit_tokens: Optional[int] = None,
              acquire: bool = True, media: Optional[Sequence[int]] = None
              ) -> Tuple[List[int], List[int]]:
        """-> (node ids, device pages or -1 when host-resident) of the longest cached prefix."""
        t = self._u32(tokens)
        cap = len(t) // self.page_tokens + 1
        ids = np.empty(cap, np.int32)
        pages = np.empty(cap, np.int32)
        m = None if media is None else np.ascontiguousarray(media, dtype=np.uint64)
        n = self._l.orinfer_prefix_match(
            self._h, t.ctypes.data_as(POINTER(c_uint32)), len(t),
            None if m is None else m.ctypes.data_as(POINTER(c_uint64)),
            len(t) if limit_tokens is None else limit_tokens, int(acquire),
            ids.ctypes.data_as(POINTER(c_int32)), pages.ctypes.data_as(POINTER(c_int32)), cap)
        return ids[:n].tolist(), pages[:n].tolist()

    def insert(self, tokens: Sequence[int], pages: Sequence[int],
               media: Optional[Sequence[int]] = None) -> Tuple[List[bool], List[int]]:
        """-> (adopted flag per full page, node ids)."""
        t = self._u32(tokens)
        pg = np.ascontiguousarray(pages, dtype=np.int32)
        adopted = np.zeros(len(pg), np.int32)
        ids = np.zeros(len(pg), np.int32)
        m = None if media is None else np.ascontiguousarray(media, dtype=np.uint64)
        n = self._l.orinfer_prefix_insert(
            self._h, t.ctypes.data_as(POINTER(c_uint32)), len(t),
            None if m is None else m.ctypes.data_as(POINTER(c_uint64)),
            pg.ctypes.data_as(POINTER(c_int32)), len(pg),
            adopted.ctypes.data_as(POINTER(c_int32)), ids.ctypes.data_as(POINTER(c_int32)))
        return [bool(x) for x in adopted[:n]], ids[:n].tolist()

    def release(self, node_ids: Sequence[int]) -> None:
        if not node_ids:
            return
        a = np.ascontiguousarray(node_ids, dtype=np.int32)
        self._l.orinfer_prefix_release(self._h, a.ctypes.data_as(POINTER(c_int32)), len(a))

    def abandon(self, node_ids: Sequence[int]) -> None:
        """Release of a match that was not used (deferred admission): also takes back the
        hits it counted."""
        if not node_ids:
            return
        a = np.ascontiguousarray(node_ids, dtype=np.int32)
        self._l.orinfer_prefix_abandon(self._h, a.ctypes.data_as(POINTER(c_int32)), len(a))

    def evict(self, want: int, to_host: bool = False) -> List[Tuple[int, int]]:
        ids = np.empty(max(want, 1), np.int32)
        pages = np.empty(max(want, 1), np.int32)
        n = self._l.orinfer_prefix_evict(self._h, want, int(to_host),
                                         ids.ctypes.data_as(POINTER(c_int32)),
                                         pages.ctypes.data_as(POINTER(c_int32)))
        return list(zip(ids[:n].tolist(), pages[:n].tolist()))

    def set_host(self, node_id: int, handle: int) -> None:
        self._l.orinfer_prefix_set_host(self._h, node_id, handle)

    def host_handle(self, node_id: int) -> int:
        return int(self._l.orinfer_prefix_host_handle(self._h, node_id))

    def restore(self, node_id: int, page: int) -> bool:
        return self._l.orinfer_prefix_restore(self._h, node_id, page) == 0

    def drop_host(self, want: int) -> List[int]:
        out = np.empty(max(want, 1), np.int64)
        n = self._l.orinfer_prefix_drop_host(self._h, want, out.ctypes.data_as(POINTER(c_int64)))
        return out[:n].tolist()

    def statistics(self) -> PrefixStatistics:
        out = (c_uint64 * 10)()
        self._l.orinfer_prefix_stats(self._h, out)
        return PrefixStatistics(*[int(v) for v in out])
