"""Python face of ``csrc/core/host_rows.cpp``: n-gram addressing, row shards and gather
plans, INT8 row stores in host memory, and the conditional-memory lookup built from them.

A conditional memory (PLE / Engram in the reference's Flash-Next and DSv4.1 models) is a very
large table of INT8 rows kept in host files.  For each token the last four committed tokens
are hashed into ``layers x 3 orders x heads`` row ids (``NgramHasher``); the rows are fetched
from the rank's shard (``Int8RowStore``, through a bounded cache or a resident copy),
dequantised and uploaded with the packet.  See the reference's
crates/orinfer-model-sdk/src/conditional_memory.rs and crates/orinfer-engine/src/host_rows.rs.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_int32, c_int64, c_uint8, c_uint32, c_uint64, c_void_p
from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np

from ._lib import lib


class HostRowError(ValueError):
    pass


_ready = False


def _l():
    global _ready
    L = lib()
    if not _ready:
        L.orinfer_rows_error.restype = c_char_p
        L.orinfer_ngram_create.restype = c_void_p
        L.orinfer_ngram_create.argtypes = [POINTER(c_uint32), c_int, c_uint32, POINTER(c_uint32),
                                           c_int, c_int, POINTER(c_int64), c_int]
        L.orinfer_ngram_destroy.argtypes = [c_void_p]
        L.orinfer_ngram_width.argtypes = [c_void_p]
        L.orinfer_ngram_hash.argtypes = [c_void_p, POINTER(c_uint32), c_int, POINTER(c_uint32),
                                         c_int, POINTER(c_int64), POINTER(c_uint8)]
        L.orinfer_row_shard.argtypes = [c_uint64, c_int, c_int, POINTER(c_uint64),
                                        POINTER(c_uint64)]
        L.orinfer_row_plan.argtypes = [POINTER(c_int64), c_int, c_uint64, c_int, c_int,
                                       POINTER(c_uint64), POINTER(c_int32), POINTER(c_int32)]
        L.orinfer_rows_open.restype = c_void_p
        L.orinfer_rows_open.argtypes = [c_char_p, c_uint64, c_uint64, c_uint64, c_uint64]
        L.orinfer_rows_close.argtypes = [c_void_p]
        L.orinfer_rows_enable_cache.restype = ctypes.c_longlong
        L.orinfer_rows_enable_cache.argtypes = [c_void_p, c_uint64]
        L.orinfer_rows_make_resident.argtypes = [c_void_p, c_uint64]
        L.orinfer_rows_is_resident.argtypes = [c_void_p]
        L.orinfer_rows_gather.argtypes = [c_void_p, POINTER(c_uint64), c_int, POINTER(c_uint8),
                                          c_uint64]
        L.orinfer_rows_stats.argtypes = [c_void_p, POINTER(c_uint64)]
        _ready = True
    return L


def _err() -> str:
    return _l().orinfer_rows_error().decode()


def _ptr(a: np.ndarray, t):
    return a.ctypes.data_as(POINTER(t))


@dataclass
class HashLayer:
    layer: int                      # model layer the table feeds
    rows: int                       # table rows = sum of the bucket sizes
    multipliers: Sequence[int]      # 4 odd positive multipliers
    primes: Sequence[int]           # heads * 3 bucket sizes (orders 2, 3, 4)


class NgramHasher:
    """Deterministic n-gram addressing over explicit committed history."""

    def __init__(self, token_map: Sequence[int], pad_token: int, barriers: Sequence[int],
                 heads: int, layers: Sequence[HashLayer]):
        if len({l.layer for l in layers}) != len(layers):
            raise HostRowError("duplicate conditional-memory layer")
        for l in layers:
            if len(l.multipliers) != 4 or len(l.primes) != heads * 3:
                raise HostRowError("invalid conditional-memory layer geometry")
        tm = np.ascontiguousarray(token_map, dtype=np.uint32)
        br = np.ascontiguousarray(list(barriers) or [0], dtype=np.uint32)
        data = np.ascontiguousarray(
            [[l.rows, *l.multipliers, *l.primes] for l in layers], dtype=np.int64)
        self._h = _l().orinfer_ngram_create(_ptr(tm, c_uint32), len(tm), pad_token,
                                            _ptr(br, c_uint32), len(barriers), heads,
                                            _ptr(data, c_int64), len(layers))
        if not self._h:
            raise HostRowError(_err())
        self.layers = list(layers)
        self.heads = heads
        self.width = _l().orinfer_ngram_width(self._h)

    def __del__(self):
        if getattr(self, "_h", None):
            _l().orinfer_ngram_destroy(self._h)
            self._h = None

    def hash(self, history: Sequence[int], tokens: Sequence[int]) -> Tuple[np.ndarray, np.ndarray]:
        """(ids ``[tokens, layers, 3, heads]`` int64, valid ``[tokens]`` bool).  ``history`` is
        what was committed before ``tokens[0]``; only its last three entries are read."""
        hist = np.ascontiguousarray(list(history)[-3:] or [0], dtype=np.uint32)
        n_hist = min(3, len(history))
        tok = np.ascontiguousarray(tokens if len(tokens) else [0], dtype=np.uint32)
        out = np.zeros((len(tokens), self.width), dtype=np.int64)
        valid = np.zeros(max(1, len(tokens)), dtype=np.uint8)
        if _l().orinfer_ngram_hash(self._h, _ptr(hist, c_uint32), n_hist, _ptr(tok, c_uint32),
                                   len(tokens), _ptr(out, c_int64), _ptr(valid, c_uint8)):
            raise HostRowError(_err())
        return (out.reshape(len(tokens), len(self.layers), 3, self.heads),
                valid[:len(tokens)].astype(bool))


def row_shard(rows: int, ranks: int, rank: int) -> Tuple[int, int]:
    """(first row, row count) of ``rank``'s contiguous shard; spans are ceil(rows / ranks)."""
    first, count = c_uint64(), c_uint64()
    if _l().orinfer_row_shard(rows, ranks, rank, ctypes.byref(first), ctypes.byref(count)):
        raise HostRowError(_err())
    return first.value, count.value


@dataclass
class RowPlan:
    rows: np.ndarray       # unique rows grouped by owning rank
    restore: np.ndarray    # query i -> position in ``rows``
    starts: np.ndarray     # ranks + 1 offsets into ``rows``

    @classmethod
    def build(cls, ids, table_rows: int, ranks: int, max_queries: int = 1 << 20) -> "RowPlan":
        q = np.ascontiguousarray(ids, dtype=np.int64).reshape(-1)
        rows = np.zeros(max(1, q.size), dtype=np.uint64)
        restore = np.zeros(max(1, q.size), dtype=np.int32)
        starts = np.zeros(max(2, ranks + 1), dtype=np.int32)
        n = _l().orinfer_row_plan(_ptr(q if q.size else np.zeros(1, np.int64), c_int64), q.size,
                                  table_rows, ranks, max_queries, _ptr(rows, c_uint64),
                                  _ptr(restore, c_int32), _ptr(starts, c_int32))
        if n < 0:
            raise HostRowError(_err())
        return cls(rows[:n], restore[:q.size], starts[:ranks + 1])

    def for_rank(self, rank: int) -> np.ndarray:
        if not 0 <= rank < len(self.starts) - 1:
            raise HostRowError("host-row rank outside plan")
        return self.rows[self.starts[rank]:self.starts[rank + 1]]


class Int8RowStore:
    """Immutable rows of ``row_bytes`` bytes in a file, holding the global rows
    ``[first_row, first_row + rows)``."""

    def __init__(self, path, row_bytes: int, rows: int, first_row: int = 0, data_offset: int = 0,
                 cache_bytes: int = 0, resident_budget: int = 0):
        self._h = _l().orinfer_rows_open(str(path).encode(), data_offset, row_bytes, first_row,
                                         rows)
        if not self._h:
            raise HostRowError(_err())
        self.row_bytes, self.rows, self.first_row = row_bytes, rows, first_row
        self.cache_slots = 0
        if resident_budget:
            if _l().orinfer_rows_make_resident(self._h, resident_budget):
                raise HostRowError(_err())
        elif cache_bytes:
            self.cache_slots = _l().orinfer_rows_enable_cache(self._h, cache_bytes)
            if self.cache_slots < 0:
                raise HostRowError(_err())

    def close(self):
        if getattr(self, "_h", None):
            _l().orinfer_rows_close(self._h)
            self._h = None

    __del__ = close

    @property
    def resident(self) -> bool:
        return bool(_l().orinfer_rows_is_resident(self._h))

    def gather(self, ids, max_bytes: int = 1 << 30) -> np.ndarray:
        q = np.ascontiguousarray(ids, dtype=np.uint64).reshape(-1)
        out = np.empty((q.size, self.row_bytes), dtype=np.uint8)
        if q.size and _l().orinfer_rows_gather(self._h, _ptr(q, c_uint64), q.size,
                                               _ptr(out, c_uint8), max_bytes):
            raise HostRowError(_err())
        return out

    def stats(self) -> dict:
        v = (c_uint64 * 6)()
        _l().orinfer_rows_stats(self._h, v)
        return dict(zip(("hits", "misses", "gathered_rows", "gathered_bytes", "cache_slots",
                         "resident_bytes"), map(int, v)))


def write_int8_table(path, values: np.ndarray) -> int:
    """Quantise ``values`` [rows, dim] to INT8 rows with a trailing FP16 scale (dim + 2 bytes
    per row) and write them; returns the row size in bytes."""
    values = np.asarray(values, dtype=np.float32)
    scale = np.maximum(np.abs(values).max(axis=1), 1e-8) / 127.0
    scale16 = scale.astype(np.float16)
    q = np.clip(np.rint(values / scale16.astype(np.float32)[:, None]), -127, 127).astype(np.int8)
    rows = np.concatenate([q.view(np.uint8), scale16[:, None].view(np.uint8)], axis=1)
    with open(path, "wb") as f:
        f.write(rows.tobytes())
    return rows.shape[1]


def dequant_rows(raw: np.ndarray) -> np.ndarray:
    """Inverse of ``write_int8_table`` for gathered rows: [n, dim] float32."""
    dim = raw.shape[1] - 2
    scale = np.ascontiguousarray(raw[:, dim:]).view(np.float16).astype(np.float32)
    return raw[:, :dim].view(np.int8).astype(np.float32) * scale


class ConditionalMemory:
    """Per-packet lookup: hash -> unique-row plan -> gather from each rank's shard ->
    dequantise -> restore query order.  With ``ranks == 1`` this is the whole table; with
    more, ``stores[r]`` is rank r's shard and the caller moves only ``plan.for_rank(r)``
    rows between ranks."""

    def __init__(self, hasher: NgramHasher, layer_stores: List[List[Int8RowStore]]):
        if len(layer_stores) != len(hasher.layers):
            raise HostRowError("one store list per hashed layer is required")
        self.hasher = hasher
        self.stores = layer_stores

    def lookup(self, history: Sequence[int], tokens: Sequence[int]):
        """float32 ``[tokens, layers, 3 * heads, dim]`` (zero rows for media tokens), valid."""
        ids, valid = self.hasher.hash(history, tokens)
        out = []
        for l, stores in enumerate(self.stores):
            q = ids[:, l].reshape(-1)
            plan = RowPlan.build(q, self.hasher.layers[l].rows, len(stores))
            parts = [stores[r].gather(plan.for_rank(r)) for r in range(len(stores))]
            rows = dequant_rows(np.concatenate(parts, axis=0))[plan.restore]
            rows = rows.reshape(len(tokens), 3 * self.hasher.heads, -1)
            rows[~valid] = 0.0
            out.append(rows)
        return np.stack(out, axis=1), valid
