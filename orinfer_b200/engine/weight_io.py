"""Parallel safetensors reader over the C++ core (``csrc/core/weight_reader.cpp``).

``read_tensors`` indexes the file, allocates one host tensor per entry (pinned when the
weights are headed for a GPU, so the upload is a true asynchronous DMA), and lets
``workers`` C++ threads copy the mmap'd payload while optionally checking each tensor's
SHA-256 against the model descriptor.  Follows the reference's loader: N reader threads,
optional digest verification (crates/orinfer-engine/src/weights/read.rs,
backend/cuda/weight_upload.rs:1-330; ``LoadOptions.load_workers`` <= 32, auto <= 4).
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_int, c_longlong, c_void_p
from typing import Dict, Optional, Tuple

import torch

from ..core._lib import lib

_DTYPES = {"I8": torch.int8, "U8": torch.uint8, "I16": torch.int16, "I32": torch.int32,
           "I64": torch.int64, "F16": torch.float16, "BF16": torch.bfloat16,
           "F32": torch.float32, "F64": torch.float64, "BOOL": torch.bool}


class WeightReadError(ValueError):
    pass


def _l():
    L = lib()
    L.orinfer_st_open.restype = c_void_p
    L.orinfer_st_open.argtypes = [c_char_p]
    L.orinfer_st_close.argtypes = [c_void_p]
    L.orinfer_st_error.restype = c_char_p
    L.orinfer_st_count.argtypes = [c_void_p]
    L.orinfer_st_info.restype = c_longlong
    L.orinfer_st_info.argtypes = [c_void_p, c_int, c_char_p, c_int, c_char_p, POINTER(c_longlong),
                                  POINTER(c_int)]
    L.orinfer_st_metadata.argtypes = [c_void_p, c_char_p, c_char_p, c_int]
    L.orinfer_st_read.argtypes = [c_void_p, POINTER(c_int), POINTER(c_void_p), c_int, c_int,
                                  POINTER(c_char_p)]
    L.orinfer_sha256_hex.argtypes = [c_void_p, c_longlong, c_char_p]
    return L


def auto_workers() -> int:
    return max(1, min(4, (os.cpu_count() or 2) // 2))


def sha256_hex(t: torch.Tensor) -> str:
    t = t.contiguous()
    out = ctypes.create_string_buffer(65)
    _l().orinfer_sha256_hex(t.data_ptr(), t.numel() * t.element_size(), out)
    return out.value.decode()


ARENA_ALIGN = 256


def plan_arena(sizes, limit: int):
    """Offsets of the tensors that share the arena (those of at most ``limit`` bytes, each on
    a 256-byte boundary) and the arena's size: -> ([offset or None per tensor], total)."""
    offsets, total = [], 0
    for size in sizes:
        if size > limit:
            offsets.append(None)
            continue
        offsets.append(total)
        total += (size + ARENA_ALIGN - 1) // ARENA_ALIGN * ARENA_ALIGN
    return offsets, total


def plan_batches(sizes, budget: int):
    """File-order batches of tensor indices whose 256-byte aligned extents fit ``budget``
    bytes of staging (a tensor larger than the budget forms a batch of its own)."""
    batches, cur, used = [], [], 0
    for i, size in enumerate(sizes):
        need = (size + ARENA_ALIGN - 1) // ARENA_ALIGN * ARENA_ALIGN
        if cur and used + need > budget:
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def read_tensors(path, *, workers: Optional[int] = None, pin: bool = False,
                 digests: Optional[Dict[str, str]] = None, device=None,
                 staging_bytes: int = 512 << 20, arena_limit: int = 64 << 20,
                 staged: Optional[bool] = None
                 ) -> Tuple[Dict[str, torch.Tensor], Dict[str, str]]:
    """-> (tensors by name, ``__metadata__``).  With ``digests`` every listed tensor is
    verified; a mismatch raises ``WeightReadError`` naming the tensor.

    Without ``device`` every tensor is a host tensor of its own (pinned with ``pin``).  With
    ``device`` the tensors are created where they will live: those of at most ``arena_limit``
    bytes are views of ONE arena allocation (256-byte aligned), larger ones (embedding, expert
    banks) get allocations of their own so that they can be released one by one.  For a CPU
    device the reader threads write straight into them.  For a GPU (or with ``staged``) the
    file is walked in batches through two pinned staging buffers of ``staging_bytes / 2``
    each: while the reader threads fill one, the copies out of the other are still in flight,
    so pinned memory stays bounded whatever the size of the model."""
    L = _l()
    h = L.orinfer_st_open(str(path).encode())
    if not h:
        raise WeightReadError(f"{path}: {L.orinfer_st_error().decode()}")
    try:
        n = L.orinfer_st_count(h)
        name, dtype = ctypes.create_string_buffer(512), ctypes.create_string_buffer(8)
        shape, ndim = (c_longlong * 8)(), c_int()
        names, shapes, dtypes, sizes = [], [], [], []
        for i in range(n):
            size = L.orinfer_st_info(h, i, name, 512, dtype, shape, ctypes.byref(ndim))
            dt = _DTYPES.get(dtype.value.decode())
            if size < 0 or dt is None:
                raise WeightReadError(f"{path}: unsupported tensor entry {i}")
            shp = [shape[j] for j in range(ndim.value)]
            count = 1
            for d in shp:
                count *= d
            if count * torch.empty(0, dtype=dt).element_size() != size:
                raise WeightReadError(f"{path}: {name.value.decode()} shape/extent mismatch")
            names.append(name.value.decode())
            shapes.append(shp)
            dtypes.append(dt)
            sizes.append(int(size))
        want = None
        if digests is not None:
            want = [digests[k].encode() if k in digests else None for k in names]

        def read(indices, pointers):
            m = len(indices)
            if not m:
                return
            idx = (c_int * m)(*indices)
            dst = (c_void_p * m)(*pointers)
            sub = None if want is None else (c_char_p * m)(*[want[i] for i in indices])
            bad = L.orinfer_st_read(h, idx, dst, m, workers or auto_workers(), sub)
            if bad:
                raise WeightReadError(f"SHA-256 mismatch for tensor {names[indices[bad - 1]]}")

        if device is None:
            tensors = []
            for shp, dt in zip(shapes, dtypes):
                t = torch.empty(shp, dtype=dt)
                tensors.append(t.pin_memory() if pin and t.numel() else t)
            read(list(range(n)), [t.data_ptr() for t in tensors])
        else:
            dev = torch.device(device)
            offsets, total = plan_arena(sizes, arena_limit)
            arena = torch.empty(total + ARENA_ALIGN, dtype=torch.uint8, device=dev)
            pad = -arena.data_ptr() % ARENA_ALIGN      # host allocations are only 64-byte aligned
            tensors = []
            for shp, dt, size, off in zip(shapes, dtypes, sizes, offsets):
                if off is None:
                    tensors.append(torch.empty(shp, dtype=dt, device=dev))
                else:
                    tensors.append(arena[pad + off:pad + off + size].view(dt).view(shp))
            if staged is None:
                staged = dev.type == "cuda"
            if not staged:
                read(list(range(n)), [t.data_ptr() for t in tensors])
            else:
                _read_staged(read, tensors, sizes, dev, staging_bytes)
        meta = {}
        buf = ctypes.create_string_buffer(4096)
        for key in ("codec", "layout", "rotation", "quant_method", "coefficients", "scale"):
            if L.orinfer_st_metadata(h, key.encode(), buf, 4096) >= 0:
                meta[key] = buf.value.decode()
        return dict(zip(names, tensors)), meta
    finally:
        L.orinfer_st_close(h)


def _read_staged(read, tensors, sizes, dev, staging_bytes: int) -> None:
    """Batches through two staging buffers; ``read(indices, pointers)`` fills host memory."""
    cuda = dev.type == "cuda"
    half = max(staging_bytes // 2, max(sizes, default=0) + ARENA_ALIGN, ARENA_ALIGN)
    half = (half + ARENA_ALIGN - 1) // ARENA_ALIGN * ARENA_ALIGN
    stages = []
    for _ in range(2):
        s = torch.empty(half, dtype=torch.uint8)
        stages.append(s.pin_memory() if cuda else s)
    busy = [None, None]                              # event of the copies out of each buffer
    for b, batch in enumerate(plan_batches(sizes, half)):
        stage = stages[b % 2]
        if busy[b % 2] is not None:
            busy[b % 2].synchronize()                # its previous copies have left the buffer
        offs, used = [], 0
        for i in batch:
            offs.append(used)
            used += (sizes[i] + ARENA_ALIGN - 1) // ARENA_ALIGN * ARENA_ALIGN
        read(batch, [stage.data_ptr() + o for o in offs])
        for i, o in zip(batch, offs):
            if sizes[i]:
                tensors[i].view(-1).view(torch.uint8).copy_(stage[o:o + sizes[i]],
                                                            non_blocking=cuda)
        if cuda:
            busy[b % 2] = torch.cuda.Event()
            busy[b % 2].record()
    if cuda:
        torch.cuda.current_stream().synchronize()
