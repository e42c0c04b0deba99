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


def read_tensors(path, *, workers: Optional[int] = None, pin: bool = False,
                 digests: Optional[Dict[str, str]] = None
                 ) -> Tuple[Dict[str, torch.Tensor], Dict[str, str]]:
    """-> (tensors by name, ``__metadata__``).  With ``digests`` every listed tensor is
    verified; a mismatch raises ``WeightReadError`` naming the tensor."""
    L = _l()
    h = L.orinfer_st_open(str(path).encode())
    if not h:
        raise WeightReadError(f"{path}: {L.orinfer_st_error().decode()}")
    try:
        n = L.orinfer_st_count(h)
        name, dtype = ctypes.create_string_buffer(512), ctypes.create_string_buffer(8)
        shape, ndim = (c_longlong * 8)(), c_int()
        names, tensors = [], []
        for i in range(n):
            size = L.orinfer_st_info(h, i, name, 512, dtype, shape, ctypes.byref(ndim))
            dt = _DTYPES.get(dtype.value.decode())
            if size < 0 or dt is None:
                raise WeightReadError(f"{path}: unsupported tensor entry {i}")
            t = torch.empty([shape[j] for j in range(ndim.value)], dtype=dt)
            if t.numel() * t.element_size() != size:
                raise WeightReadError(f"{path}: {name.value.decode()} shape/extent mismatch")
            if pin and t.numel():
                t = t.pin_memory()
            names.append(name.value.decode())
            tensors.append(t)
        idx = (c_int * n)(*range(n))
        dst = (c_void_p * n)(*[t.data_ptr() for t in tensors])
        want = None
        if digests is not None:
            want = (c_char_p * n)(*[digests[k].encode() if k in digests else None for k in names])
        bad = L.orinfer_st_read(h, idx, dst, n, workers or auto_workers(), want)
        if bad:
            raise WeightReadError(f"SHA-256 mismatch for tensor {names[bad - 1]}")
        meta = {}
        buf = ctypes.create_string_buffer(4096)
        for key in ("codec", "layout", "rotation", "quant_method", "coefficients", "scale"):
            if L.orinfer_st_metadata(h, key.encode(), buf, 4096) >= 0:
                meta[key] = buf.value.decode()
        return dict(zip(names, tensors)), meta
    finally:
        L.orinfer_st_close(h)
