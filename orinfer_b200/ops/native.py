"""ctypes binding of ``liborinfer_kernels.so`` (the sm_100a kernel library).

Kernels take raw device pointers plus the current CUDA stream, so launches made
inside ``torch.cuda.graph`` capture are recorded like any other.  There is no
PyTorch fallback: on a machine with a GPU a missing library is an error.
"""

from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_longlong, c_size_t, c_void_p
from pathlib import Path
from typing import Optional

import torch

_LIB_PATH = Path(__file__).resolve().parents[1] / "_native" / "liborinfer_kernels.so"
_lib: Optional[ctypes.CDLL] = None
_launches = 0           # kernels launched through this binding (for benchmark accounting)

FMT = {"w8": 0, "q4": 1, "q2": 2}


class KernelError(RuntimeError):
    pass


def _load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise KernelError(
            f"{_LIB_PATH} is missing: run `python -m orinfer_b200.ops.build` "
            "(there is no non-CUDA fallback for the device ops)")
    lib = ctypes.CDLL(str(_LIB_PATH))
    P, I = c_void_p, c_int
    sig = {
        "orinfer_init": ([], I),
        "orinfer_read_status": ([P], I),
        "orinfer_clear_status": ([], I),
        "orinfer_status_async": ([P, P], I),
        "orinfer_set_wait_limit_us": ([c_longlong], I),
        "orinfer_current_device": ([], I),
        "orinfer_qgemm_set_impl": ([I], I),
        "orinfer_qgemv_fused": ([I, I, P, P, P, P, c_float, I, P, P, P, P, P, P, P, I, I, I, P], I),
        "orinfer_e8p_basis_host": ([P], I),
        "orinfer_embed_w8": ([P, P, P, P, I, I, I, P], I),
        "orinfer_act_prep": ([P, P, P, P, P, P, P, I, I, c_float, I, I, P], I),
        "orinfer_rope_table": ([P, P, P, I, I, c_double, P], I),
        "orinfer_qk_rope_kv": ([P, P, P, P, P, P, P, P, I, I, I, I, I, I, c_float, I, P, P, P, P,
                                P, P, I, P], I),
        "orinfer_argmax_parts": ([I], I),
        "orinfer_argmax": ([P, I, I, P, P, P, P], I),
        "orinfer_qgemm": ([I, P, P, P, P, P, I, I, I, I, I, P], I),
        "orinfer_attention_scratch_bytes": ([I, I, I, I], c_size_t),
        "orinfer_attention": ([P, P, P, P, P, I, P, P, P, P, P, I, I, I, I, I, P, P], I),
        "orinfer_e8p_encode": ([P, P, c_longlong, P], I),
        "orinfer_router_topk": ([P, P, I, I, I, I, I, I, P, P, P, P], I),
        "orinfer_moe_dispatch": ([P, I, I, I, P, P, I, P, P, P, P, I, P, P, P, P], I),
        "orinfer_moe_combine": ([P, P, P, I, I, P, P, P, I, P], I),
        "orinfer_qgemm_grouped": ([I, P, P, P, P, P, I, I, I, I, P, P, I, P], I),
        "orinfer_moe_dispatch_ep": ([P, I, I, I, I, P, P, I, P, P, P, P, I, P, P, P, P], I),
        "orinfer_sample_topk": ([P, I, I, c_longlong, P, P, P, P, P, P, P], I),
        "orinfer_qgemm_launches": ([I, I, I, I, I], I),
        "orinfer_qgemm_launches_fmt": ([I, I, I, I, I, I], I),
        "orinfer_qgemm_set_variant": ([I, I, I, I, I, I, I, I], I),
        "orinfer_qgemm_clear_variants": ([], None),
        "orinfer_qgemm_plan": ([I, I, I, I, I, P], None),
        "orinfer_act_prep_limited": ([P, P, P, P, I, I, I, P, P], I),
        "orinfer_small_proj": ([P, P, P, I, I, I, P], I),
        "orinfer_gdn_conv": ([P, I, P, P, P, P, P, P, I, I, I, I, I, P, P, I], I),
        "orinfer_gdn_scan": ([P, P, P, P, P, I, P, P, I, I, I, P, P, P, P], I),
        "orinfer_gdn_commit": ([P, I, P, P, I, P, P, P, I, I, I, P, P, P], I),
        "orinfer_gdn_gated_norm": ([P, P, I, P, c_float, I, I, I, I, P, P], I),
        "orinfer_attention_prefill": ([P, P, P, I, I, I, P, I, P, P, P, P, P, I, I, I, I, P], I),
    }
    for name, (args, res) in sig.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, res
    _lib = lib
    return lib


def loaded() -> bool:
    try:
        _load()
        return True
    except (KernelError, OSError):
        return False


def has(symbol: str) -> bool:
    return loaded() and hasattr(_lib, symbol)


def lib() -> ctypes.CDLL:
    return _load()


def launches() -> int:
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(code: int, what: str) -> None:
    if code != 0:
        detail = "invalid argument" if code < 0 else f"cudaError {code}"
        raise KernelError(f"{what} failed: {detail} ({code})")


def init() -> None:
    check(_load().orinfer_init(), "orinfer_init")
    from ..tuning import tables
    tables.load_default()


def expect_device(device) -> None:
    """The library answers for the CUDA device that is current on the calling thread; refuse
    to go on when that is not the device the caller's tensors live on (kernels would run on
    one GPU with another GPU's pointers)."""
    want = torch.device(device)
    index = want.index if want.index is not None else torch.cuda.current_device()
    have = int(_load().orinfer_current_device())
    if have != index:
        raise KernelError(f"kernel library is bound to cuda:{have} on this thread but the "
                          f"tensors are on cuda:{index}: call torch.cuda.set_device first")


def read_status() -> int:
    """Synchronise and return the device status word (0 = no bounded wait ran out)."""
    buf = (c_int * 4)()
    check(_load().orinfer_read_status(buf), "orinfer_read_status")
    return int(buf[0])


def clear_status() -> None:
    check(_load().orinfer_clear_status(), "orinfer_clear_status")


def set_wait_limit_us(us: int) -> None:
    """How long a bounded device wait (peer flag, TMA / MMA barrier) spins before it records
    a status and returns; about one second by default."""
    check(_load().orinfer_set_wait_limit_us(int(us)), "orinfer_set_wait_limit_us")


class StatusReader:
    """Reads the device status word without a synchronisation of its own: ``enqueue()`` queues
    a 16-byte copy into pinned memory behind the work already on the current stream, and
    ``value()`` is valid once the caller has waited for that stream (which it does anyway to
    read the step's tokens)."""

    def __init__(self):
        self.buf = torch.zeros(4, dtype=torch.int32).pin_memory()

    def enqueue(self) -> None:
        check(_load().orinfer_status_async(self.buf.data_ptr(), stream()), "orinfer_status_async")

    def value(self) -> int:
        return int(self.buf[0])


def qgemm_set_impl(impl: int) -> None:
    """0: persistent tcgen05 GEMM kernel (default); 1: one tile per CTA."""
    check(_load().orinfer_qgemm_set_impl(int(impl)), "orinfer_qgemm_set_impl")


def basis_host() -> torch.Tensor:
    out = torch.empty(256, 8, dtype=torch.int8)
    check(_load().orinfer_e8p_basis_host(out.data_ptr()), "orinfer_e8p_basis_host")
    return out


def e8p_encode(x: torch.Tensor) -> torch.Tensor:
    assert x.is_cuda and x.dtype == torch.float32 and x.shape[-1] == 8 and x.is_contiguous()
    codes = torch.empty(x.shape[0], dtype=torch.int32, device=x.device)
    check(_load().orinfer_e8p_encode(x.data_ptr(), codes.data_ptr(), x.shape[0], stream()),
          "orinfer_e8p_encode")
    count_launches(1)
    return codes
