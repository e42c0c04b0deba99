"""Expert parallelism with sharded tokens: dispatch all-to-all -> grouped expert GEMM ->
combine all-to-all, every transfer a push kernel over CUDA-IPC peer memory
(``csrc/kernels/moe_a2a.cu``).

A rank owns ``rows`` tokens and ``experts / world`` experts.  ``forward`` routes the owned
tokens' quantised rows to the ranks owning their experts, runs the grouped gate_up / SwiGLU /
down GEMMs over what it received for its own experts, returns the result rows to their
senders and combines ``top_k`` returned rows per owned token.  Bytes over NVLink per rank:
``rows * top_k * (K + 8)`` out and ``rows * top_k * 2H`` back, instead of the
``(world - 1) * rows_total * 2H`` of the replicated-token form.  NCCL is only used once, to
exchange the IPC handles.
"""

from __future__ import annotations

import ctypes
from ctypes import c_int, c_void_p
from typing import Optional

import torch
import torch.distributed as dist

from ..models.weights import ExpertBank
from ..ops import functional as F
from ..ops import native
from ..ops.native import check, count_launches, ptr, stream
from .fused import _DeviceView


class _Dispatch(ctypes.Structure):
    _fields_ = [("rows", c_void_p * 8), ("scale", c_void_p * 8), ("expert", c_void_p * 8),
                ("header", c_void_p * 8), ("flag", c_void_p * 8), ("sent", c_void_p),
                ("ticket", c_void_p), ("tp", c_int), ("rank", c_int), ("cap", c_int)]


class _Return(ctypes.Structure):
    _fields_ = [("ret", c_void_p * 8), ("flag", c_void_p * 8), ("sent", c_void_p),
                ("ticket", c_void_p), ("tp", c_int), ("rank", c_int), ("cap", c_int)]


def _align(n: int) -> int:
    return (n + 255) // 256 * 256


class ExpertA2A:
    def __init__(self, gate_up: ExpertBank, down: ExpertBank, experts_total: int, top_k: int,
                 max_rows: int, group=None):
        """``gate_up`` / ``down`` fix the geometry (and are the default banks of ``forward``);
        layers sharing that geometry share one instance and pass their own banks."""
        lib = native.lib()
        lib.orinfer_peer_alloc.restype = c_void_p
        lib.orinfer_peer_alloc.argtypes = [ctypes.c_size_t]
        lib.orinfer_peer_export.argtypes = [c_void_p, c_void_p]
        lib.orinfer_peer_import.argtypes = [c_void_p, ctypes.POINTER(c_void_p)]
        lib.orinfer_peer_unmap.argtypes = [c_void_p]
        lib.orinfer_peer_free.argtypes = [c_void_p]
        P, I = c_void_p, c_int
        lib.orinfer_a2a_dispatch_push.argtypes = [P, P, P, P, P, I, I, I, I,
                                                  ctypes.POINTER(_Dispatch), P]
        lib.orinfer_a2a_recv_prepare.argtypes = [P, P, P, P, I, I, P]
        lib.orinfer_a2a_return_push.argtypes = [P, P, P, I, ctypes.POINTER(_Return), P]
        lib.orinfer_a2a_wait.argtypes = [P, P, I, P]
        self.lib = lib
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.gate_up, self.down = gate_up, down
        self.experts_total, self.top_k = experts_total, top_k
        self.local_experts = gate_up.experts
        if self.local_experts * self.world != experts_total:
            raise ValueError("experts must split evenly over the ranks for the all-to-all form")
        self.k, self.h, self.ffn = gate_up.k, down.n, gate_up.n // 2
        dev = gate_up.codes.device
        self.device = dev
        tp, cap = self.world, max_rows * top_k
        self.cap = cap
        sizes = [("rows", tp * cap * self.k), ("scale", tp * cap * 4), ("expert", tp * cap * 4),
                 ("header", tp * 2 * 4), ("flag_d", 256), ("ret", cap * self.h * 2),
                 ("flag_r", 256)]
        off, self.off = 0, {}
        for name, n in sizes:
            self.off[name] = off
            off += _align(n)
        self.base = lib.orinfer_peer_alloc(off)
        if not self.base:
            raise native.KernelError(f"cannot allocate {off} bytes of peer memory")
        handle = (ctypes.c_ubyte * 64)()
        check(lib.orinfer_peer_export(self.base, handle), "peer_export")
        handles = [None] * tp
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.bases, self._mapped = [], []
        for r, hnd in enumerate(handles):
            if r == self.rank:
                self.bases.append(int(self.base))
                continue
            out = c_void_p()
            check(lib.orinfer_peer_import((ctypes.c_ubyte * 64).from_buffer_copy(hnd),
                                          ctypes.byref(out)), "peer_import")
            self.bases.append(int(out.value))
            self._mapped.append(out.value)
        self.local = torch.zeros(8, dtype=torch.int32, device=dev)       # sent/ticket x 2
        lp = self.local.data_ptr()
        d, rt = _Dispatch(), _Return()
        for r in range(8):
            b = self.bases[r] if r < tp else None
            d.rows[r] = b + self.off["rows"] if b else None
            d.scale[r] = b + self.off["scale"] if b else None
            d.expert[r] = b + self.off["expert"] if b else None
            d.header[r] = b + self.off["header"] if b else None
            d.flag[r] = b + self.off["flag_d"] if b else None
            rt.ret[r] = b + self.off["ret"] if b else None
            rt.flag[r] = b + self.off["flag_r"] if b else None
        d.sent, d.ticket, d.tp, d.rank, d.cap = lp, lp + 4, tp, self.rank, cap
        rt.sent, rt.ticket, rt.tp, rt.rank, rt.cap = lp + 8, lp + 12, tp, self.rank, cap
        self.d, self.r = d, rt
        mine = self.bases[self.rank]
        view = lambda name, shape, ts: torch.as_tensor(
            _DeviceView(mine + self.off[name], shape, ts), device=dev)
        self.recv_rows = view("rows", (tp * cap, self.k), "|i1")
        self.recv_scale = view("scale", (tp * cap,), "<f4")
        self.recv_expert = view("expert", (tp * cap, 1), "<i4")
        self.ret = view("ret", (cap, self.h), "<f2")
        self._p = {n: mine + self.off[n] for n in ("header", "flag_d", "flag_r")}
        self.by_dst = F.MoeScratch(max_rows, top_k, tp, 16, 8, dev)     # numbering only
        self.by_expert = F.MoeScratch(tp * cap, 1, self.local_experts, self.k, self.ffn, dev)
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def forward(self, q8: torch.Tensor, scale: torch.Tensor, ids: torch.Tensor,
                probs: torch.Tensor, out: torch.Tensor, shared: Optional[torch.Tensor] = None,
                gate: Optional[torch.Tensor] = None, rows: Optional[int] = None,
                gate_up: Optional[ExpertBank] = None,
                down: Optional[ExpertBank] = None) -> torch.Tensor:
        """q8 int8 [R, K] / scale fp32 [R]: the owned tokens, normalised, rotated for the
        experts' gate_up and quantised; ids int32 [R, top_k] global expert ids; probs fp32.
        Writes fp16 ``out[R, H] = sum_k probs * expert(ids)(token) (+ gate * shared)``."""
        lib, tp, cap = self.lib, self.world, self.cap
        up = self.gate_up if gate_up is None else gate_up
        dn = self.down if down is None else down
        rows = q8.shape[0] if rows is None else rows
        if rows * self.top_k > cap:
            raise ValueError("more owned rows than the all-to-all buffers were sized for")
        s = stream()
        # 1. rank of every assignment among those bound for the same destination rank
        dst = torch.div(ids[:rows], self.local_experts, rounding_mode="floor").to(torch.int32)
        F.moe_dispatch(dst.contiguous(), None, None, tp, self.by_dst, rows)
        # 2. dispatch all-to-all
        check(lib.orinfer_a2a_dispatch_push(ptr(ids), ptr(self.by_dst.slots),
                                            ptr(self.by_dst.offsets), ptr(q8), ptr(scale), rows,
                                            self.top_k, self.k, self.local_experts,
                                            ctypes.byref(self.d), s), "a2a_dispatch_push")
        check(lib.orinfer_a2a_recv_prepare(self._p["flag_d"], self.d.sent, self._p["header"],
                                           ptr(self.recv_expert), tp, cap, s), "a2a_recv_prepare")
        # 3. local experts over everything received
        be, total = self.by_expert, tp * cap
        F.moe_dispatch(self.recv_expert, self.recv_rows, self.recv_scale, self.experts_total, be,
                       total, up.base, self.local_experts)
        F.qgemm_grouped(be.q8, be.scale, up.codes, up.scale, up.fmt, 2 * self.ffn, be.gate_up, be,
                        total)
        F.act_prep_limited(be.gate_up, dn.signs, be.offsets[self.local_experts:], swiglu=True,
                           rows=total, q_out=be.q8_mid, scale_out=be.scale_mid)
        F.qgemm_grouped(be.q8_mid, be.scale_mid, dn.codes, dn.scale, dn.fmt, self.h, be.down, be,
                        total)
        # 4. combine all-to-all
        check(lib.orinfer_a2a_return_push(ptr(be.down), ptr(be.slots), self._p["header"], self.h,
                                          ctypes.byref(self.r), s), "a2a_return_push")
        check(lib.orinfer_a2a_wait(self._p["flag_r"], self.r.sent, tp, s), "a2a_wait")
        count_launches(4)
        return F.moe_combine(self.ret, self.by_dst.slots, probs, shared, gate, out, rows)

    def close(self) -> None:
        for p in self._mapped:
            self.lib.orinfer_peer_unmap(p)
        self._mapped = []
        if self.base:
            self.lib.orinfer_peer_free(self.base)
            self.base = None
