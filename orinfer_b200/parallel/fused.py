"""Fused compute+collective tensor-parallel path over NVLink peer memory.

Every row-parallel projection (o_proj, down_proj) is ONE kernel that multiplies on the
tensor cores (or dp4a for decode batches) and, from its epilogue, stores its FP16 partial
tile straight into slot ``[rank]`` of every peer's inbox with plain peer stores; the last
CTA publishes a sequence number to the peers (release, system scope).  The all-reduce's
reduction is fused into the consumer: the following residual-add/RMSNorm/rotate/quantise
kernel waits (bounded) for the tp sequence flags and sums the tp partial rows in fixed
source order.  No NCCL call and no separate reduction kernel remains on that path; NCCL
(``TPRunner``) is kept as the baseline arm and for the tiny head merge.

Prefill packets (``rows >= SP_MIN_ROWS``, dense models) run sequence-parallel instead: the
GEMM epilogue stores each partial row only into its owner's inbox (reduce-scatter, 1/tp of
the bytes), the owner's norm kernel reduces, normalises, rotates and quantises ITS rows and
stores the INT8 rows + scales into every rank's activation buffer (all-gather by push, one
byte per element), and the following column-parallel GEMM waits per M tile for the source
ranks it needs before its first TMA load.  The FP32 residual stream stays row-sharded.

Buffers are cudaMalloc'd per rank and mapped into every peer with CUDA IPC handles
exchanged once at start-up (``csrc/kernels/peer_mem.cu``).  Counters live in device memory, so a
captured CUDA graph replays the protocol unchanged.  No TMA multicast is used anywhere;
peers are only ever written with ordinary ``st.global``.

Replaces collective call sites C1/C2 of the reference's TP8 plans (AllReduce after
``wo_b`` and after the FFN: python/orinfer_build/models/deepseek_v41/build.py:1086-1110,
1355-1364).
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_uint, c_void_p
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..models.runner import KVPool
from ..models.weights import ModelWeights, QLinear
from ..ops import native
from ..ops.native import FMT, check, count_launches, ptr, stream
from .tp_runner import TPRunner


def enabled() -> bool:
    return os.environ.get("ORINFER_TP_FUSED", "1") != "0"


class _PeerOut(ctypes.Structure):
    _fields_ = [("inbox", c_void_p * 8), ("flag", c_void_p * 8), ("sent", c_void_p),
                ("ticket", c_void_p), ("tp", c_int), ("rank", c_int), ("rows_cap", c_int),
                ("rows_per", c_int)]


class _AgOut(ctypes.Structure):
    _fields_ = [("q", c_void_p * 8), ("scale", c_void_p * 8), ("flag", c_void_p * 8),
                ("sent", c_void_p), ("ticket", c_void_p), ("tp", c_int), ("rank", c_int),
                ("rows_per", c_int)]


class _AgIn(ctypes.Structure):
    _fields_ = [("flag", c_void_p), ("sent", c_void_p), ("tp", c_int), ("rows_per", c_int)]


class _DeviceView:
    """Exposes a raw device range to torch through the CUDA array interface."""

    def __init__(self, address: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr,
                                         "data": (address, False), "version": 2}


SP_MIN_ROWS = int(os.environ.get("ORINFER_TP_SP_MIN_ROWS", "256"))


class _Inbox(ctypes.Structure):
    _fields_ = [("inbox", c_void_p), ("flag", c_void_p), ("seen", c_void_p),
                ("ticket", c_void_p), ("tp", c_int), ("rows_cap", c_int), ("ll", c_void_p)]


class _HeadMerge(ctypes.Structure):
    _fields_ = [("table", c_void_p * 8), ("seq", c_void_p), ("tp", c_int), ("rank", c_int),
                ("cap", c_int)]


HEAD_ROWS = 1024


LL_MODE, LL_ROWS = -1, 8


OPS = ("o", "down")


class PeerMemory:
    """One peer-mapped allocation per rank holding, per fused op, an inbox
    ``fp16 [tp][rows_cap][hidden]`` and a flag array ``int32 [tp]``; plus local sequence
    and ticket counters.  Handles are CUDA IPC handles exchanged with an object gather."""

    def __init__(self, hidden: int, rows_cap: int, group, device):
        lib = native.lib()
        lib.orinfer_peer_alloc.restype = c_void_p
        lib.orinfer_peer_alloc.argtypes = [ctypes.c_size_t]
        lib.orinfer_peer_export.argtypes = [c_void_p, c_void_p]
        lib.orinfer_peer_import.argtypes = [c_void_p, ctypes.POINTER(c_void_p)]
        lib.orinfer_peer_unmap.argtypes = [c_void_p]
        lib.orinfer_peer_free.argtypes = [c_void_p]
        self.lib = lib
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rows_cap = rows_cap
        inbox_bytes = self.world * rows_cap * hidden * 2
        inbox_bytes = (inbox_bytes + 255) // 256 * 256
        flag_bytes = 256
        ag_q_bytes = (rows_cap * hidden + 255) // 256 * 256
        ag_s_bytes = (rows_cap * 4 + 255) // 256 * 256
        ag_off = len(OPS) * (inbox_bytes + flag_bytes)
        # low-latency regions (decode-sized packets): units of {2 x fp16, sequence number}
        ll_bytes = (self.world * LL_ROWS * (hidden // 2) * 8 + 255) // 256 * 256
        ll_off = ag_off + ag_q_bytes + ag_s_bytes + flag_bytes
        head_off = ll_off + len(OPS) * ll_bytes        # greedy-token merge table [tp][rows][16 B]
        total = head_off + self.world * HEAD_ROWS * 16
        self.base = lib.orinfer_peer_alloc(total)
        if not self.base:
            raise native.KernelError(f"cannot allocate {total} bytes of peer memory")
        handle = (ctypes.c_ubyte * 64)()
        check(lib.orinfer_peer_export(self.base, handle), "peer_export")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        bases = []
        self._mapped = []
        for r, h in enumerate(handles):
            if r == self.rank:
                bases.append(int(self.base))
                continue
            out = c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            check(lib.orinfer_peer_import(buf, ctypes.byref(out)), "peer_import")
            bases.append(int(out.value))
            self._mapped.append(out.value)
        self.bases = bases
        self.local = torch.zeros(64, dtype=torch.int32, device=device)   # sent/seen/tickets
        lp = self.local.data_ptr()
        self.peer_out: Dict[str, _PeerOut] = {}
        self.inbox: Dict[str, _Inbox] = {}
        self.ll_out: Dict[str, _PeerOut] = {}
        self.ll_in: Dict[str, _Inbox] = {}
        for i, op in enumerate(OPS):
            off_inbox = i * (inbox_bytes + flag_bytes)
            off_flag = off_inbox + inbox_bytes
            po = _PeerOut()
            for r in range(8):
                po.inbox[r] = bases[r] + off_inbox if r < self.world else None
                po.flag[r] = bases[r] + off_flag if r < self.world else None
            po.sent = lp + (4 * i + 0) * 4
            po.ticket = lp + (4 * i + 1) * 4
            po.tp, po.rank, po.rows_cap = self.world, self.rank, rows_cap
            ib = _Inbox(bases[self.rank] + off_inbox, bases[self.rank] + off_flag,
                        lp + (4 * i + 2) * 4, lp + (4 * i + 3) * 4, self.world, rows_cap, None)
            self.peer_out[op], self.inbox[op] = po, ib
            # low-latency twin of the same op: own regions and counters
            lo = _PeerOut()
            for r in range(8):
                lo.inbox[r] = bases[r] + ll_off + i * ll_bytes if r < self.world else None
                lo.flag[r] = None
            lo.sent = lp + (40 + 4 * i + 0) * 4
            lo.ticket = lp + (40 + 4 * i + 1) * 4
            lo.tp, lo.rank, lo.rows_cap, lo.rows_per = self.world, self.rank, rows_cap, LL_MODE
            li = _Inbox(None, None, lp + (40 + 4 * i + 2) * 4, lp + (40 + 4 * i + 3) * 4,
                        self.world, rows_cap, bases[self.rank] + ll_off + i * ll_bytes)
            self.ll_out[op], self.ll_in[op] = lo, li
        hm = _HeadMerge()
        for r in range(8):
            hm.table[r] = bases[r] + head_off if r < self.world else None
        hm.seq = lp + 56 * 4
        hm.tp, hm.rank, hm.cap = self.world, self.rank, HEAD_ROWS
        self.head_merge = hm
        # all-gather activation buffer (INT8 rows + scales) and its flags
        ag = _AgOut()
        for r in range(8):
            ag.q[r] = bases[r] + ag_off if r < self.world else None
            ag.scale[r] = bases[r] + ag_off + ag_q_bytes if r < self.world else None
            ag.flag[r] = bases[r] + ag_off + ag_q_bytes + ag_s_bytes if r < self.world else None
        ag.sent, ag.ticket = lp + 32 * 4, lp + 33 * 4
        ag.tp, ag.rank, ag.rows_per = self.world, self.rank, 0
        self.ag_out = ag
        mine = bases[self.rank] + ag_off
        self.ag_in = _AgIn(mine + ag_q_bytes + ag_s_bytes, lp + 32 * 4, self.world, 0)
        self.ag_q = torch.as_tensor(_DeviceView(mine, (rows_cap, hidden), "|i1"), device=device)
        self.ag_scale = torch.as_tensor(_DeviceView(mine + ag_q_bytes, (rows_cap,), "<f4"),
                                        device=device)
        if self.ag_q.data_ptr() != mine:
            raise native.KernelError("activation buffer view does not alias peer memory")
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def close(self) -> None:
        for p in self._mapped:
            self.lib.orinfer_peer_unmap(p)
        self._mapped = []
        if self.base:
            self.lib.orinfer_peer_free(self.base)
            self.base = None


def _setup_lib():
    lib = native.lib()
    P, I = c_void_p, c_int
    lib.orinfer_qgemm_peer.argtypes = [I, P, P, P, P, ctypes.POINTER(_PeerOut), I, I, I, I, P]
    lib.orinfer_qgemm_peer.restype = I
    lib.orinfer_act_prep_inbox.argtypes = [ctypes.POINTER(_Inbox), P, P, P, P, P, P, I, I,
                                           ctypes.c_float, I, P]
    lib.orinfer_act_prep_inbox.restype = I
    lib.orinfer_moe_combine_peer.argtypes = [P, P, P, I, I, P, P, ctypes.POINTER(_PeerOut), I, P]
    lib.orinfer_moe_combine_peer.restype = I
    lib.orinfer_act_prep_sp.argtypes = [ctypes.POINTER(_Inbox), ctypes.POINTER(_AgOut), P, P, P,
                                        I, I, ctypes.c_float, I, P, P]
    lib.orinfer_act_prep_sp.restype = I
    lib.orinfer_act_prep_inbox_rows.argtypes = [ctypes.POINTER(_Inbox), P, P, P, P, P, P, I, I, I,
                                                ctypes.c_float, I, P]
    lib.orinfer_act_prep_inbox_rows.restype = I
    lib.orinfer_qgemm_ag.argtypes = [I, P, P, P, P, P, ctypes.POINTER(_AgIn), I, I, I, I, P]
    lib.orinfer_qgemm_ag.restype = I
    lib.orinfer_ag_wait.argtypes = [ctypes.POINTER(_AgIn), I, P]
    lib.orinfer_ag_wait.restype = I
    lib.orinfer_tp_head_merge.argtypes = [P, P, I, I, I, ctypes.POINTER(_HeadMerge), P, P]
    lib.orinfer_tp_head_merge.restype = I
    return lib


class FusedTPRunner(TPRunner):
    """Tensor-parallel runner whose row-parallel projections scatter their partial results
    to the peers from the GEMM epilogue and whose norm kernels reduce them."""

    def __init__(self, weights: ModelWeights, kv: KVPool, max_rows: int, group=None):
        super().__init__(weights, kv, max_rows, group)
        self.lib = _setup_lib()
        self.mem = PeerMemory(self.cfg.hidden, max_rows, group, self.device)
        self._sp_rows_per, self._sp_total = 0, 0
        self._ll = os.environ.get("ORINFER_TP_LL", "1") != "0"

    def close(self, collective: bool = True) -> None:
        """Unmaps the peers' buffers and frees this rank's (collective: every rank arrives at
        the barrier first, so nobody unmaps memory a peer's kernel may still write).
        ``collective=False`` is for leaving after a peer was lost: no barrier, the peers are
        not coming."""
        import torch.distributed as dist
        torch.cuda.synchronize()
        if collective and dist.is_initialized() and self.world > 1:
            dist.barrier(group=self.group)
        a2a = getattr(self, "_a2a", None)
        if a2a is not None and hasattr(a2a, "close"):
            a2a.close()
        self.mem.close()

    def greedy(self, p, logits_out=None, token_out=None, need_logits: bool = True):
        """The sharded head's greedy token through the peer tables (one small kernel, no
        collective call); full logits are still gathered with NCCL when a caller needs them."""
        from ..ops import functional as F
        local = self._last_local = self.logits(p)                      # [n_sel, V/tp]
        rows = local.shape[0]
        if rows > HEAD_ROWS or os.environ.get("ORINFER_TP_HEAD_MERGE", "1") == "0":
            return super().greedy(p, logits_out, token_out, need_logits)
        ltok = F.argmax(local)
        tok = token_out if token_out is not None else \
            torch.empty(rows, dtype=torch.int32, device=local.device)
        check(self.lib.orinfer_tp_head_merge(ptr(local), ptr(ltok), rows, local.shape[1],
                                             self.vocab0, ctypes.byref(self.mem.head_merge),
                                             ptr(tok), stream()), "tp_head_merge")
        count_launches(1)
        full = None
        if need_logits:
            full = self._gather_logits(local)
            if logits_out is not None:
                logits_out[:full.shape[0]].copy_(full)
                full = logits_out
        return tok, full

    _SLOT = {"o": "o", "gdn_out": "o", "down": "down"}

    # a paused forward would leave partial sums in the peers' inboxes while other packets use
    # them: layered prefill is for the single-GPU and NCCL runners
    supports_stages = False

    def forward_hidden(self, p):
        # sequence-parallel for prefill-sized packets of dense models; decode-sized packets
        # keep the one-hop all-reduce form (latency, not bytes, is what matters there)
        cfg = self.cfg
        self._sp_rows_per = 0
        if self.world > 1 or os.environ.get("ORINFER_TP_SP_WORLD1") == "1":
            dense = not cfg.experts and cfg.arch == "dense"
            moe = bool(cfg.experts) and cfg.arch == "moe" and cfg.experts % self.world == 0 \
                and os.environ.get("ORINFER_EP_A2A", "1") != "0"
            if p.rows >= SP_MIN_ROWS and (dense or moe):
                self._sp_rows_per = (p.rows + self.world - 1) // self.world
        self._sp_total = p.rows
        return super().forward_hidden(p)

    def _moe_ffn(self, lw, x, rows: int):
        """Prefill-sized packets of MoE models keep the tokens sharded: this rank normalises
        the rows it owns (completing the attention's reduce-scatter), routes them, sends each
        (row, expert) to the expert's owner, runs its own experts over what it received,
        returns the results and combines top-k rows per owned token.  The shared expert runs
        on the owned rows with its full weights."""
        rows_per = self._sp_rows_per if rows == self._sp_total else 0
        if not rows_per or not isinstance(x, tuple) or x[0] == "local":
            return super()._moe_ffn(lw, x, rows)
        from ..ops import functional as F
        from .ep_a2a import ExpertA2A
        cfg, ws = self.cfg, self.ws
        h, f = cfg.hidden, cfg.expert_ffn
        base = self.tp.rank * rows_per
        cnt = min(rows_per, rows - base)
        if cnt <= 0:
            raise native.KernelError("a rank owns no rows of a sequence-parallel packet")
        bank_up, bank_dn = lw.expert_gate_up, lw.expert_down
        cap_rows = (ws.max_rows + self.world - 1) // self.world
        if getattr(self, "_a2a", None) is None:
            self._a2a = ExpertA2A(bank_up, bank_dn, cfg.experts, cfg.top_k, cap_rows, self.group)
            e = lambda *s_, dt: torch.empty(*s_, dtype=dt, device=self.device)
            self._a2a_buf = dict(ids=e(cap_rows, cfg.top_k, dt=torch.int32),
                                 probs=e(cap_rows, cfg.top_k, dt=torch.float32),
                                 gate=e(cap_rows, dt=torch.float32),
                                 shared=e(cap_rows, h, dt=torch.float16),
                                 q8s=e(cap_rows, max(cfg.shared_expert_ffn, 16), dt=torch.int8))
        b = self._a2a_buf
        y16 = ws.attn_norm(rows, h)
        q8, sc = ws.q8[h], ws.scale
        ib = self.mem.inbox[x[0]]
        check(self.lib.orinfer_act_prep_inbox_rows(
            ctypes.byref(ib), ptr(ws.resid), ptr(lw.post_norm), ptr(bank_up.signs), ptr(q8),
            ptr(sc), ptr(y16), base, cnt, h, float(cfg.eps), int(cfg.zero_centered_norm),
            stream()), "act_prep_inbox_rows")
        count_launches(1)
        q8o, sco, y16o = q8[base:base + cnt], sc[base:base + cnt], y16[base:base + cnt]
        F.router_topk(y16o, lw.router, cfg.experts, cfg.top_k, renorm=cfg.renormalize, rows=cnt,
                      ids=b["ids"], probs=b["probs"], gate=b["gate"])
        shared = None
        if lw.shared_gate_up is not None:
            fs = lw.shared_gate_up.n // 2
            gu = self._linear(lw.shared_gate_up, q8o, sco, cnt,
                              ws.gate_up.view(-1)[: ws.max_rows * 2 * fs].view(ws.max_rows, 2 * fs))
            q8s, s8s = F.act_prep(gu, None, None, self._signs(lw.shared_down), swiglu=True,
                                  rows=cnt, q_out=b["q8s"], scale_out=ws.scale_alt(cnt))
            shared = self._linear(lw.shared_down, q8s, s8s, cnt, b["shared"])
        has_gate = lw.router.shape[0] == cfg.experts + 1
        self._a2a.forward(q8o, sco, b["ids"], b["probs"], ws.hidden[base:base + cnt], shared,
                          b["gate"] if has_gate and shared is not None else None, rows=cnt,
                          gate_up=bank_up, down=bank_dn)
        return ("local", rows_per)

    def _moe_combine(self, sc, shared, gate, rows: int):
        """Expert-parallel combine fused with the scatter half of the all-reduce: the kernel
        that sums this rank's expert rows stores the partial row into every peer's inbox."""
        po = self.mem.peer_out["down"]
        check(self.lib.orinfer_moe_combine_peer(ptr(sc.down), ptr(sc.slots), ptr(sc.probs), rows,
                                                sc.probs.shape[1], ptr(shared), ptr(gate),
                                                ctypes.byref(po), self.cfg.hidden, stream()),
              "moe_combine_peer")
        count_launches(1)
        return "down"

    def mtp_rows(self, tokens, hidden, p):
        """The draft layer's two row-parallel projections are reduced with plain all-reduces
        (the peer inboxes belong to the model's own layers and their sequence counters)."""
        self._plain_reduce = True
        try:
            return super().mtp_rows(tokens, hidden, p)
        finally:
            self._plain_reduce = False

    _plain_reduce = False

    def _row_parallel(self, name: str, lin: QLinear, q8, sc, rows: int):
        if self._plain_reduce:
            return TPRunner._row_parallel(self, name, lin, q8, sc, rows)
        name = self._SLOT[name]
        if rows <= LL_ROWS and lin.fmt != "w8" and lin.n % 16 == 0 and self._ll:
            # decode-sized: data and readiness travel in the same 8-byte units
            po = self.mem.ll_out[name]
            check(self.lib.orinfer_qgemm_peer(FMT[lin.fmt], ptr(q8), ptr(sc), ptr(lin.codes),
                                              ptr(lin.scale), ctypes.byref(po), rows, lin.n,
                                              lin.k, 0, stream()), "qgemm_peer_ll")
            count_launches(1)
            return (name, LL_MODE)
        po = self.mem.peer_out[name]
        po.rows_per = self._sp_rows_per if rows == self._sp_total else 0
        check(self.lib.orinfer_qgemm_peer(FMT[lin.fmt], ptr(q8), ptr(sc), ptr(lin.codes),
                                          ptr(lin.scale), ctypes.byref(po), rows, lin.n, lin.k, 0,
                                          stream()), "qgemm_peer")
        count_launches(1)
        return (name, po.rows_per)          # a pending reduction, completed by _prep

    def _prep(self, x, norm_w, signs, rows: int, y_out=None):
        if isinstance(x, torch.Tensor):
            return super()._prep(x, norm_w, signs, rows, y_out)
        cfg, ws = self.cfg, self.ws
        name, rows_per = x if isinstance(x, tuple) else (x, 0)
        if rows_per == LL_MODE:
            ib, rows_per = self.mem.ll_in[name], 0
        else:
            ib = self.mem.inbox[name] if name != "local" else None
        if rows_per:
            if y_out is not None:
                raise native.KernelError("sequence-parallel norm has no fp16 output")
            ag = self.mem.ag_out
            ag.rows_per = rows_per
            # "local": the owned rows' branch output sits in ws.hidden (token-sharded MoE)
            check(self.lib.orinfer_act_prep_sp(ctypes.byref(ib) if ib is not None else None,
                                               ctypes.byref(ag), ptr(ws.resid), ptr(norm_w),
                                               ptr(signs), rows, cfg.hidden, float(cfg.eps),
                                               int(cfg.zero_centered_norm), stream(),
                                               None if ib is not None else ptr(ws.hidden)),
                  "act_prep_sp")
            count_launches(1)
            return self.mem.ag_q, self.mem.ag_scale       # gathered; consumers must wait
        q8, sc = ws.q8[cfg.hidden], ws.scale
        check(self.lib.orinfer_act_prep_inbox(ctypes.byref(ib), ptr(ws.resid), ptr(norm_w),
                                              ptr(signs), ptr(q8), ptr(sc), ptr(y_out), rows,
                                              cfg.hidden, float(cfg.eps),
                                              int(cfg.zero_centered_norm), stream()),
              "act_prep_inbox")
        count_launches(1)
        return q8, sc

    def _linear(self, lin: QLinear, q8, scale, rows, out, out_f32=False):
        if q8 is not self.mem.ag_q:
            return super()._linear(lin, q8, scale, rows, out, out_f32)
        # all-gather fused into the GEMM: its TMA warp waits for the source ranks of each tile
        ai = self.mem.ag_in
        ai.rows_per = self._sp_rows_per
        check(self.lib.orinfer_qgemm_ag(FMT[lin.fmt], ptr(q8), ptr(scale), ptr(lin.codes),
                                        ptr(lin.scale), ptr(out), ctypes.byref(ai), rows, lin.n,
                                        lin.k, int(out_f32), stream()), "qgemm_ag")
        count_launches(1)
        return out

    def _head(self, x, p, out):
        if isinstance(x, torch.Tensor) or not (isinstance(x, tuple) and x[1] > 0):
            return super()._head(x, p, out)
        # sequence-parallel: owners normalise + rotate + quantise their rows and push them to
        # every rank; wait for all sources, pick the rows that need logits, run the local
        # vocabulary shard of the head
        head, rows = self.w.head, p.rows
        q8, sc = self._prep(x, self.w.final_norm, head.signs, rows)
        ai = self.mem.ag_in
        ai.rows_per = self._sp_rows_per
        check(self.lib.orinfer_ag_wait(ctypes.byref(ai), rows, stream()), "ag_wait")
        count_launches(1)
        q8, sc = q8[:rows], sc[:rows]
        if p.logit_rows is not None:
            q8 = q8.index_select(0, p.logit_rows).contiguous()
            sc = sc.index_select(0, p.logit_rows).contiguous()
            rows = p.logit_rows.shape[0]
        else:
            q8, sc = q8.clone(), sc.clone()
        if out is None:
            out = torch.empty(rows, head.n, dtype=torch.float32, device=self.device)
        from ..ops import functional as F
        return F.qgemm(q8, sc, head.codes, head.scale, head.fmt, head.n, out=out, out_f32=True,
                       rows=rows)
