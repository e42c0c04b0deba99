"""Tensor-level wrappers of the CUDA kernels (one function per device op).

Every wrapper validates shapes/dtypes, takes optional preallocated outputs (so a
captured CUDA graph owns static buffers) and launches on the current stream.
The matching fp32 PyTorch statement of each op lives in ``orinfer_b200.ref.ops_ref``.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import native
from .native import FMT, check, count_launches, ptr, stream


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise native.KernelError("device op called with a CPU tensor")


def embed_w8(ids: torch.Tensor, table_q: torch.Tensor, table_s: torch.Tensor,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _cuda(ids, table_q, table_s)
    rows, hidden = ids.shape[0], table_q.shape[1]
    assert ids.dtype == torch.int32 and table_q.dtype == torch.int8 and table_s.dtype == torch.float16
    if out is None:
        out = torch.empty(rows, hidden, dtype=torch.float16, device=ids.device)
    check(native.lib().orinfer_embed_w8(ptr(ids), ptr(table_q), ptr(table_s), ptr(out), rows,
                                        hidden, table_q.shape[0], stream()), "embed_w8")
    count_launches(1)
    return out


def act_prep(x: Optional[torch.Tensor], resid: Optional[torch.Tensor],
             norm_w: Optional[torch.Tensor], signs: Optional[torch.Tensor], *, eps: float = 1e-6,
             zero_centered: bool = False, swiglu: bool = False, rows: Optional[int] = None,
             q_out: Optional[torch.Tensor] = None, scale_out: Optional[torch.Tensor] = None,
             y_out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """residual add (in place into ``resid``) -> RMSNorm -> (SwiGLU) -> rotation -> A8."""
    _cuda(x, resid, norm_w, signs)
    ref = x if x is not None else resid
    rows = ref.shape[0] if rows is None else rows
    k = ref.shape[1] // 2 if swiglu else ref.shape[1]
    if x is not None:
        assert x.dtype == torch.float16 and x.is_contiguous()
    if resid is not None:
        assert resid.dtype == torch.float32 and resid.is_contiguous() and not swiglu
    if q_out is None:
        q_out = torch.empty(ref.shape[0], k, dtype=torch.int8, device=ref.device)
    if scale_out is None:
        scale_out = torch.empty(ref.shape[0], dtype=torch.float32, device=ref.device)
    check(native.lib().orinfer_act_prep(ptr(x), ptr(resid), ptr(norm_w), ptr(signs), ptr(q_out),
                                        ptr(scale_out), ptr(y_out), rows, k, float(eps),
                                        int(zero_centered), int(swiglu), stream()), "act_prep")
    count_launches(1)
    return q_out, scale_out


def act_prep_limited(x: torch.Tensor, signs: Optional[torch.Tensor], row_limit: torch.Tensor, *,
                     swiglu: bool, rows: int, q_out: torch.Tensor,
                     scale_out: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``act_prep`` (no residual / norm) for a launch sized for the worst case: only rows below
    the device-side count ``row_limit[0]`` are processed."""
    _cuda(x, signs, row_limit)
    k = x.shape[1] // 2 if swiglu else x.shape[1]
    assert x.dtype == torch.float16 and x.is_contiguous() and row_limit.dtype == torch.int32
    check(native.lib().orinfer_act_prep_limited(ptr(x), ptr(signs), ptr(q_out), ptr(scale_out),
                                                rows, k, int(swiglu), ptr(row_limit), stream()),
          "act_prep_limited")
    count_launches(1)
    return q_out, scale_out


def rope_table(positions: torch.Tensor, head_dim: int, theta: float,
               cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
               rows: Optional[int] = None):
    _cuda(positions)
    assert positions.dtype == torch.int32
    n = positions.shape[0]
    if cos is None:
        cos = torch.empty(n, head_dim // 2, dtype=torch.float32, device=positions.device)
        sin = torch.empty_like(cos)
    check(native.lib().orinfer_rope_table(ptr(positions), ptr(cos), ptr(sin),
                                          n if rows is None else rows, head_dim, float(theta),
                                          stream()), "rope_table")
    count_launches(1)
    return cos, sin


def qk_rope_kv(qkv: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor],
               cos: torch.Tensor, sin: torch.Tensor, row_req: torch.Tensor, row_pos: torch.Tensor,
               page_table: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
               kscale: torch.Tensor, vscale: torch.Tensor, *, qh: int, kvh: int, head_dim: int,
               gated: bool = False, eps: float = 1e-6, zero_centered: bool = False,
               q_out: Optional[torch.Tensor] = None, gate_out: Optional[torch.Tensor] = None,
               rows: Optional[int] = None):
    """Per-head RMSNorm of q/k, NeoX RoPE, and the INT8 group-64 write of K/V into
    the paged cache ``[pages, 128, kvh, D]`` (scales ``[pages, 128, kvh, D/64]``)."""
    _cuda(qkv, cos, row_req, page_table, kcache)
    n = qkv.shape[0]
    assert qkv.dtype == torch.float16 and qkv.is_contiguous()
    assert row_req.dtype == torch.int32 and row_pos.dtype == torch.int32
    assert page_table.dtype == torch.int32 and page_table.dim() == 2
    if q_out is None:
        q_out = torch.empty(n, qh, head_dim, dtype=torch.float16, device=qkv.device)
    if gated and gate_out is None:
        gate_out = torch.empty_like(q_out)
    check(native.lib().orinfer_qk_rope_kv(
        ptr(qkv), ptr(wq), ptr(wk), ptr(cos), ptr(sin), ptr(row_req), ptr(row_pos),
        ptr(page_table), page_table.shape[1], n if rows is None else rows, qh, kvh, head_dim,
        int(gated), float(eps), int(zero_centered), ptr(q_out), ptr(gate_out), ptr(kcache),
        ptr(vcache), ptr(kscale), ptr(vscale), kcache.shape[0], stream()), "qk_rope_kv")
    count_launches(1)
    return q_out, gate_out


def qgemm(a: torch.Tensor, a_scale: torch.Tensor, codes: torch.Tensor, w_scale: torch.Tensor,
          fmt: str, n: int, *, out: Optional[torch.Tensor] = None, out_f32: bool = False,
          rows: Optional[int] = None, path: int = 0) -> torch.Tensor:
    """out[m, n] = (sum_k a[m,k] * W[n,k]) * w_scale[n] * a_scale[m].

    ``path``: 0 auto, 1 SIMT dp4a kernel, 2 tcgen05 tensor-core kernel."""
    _cuda(a, a_scale, codes, w_scale)
    m, k = a.shape
    assert a.dtype == torch.int8 and a.is_contiguous() and a_scale.dtype == torch.float32
    assert w_scale.dtype == torch.float16 and codes.is_contiguous()
    if out is None:
        out = torch.empty(m, n, dtype=torch.float32 if out_f32 else torch.float16, device=a.device)
    else:
        assert out.dtype == (torch.float32 if out_f32 else torch.float16)
    mm = m if rows is None else rows
    check(native.lib().orinfer_qgemm(FMT[fmt], ptr(a), ptr(a_scale), ptr(codes), ptr(w_scale),
                                     ptr(out), mm, n, k, int(out_f32), path, stream()), "qgemm")
    count_launches(native.lib().orinfer_qgemm_launches_fmt(FMT[fmt], mm, n, k, int(out_f32), path))
    return out


PRE_NORM, PRE_PLAIN, PRE_SWIGLU = 1, 2, 3


def qgemv_fused(pre: int, x: Optional[torch.Tensor], resid: Optional[torch.Tensor],
                norm_w: Optional[torch.Tensor], signs: Optional[torch.Tensor], codes: torch.Tensor,
                w_scale: torch.Tensor, fmt: str, n: int, k: int, rows: int, *, eps: float = 1e-6,
                zero_centered: bool = False, out: Optional[torch.Tensor] = None,
                resid_accum: Optional[torch.Tensor] = None, y_out: Optional[torch.Tensor] = None,
                q_out: Optional[torch.Tensor] = None,
                scale_out: Optional[torch.Tensor] = None) -> bool:
    """Projection of at most 8 rows with the row preparation fused into the kernel
    (``pre``: PRE_NORM = resid (+ x) -> RMSNorm -> rotation -> A8; PRE_PLAIN = x -> rotation ->
    A8; PRE_SWIGLU = SwiGLU(x [rows, 2k]) -> rotation -> A8) and, with ``resid_accum``, the
    FP16-rounded result added into an FP32 matrix.  Same bits as ``act_prep`` followed by
    ``qgemm``.  Returns False when the shape does not fit (the caller then runs the separate
    kernels); E8P weights only."""
    if rows > 8 or fmt not in ("q4", "q2"):
        return False
    code = native.lib().orinfer_qgemv_fused(
        FMT[fmt], pre, ptr(x), ptr(resid), ptr(norm_w), ptr(signs), float(eps),
        int(zero_centered), ptr(q_out), ptr(scale_out), ptr(y_out), ptr(codes), ptr(w_scale),
        ptr(out), ptr(resid_accum), rows, n, k, stream())
    if code == -1:
        return False
    check(code, "qgemv_fused")
    count_launches(1)
    return True


def attention_splits(max_kv_len: int, rows: int, kvh: int) -> int:
    """Split the key axis when there are too few (row, kv head) CTAs to fill 148 SMs: about
    three CTAs per SM, at least 64 keys per split.  An ``attention`` entry of the tuning table
    (``tuning/tables.py``) replaces the first rule for its row and context range."""
    if max_kv_len <= 128:
        return 1
    from ..tuning import tables
    tuned = tables.attention_lookup(max_kv_len, rows, kvh)      # a tuned table overrides
    want = tuned if tuned is not None else max(1, (148 * 3) // max(rows * kvh, 1))
    return int(max(1, min(want, (max_kv_len + 63) // 64, 32)))


def attention(q: torch.Tensor, gate: Optional[torch.Tensor], row_req: torch.Tensor,
              row_pos: torch.Tensor, page_table: torch.Tensor, kcache: torch.Tensor,
              vcache: torch.Tensor, kscale: torch.Tensor, vscale: torch.Tensor, *, splits: int = 1,
              scratch: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
              rows: Optional[int] = None) -> torch.Tensor:
    _cuda(q, row_req, page_table, kcache)
    n, qh, d = q.shape
    kvh = kcache.shape[2]
    if out is None:
        out = torch.empty(n, qh * d, dtype=torch.float16, device=q.device)
    if splits > 1 and scratch is None:
        need = native.lib().orinfer_attention_scratch_bytes(n, qh, d, splits)
        scratch = torch.empty(need // 4, dtype=torch.float32, device=q.device)
    check(native.lib().orinfer_attention(
        ptr(q), ptr(gate), ptr(row_req), ptr(row_pos), ptr(page_table), page_table.shape[1],
        ptr(kcache), ptr(vcache), ptr(kscale), ptr(vscale), ptr(out), n if rows is None else rows,
        qh, kvh, d, splits, ptr(scratch), stream()), "attention")
    count_launches(2 if splits > 1 else 1)
    return out


def attention_prefill(q: torch.Tensor, gate: Optional[torch.Tensor], chunks: torch.Tensor,
                      max_q_len: int, page_table: torch.Tensor, kcache: torch.Tensor,
                      vcache: torch.Tensor, kscale: torch.Tensor, vscale: torch.Tensor, *,
                      out: Optional[torch.Tensor] = None, total_rows: Optional[int] = None) -> bool:
    """tcgen05 flash attention over prefill chunks.  ``chunks`` is int32 [C, 4] =
    (first row, rows, position of the first row, page-table row).  Returns False when the
    head size is not implemented by the tensor-core kernel (nothing was launched)."""
    _cuda(q, chunks, page_table, kcache)
    n, qh, d = q.shape
    assert chunks.dtype == torch.int32 and chunks.dim() == 2 and chunks.shape[1] == 4
    if out is None:
        raise native.KernelError("attention_prefill needs a preallocated output")
    rc = native.lib().orinfer_attention_prefill(
        ptr(q), ptr(gate), ptr(chunks), chunks.shape[0], max_q_len,
        n if total_rows is None else total_rows, ptr(page_table), page_table.shape[1],
        ptr(kcache), ptr(vcache), ptr(kscale), ptr(vscale), ptr(out), qh, kcache.shape[2], d,
        kcache.shape[0], stream())
    if rc == -4:
        return False
    check(rc, "attention_prefill")
    count_launches(1)
    return True


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None,
           scratch: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
           rows: Optional[int] = None) -> torch.Tensor:
    _cuda(logits)
    m, v = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    parts = native.lib().orinfer_argmax_parts(v)
    if scratch is None:
        scratch = (torch.empty(m * parts, dtype=torch.float32, device=logits.device),
                   torch.empty(m * parts, dtype=torch.int32, device=logits.device))
    if out is None:
        out = torch.empty(m, dtype=torch.int32, device=logits.device)
    check(native.lib().orinfer_argmax(ptr(logits), m if rows is None else rows, v, ptr(scratch[0]),
                                      ptr(scratch[1]), ptr(out), stream()), "argmax")
    count_launches(2)
    return out


# ---------------------------------------------------------------------------- MoE
def router_topk(y: torch.Tensor, router_w: torch.Tensor, experts: int, top_k: int, *,
                renorm: bool = True, rows: Optional[int] = None, ids=None, probs=None,
                gate=None):
    """Router projection + softmax + top-k (ties to the lower expert id).  ``router_w`` has
    ``experts`` rows plus an optional shared-expert gate row.  Returns (ids int32 [M,k],
    probs fp32 [M,k], sigmoid shared gate fp32 [M] or None)."""
    _cuda(y, router_w)
    m, h = y.shape
    has_shared = router_w.shape[0] == experts + 1
    dev = y.device
    ids = torch.empty(m, top_k, dtype=torch.int32, device=dev) if ids is None else ids
    probs = torch.empty(m, top_k, dtype=torch.float32, device=dev) if probs is None else probs
    if has_shared and gate is None:
        gate = torch.empty(m, dtype=torch.float32, device=dev)
    check(native.lib().orinfer_router_topk(ptr(y), ptr(router_w), m if rows is None else rows, h,
                                           experts, int(has_shared), top_k, int(renorm), ptr(ids),
                                           ptr(probs), ptr(gate), stream()), "router_topk")
    count_launches(1)
    return ids, probs, gate


class MoeScratch:
    """Static buffers of one MoE layer evaluation for up to ``max_rows`` tokens."""

    def __init__(self, max_rows: int, top_k: int, experts: int, hidden: int, ffn: int, device):
        s = max_rows * top_k
        e = lambda *shape, dt: torch.empty(*shape, dtype=dt, device=device)
        self.max_tiles = (s + 127) // 128 + experts
        self.ids = e(max_rows, top_k, dt=torch.int32)
        self.probs = e(max_rows, top_k, dt=torch.float32)
        self.gate = e(max_rows, dt=torch.float32)
        self.counts = e(experts, dt=torch.int32)
        self.offsets = e(experts + 1, dt=torch.int32)
        self.tiles = torch.zeros(self.max_tiles, 4, dtype=torch.int32, device=device)
        self.meta = torch.zeros(4, dtype=torch.int32, device=device)
        self.slots = e(s, dt=torch.int32)
        self.q8 = e(s, hidden, dt=torch.int8)
        self.scale = e(s, dt=torch.float32)
        self.gate_up = e(s, 2 * ffn, dt=torch.float16)
        self.q8_mid = e(s, ffn, dt=torch.int8)
        self.scale_mid = e(s, dt=torch.float32)
        self.down = e(s, hidden, dt=torch.float16)


def moe_dispatch(ids: torch.Tensor, q8: Optional[torch.Tensor], scale: Optional[torch.Tensor],
                 experts: int, sc: MoeScratch, rows: int, base_expert: int = 0,
                 local_experts: Optional[int] = None) -> None:
    """Deterministic dispatch metadata + copy of the routed rows into expert-contiguous
    slots (``q8 = None``: numbering only).  With ``local_experts`` only rows routed to experts
    [base_expert, base_expert + local_experts) are dispatched; other slots become -1."""
    top_k = ids.shape[1]
    width = sc.q8.shape[1] if q8 is None else q8.shape[1]
    if local_experts is not None and local_experts != experts:
        check(native.lib().orinfer_moe_dispatch_ep(
            ptr(ids), rows, top_k, base_expert, local_experts, ptr(q8), ptr(scale), width,
            ptr(sc.counts), ptr(sc.offsets), ptr(sc.tiles), ptr(sc.meta), sc.max_tiles,
            ptr(sc.slots), ptr(sc.q8), ptr(sc.scale), stream()), "moe_dispatch_ep")
        count_launches(3)
        return
    check(native.lib().orinfer_moe_dispatch(
        ptr(ids), rows, top_k, experts, ptr(q8), ptr(scale), width, ptr(sc.counts),
        ptr(sc.offsets), ptr(sc.tiles), ptr(sc.meta), sc.max_tiles, ptr(sc.slots), ptr(sc.q8),
        ptr(sc.scale), stream()), "moe_dispatch")
    count_launches(3)


def qgemm_grouped(a: torch.Tensor, a_scale: torch.Tensor, codes: torch.Tensor,
                  w_scale: torch.Tensor, fmt: str, n: int, out: torch.Tensor, sc: MoeScratch,
                  total_rows: int) -> torch.Tensor:
    experts = codes.shape[0]
    check(native.lib().orinfer_qgemm_grouped(
        FMT[fmt], ptr(a), ptr(a_scale), ptr(codes), ptr(w_scale), ptr(out), total_rows, n,
        a.shape[1], experts, ptr(sc.tiles), ptr(sc.meta), sc.max_tiles, stream()),
        "qgemm_grouped")
    count_launches(1)
    return out


def moe_combine(expert_out: torch.Tensor, slots: torch.Tensor, probs: torch.Tensor,
                shared_out: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                out: torch.Tensor, rows: int) -> torch.Tensor:
    check(native.lib().orinfer_moe_combine(ptr(expert_out), ptr(slots), ptr(probs), rows,
                                           probs.shape[1], ptr(shared_out), ptr(gate), ptr(out),
                                           out.shape[1], stream()), "moe_combine")
    count_launches(1)
    return out


# ---------------------------------------------------------------- gated delta rule
def small_proj(x: torch.Tensor, w: torch.Tensor, rows: Optional[int] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 ``x[rows, H] @ w[N, H]^T`` for a narrow fp16 weight (the GDN a/b gates)."""
    _cuda(x, w)
    assert x.dtype == torch.float16 and w.dtype == torch.float16 and x.is_contiguous()
    rows = x.shape[0] if rows is None else rows
    if out is None:
        out = torch.empty(x.shape[0], w.shape[0], dtype=torch.float32, device=x.device)
    check(native.lib().orinfer_small_proj(ptr(x), ptr(w), ptr(out), rows, x.shape[1], w.shape[0],
                                          stream()), "small_proj")
    count_launches(1)
    return out


def gdn_conv(x: torch.Tensor, weight: torch.Tensor, hist: torch.Tensor, row_first: torch.Tensor,
             row_slot: torch.Tensor, row_pos: torch.Tensor, segs: torch.Tensor, n_segs: int,
             rows: int, hk: int, hv: int, head_dim: int,
             out: Optional[torch.Tensor] = None, update_history: bool = True) -> torch.Tensor:
    """Causal conv4 + SiLU + L2(q, k) over the q|k|v channels of ``x`` [rows, >= conv_dim];
    ``hist`` fp16 [slots, 3, conv_dim] is read, then advanced in place per segment (unless
    ``update_history`` is off: a verification pass commits its history later)."""
    _cuda(x, weight, hist, row_first, row_slot, row_pos, segs)
    conv_dim = (2 * hk + hv) * head_dim
    assert x.dtype == torch.float16 and x.stride(1) == 1 and hist.shape[-1] == conv_dim
    assert weight.shape == (conv_dim, 4) and weight.is_contiguous()
    if out is None:
        out = torch.empty(x.shape[0], conv_dim, dtype=torch.float16, device=x.device)
    check(native.lib().orinfer_gdn_conv(ptr(x), x.stride(0), ptr(weight), ptr(hist),
                                        ptr(row_first), ptr(row_slot), ptr(row_pos), ptr(segs),
                                        n_segs, rows,
                                        hk, hv, head_dim, ptr(out), stream(),
                                        int(update_history)), "gdn_conv")
    count_launches(2 if update_history else 1)
    return out


def gdn_scan(qkv: torch.Tensor, ab: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
             segs: torch.Tensor, n_segs: int, row_slot: torch.Tensor, row_pos: torch.Tensor,
             hk: int, hv: int, head_dim: int, state: torch.Tensor,
             out: Optional[torch.Tensor] = None,
             factors: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sequential gated-delta recurrence; ``state`` fp32 [slots, HV, D, D] updated in place.
    With ``factors`` (fp32 [rows, HV, 2D+1]) the state is left untouched and every step's
    (decay, k, delta) is recorded for :func:`gdn_commit`."""
    _cuda(qkv, ab, a_log, dt_bias, segs, state, row_slot, row_pos)
    assert ab.dtype == torch.float32 and state.dtype == torch.float32 and state.is_contiguous()
    assert a_log.dtype == torch.float32 and dt_bias.dtype == torch.float32
    if out is None:
        out = torch.empty(qkv.shape[0], hv, head_dim, dtype=torch.float32, device=qkv.device)
    check(native.lib().orinfer_gdn_scan(ptr(qkv), ptr(ab), ptr(a_log), ptr(dt_bias), ptr(segs),
                                        n_segs, ptr(row_slot), ptr(row_pos), hk, hv, head_dim,
                                        ptr(state), ptr(out), stream(), ptr(factors)),
          "gdn_scan")
    count_launches(1)
    return out


def gdn_commit(x: torch.Tensor, factors: torch.Tensor, segs: torch.Tensor, n_segs: int,
               accepted: torch.Tensor, row_slot: torch.Tensor, row_pos: torch.Tensor, hk: int,
               hv: int, head_dim: int, hist: torch.Tensor, state: torch.Tensor) -> None:
    """Keeps the first ``accepted[s]`` rows of every segment of a verification pass: advances
    the convolution history by them and replays their recorded state updates."""
    _cuda(x, factors, segs, accepted, row_slot, row_pos, hist, state)
    assert accepted.dtype == torch.int32 and factors.dtype == torch.float32
    check(native.lib().orinfer_gdn_commit(ptr(x), x.stride(0), ptr(factors), ptr(segs), n_segs,
                                          ptr(accepted), ptr(row_slot), ptr(row_pos), hk, hv,
                                          head_dim, ptr(hist), ptr(state), stream()),
          "gdn_commit")
    count_launches(2)


def gdn_gated_norm(o: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float, rows: int,
                   hv: int, head_dim: int, sigmoid_gate: bool = False,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``rmsnorm(o) * w * silu(z)`` per head; ``z`` may be a column view of the projection."""
    _cuda(o, z, weight)
    assert o.dtype == torch.float32 and z.dtype == torch.float16 and z.stride(1) == 1
    if out is None:
        out = torch.empty(o.shape[0], hv * head_dim, dtype=torch.float16, device=o.device)
    check(native.lib().orinfer_gdn_gated_norm(ptr(o), ptr(z), z.stride(0), ptr(weight), float(eps),
                                              int(sigmoid_gate), rows, hv, head_dim, ptr(out),
                                              stream()), "gdn_gated_norm")
    count_launches(1)
    return out


# ---------------------------------------------------------------- sampling
def sample_topk(logits: torch.Tensor, top_k: torch.Tensor, temperature: torch.Tensor,
                top_p: torch.Tensor, uniform: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row top-k/top-p categorical draw on the device.  ``logits`` fp32 [rows, vocab];
    ``top_k`` int32, ``temperature`` / ``top_p`` / ``uniform`` fp64, all [rows].  Returns
    (tokens int32, flags int32); a set flag means the host law must serve that row."""
    _cuda(logits, top_k, temperature, top_p, uniform)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and top_k.dtype == torch.int32
    assert temperature.dtype == torch.float64 and top_p.dtype == torch.float64
    assert uniform.dtype == torch.float64
    rows, vocab = logits.shape
    tok = torch.empty(rows, dtype=torch.int32, device=logits.device)
    flag = torch.zeros(rows, dtype=torch.int32, device=logits.device)
    check(native.lib().orinfer_sample_topk(ptr(logits), rows, vocab, logits.stride(0), ptr(top_k),
                                           ptr(temperature), ptr(top_p), ptr(uniform), ptr(tok),
                                           ptr(flag), stream()), "sample_topk")
    count_launches(1)
    return tok, flag
