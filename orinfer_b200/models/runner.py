"""Device model runner: one packed-row forward pass over the CUDA kernels.

A *packet* is a set of token rows from any mix of requests (decode rows and
prefill chunks).  Shared ops (projections, norms) run once over all rows;
request-private ops (KV write, attention, GDN state) are natively batched
through ``row_req`` / ``row_pos`` / the page table, so no per-request launches
exist.  This mirrors the packet structure of the reference's row adapter
(crates/orinfer-models/src/qwen3_5/rows.rs:1137-1463) with page-table
indirection in place of its pointer tables; op order follows
python/orinfer_build/models/qwen35/build.py:802-1116.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..config import KV_GROUP, PAGE_TOKENS, ModelConfig
from ..ops import functional as F
from ..utils import trace
from .weights import LayerWeights, ModelWeights, QLinear


@dataclass
class KVPool:
    """Paged INT8 KV storage for every full-attention layer. Page 0 is a dummy
    target for padded rows and is never handed out."""
    k: List[torch.Tensor]
    v: List[torch.Tensor]
    ks: List[torch.Tensor]
    vs: List[torch.Tensor]
    pages: int

    @classmethod
    def allocate(cls, cfg: ModelConfig, pages: int, device, extra_layers: int = 0) -> "KVPool":
        n = sum(cfg.is_full_attention(i) for i in range(cfg.layers)) + extra_layers
        mk = lambda last, dt: [torch.zeros(pages, PAGE_TOKENS, cfg.kv_heads, last, dtype=dt,
                                           device=device) for _ in range(n)]
        g = cfg.head_dim // KV_GROUP
        return cls(mk(cfg.head_dim, torch.int8), mk(cfg.head_dim, torch.int8),
                   mk(g, torch.float16), mk(g, torch.float16), pages)

    @staticmethod
    def bytes_per_page(cfg: ModelConfig, extra_layers: int = 0) -> int:
        n = sum(cfg.is_full_attention(i) for i in range(cfg.layers)) + extra_layers
        per_tok = 2 * cfg.kv_dim + 2 * 2 * (cfg.kv_dim // KV_GROUP)
        return n * per_tok * PAGE_TOKENS


class Workspace:
    """Static activation buffers sized for ``max_rows`` packed rows."""

    def __init__(self, cfg: ModelConfig, max_rows: int, device):
        self.max_rows = max_rows
        f16, f32, i8 = torch.float16, torch.float32, torch.int8
        e = lambda *s, dt=f16: torch.empty(*s, dtype=dt, device=device)
        h = cfg.hidden
        self.hidden = e(max_rows, h)
        self.resid = e(max_rows, h, dt=f32)
        self.scale = e(max_rows, dt=f32)
        self.q8: Dict[int, torch.Tensor] = {}
        widths = {h, cfg.q_heads * cfg.head_dim}
        ffn_w = cfg.ffn or 0
        if ffn_w:
            widths.add(ffn_w)
        if cfg.experts:
            widths.update({cfg.expert_ffn, cfg.shared_expert_ffn or cfg.expert_ffn})
        if cfg.arch == "hybrid":
            widths.add(cfg.gdn_v_heads * cfg.gdn_head_dim)
        if cfg.mtp_layers:
            widths.add(2 * h)
            widths.add(cfg.ffn or max(cfg.expert_ffn * 4, 512))
        for w in widths:
            if w:
                self.q8[w] = e(max_rows, w, dt=i8)
        self.qkv = e(max_rows, cfg.q_dim + 2 * cfg.kv_dim)
        self.q = e(max_rows, cfg.q_heads, cfg.head_dim)
        self.gate = e(max_rows, cfg.q_heads, cfg.head_dim) if cfg.gated_attention else None
        self.attn = e(max_rows, cfg.q_heads * cfg.head_dim)
        mtp_f = (cfg.ffn or max(cfg.expert_ffn * 4, 512)) if cfg.mtp_layers else 0
        self.gate_up = e(max_rows, 2 * max(ffn_w, cfg.shared_expert_ffn, mtp_f, 64))
        self.cos = e(max_rows, cfg.head_dim // 2, dt=f32)
        self.sin = e(max_rows, cfg.head_dim // 2, dt=f32)
        # split-KV partial records: (rows * splits) <= SPLIT_ROWS by construction, and the
        # buffer never moves, so captured graphs may keep its address.
        self.attn_scratch = e(self.SPLIT_ROWS * cfg.q_heads * (cfg.head_dim + 2), dt=f32)

    SPLIT_ROWS = 512

    def scale_alt(self, rows: int) -> torch.Tensor:
        """A second row-scale buffer, for a quantisation whose input scales are still live."""
        if getattr(self, "_scale_alt", None) is None:
            self._scale_alt = torch.empty(self.max_rows, dtype=torch.float32,
                                          device=self.hidden.device)
        return self._scale_alt

    def attn_norm(self, rows: int, hidden: int) -> torch.Tensor:
        """fp16 scratch [max_rows, hidden] for normalised hidden states (final norm)."""
        if getattr(self, "_norm_buf", None) is None:
            self._norm_buf = torch.empty(self.max_rows, hidden, dtype=torch.float16,
                                         device=self.hidden.device)
        return self._norm_buf


@dataclass
class Packet:
    """Device-side description of one forward pass (all int32, on the GPU)."""
    ids: torch.Tensor            # [rows]
    row_req: torch.Tensor        # [rows] index into page_table
    row_pos: torch.Tensor        # [rows] absolute position of the row in its request
    page_table: torch.Tensor     # [requests, max_pages]
    rows: int
    max_kv_len: int              # host-side bound used to pick the split count
    logit_rows: Optional[torch.Tensor] = None   # int64 rows whose logits are needed (None = all)
    # Prefill chunks for the tensor-core attention kernel: int32 [C, 4] = (first row, rows,
    # position of the first row, page-table row).  Rows [0, decode_rows) are single-row
    # requests handled by the row kernel; None = every row goes through the row kernel.
    chunks: Optional[torch.Tensor] = None
    max_q_len: int = 0
    decode_rows: int = 0
    # Runs of consecutive rows of one request, for the recurrent (GDN) layers: int32 [S, 4] =
    # (first row, rows, 0, 0) and, per row, the first row of its run.  Derived from row_req on
    # the host when absent (one readback), so graph-captured packets must carry them.
    segments: Optional[torch.Tensor] = None
    n_segments: int = 0
    row_first: Optional[torch.Tensor] = None
    # A verification packet of a speculative round: recurrent layers leave their state and
    # convolution history untouched and record what ``gdn_commit`` needs to keep a prefix.
    tentative: bool = False
    # Media rows: ``overlay`` [n, hidden] replaces the embedding of rows ``overlay_rows``
    # (int64 [n]); ``mrope`` int32 [3, rows] gives (t, h, w) rotary positions when they differ
    # from ``row_pos`` (which always addresses the KV cache).
    overlay_rows: Optional[torch.Tensor] = None
    overlay: Optional[torch.Tensor] = None
    mrope: Optional[torch.Tensor] = None
    # Encoder passes: row r may attend to keys 0..attend_pos[r] instead of 0..row_pos[r]
    # (all rows of a bidirectional input carry the last position).  int32 [rows].
    attend_pos: Optional[torch.Tensor] = None

    def ensure_segments(self) -> None:
        if self.segments is not None:
            return
        req = self.row_req[: self.rows].cpu().tolist()
        segs, first, start = [], [], 0
        for i in range(self.rows + 1):
            if i == self.rows or (i > 0 and req[i] != req[i - 1]):
                segs.append([start, i - start, 0, 0])
                first += [start] * (i - start)
                start = i
        dev = self.row_req.device
        self.segments = torch.tensor(segs, dtype=torch.int32, device=dev)
        self.row_first = torch.tensor(first, dtype=torch.int32, device=dev)
        self.n_segments = len(segs)


class ModelRunner:
    def __init__(self, weights: ModelWeights, kv: KVPool, max_rows: int):
        self.w = weights
        self.cfg = weights.config
        self.kv = kv
        self.device = weights.embed_q.device
        self.ws = Workspace(self.cfg, max_rows, self.device)
        self._attn_index = {}
        n = 0
        for i in range(self.cfg.layers):
            if self.cfg.is_full_attention(i):
                self._attn_index[i] = n
                n += 1
        self.mtp_kv_index = n
        self._argmax_scratch = None
        self.layer_hooks = {}
        # Decode steps of one or two rows on a dense model with lattice-coded projections run
        # with the row kernels fused into the projections (four launches fewer per layer;
        # every CTA repeats the row preparation, which stops paying off beyond two rows).
        # Runners that reduce across ranks keep the separate kernels.
        import os
        e8p = lambda lin: lin is not None and lin.fmt in ("q4", "q2")
        self._fused_decode = (
            type(self) is ModelRunner and os.environ.get("ORINFER_FUSED_DECODE", "1") != "0"
            and self.cfg.arch == "dense" and not self.cfg.experts
            and all(lw.kind == "attn" and e8p(lw.qkv) and e8p(lw.o) and e8p(lw.gate_up)
                    and e8p(lw.down) for lw in weights.layers))

    # ---------------------------------------------------------------- helpers
    def _signs(self, lin: QLinear):
        return lin.signs

    def _linear(self, lin: QLinear, q8, scale, rows, out, out_f32=False):
        return F.qgemm(q8, scale, lin.codes, lin.scale, lin.fmt, lin.n, out=out, out_f32=out_f32,
                       rows=rows)

    def _attention_block(self, lw: LayerWeights, kv_slot: int, x, p: Packet, rows: int,
                         first: bool):
        cfg, ws = self.cfg, self.ws
        q8, sc = self._prep(x, lw.in_norm, self._signs(lw.qkv), rows)
        qkv = self._linear(lw.qkv, q8, sc, rows, ws.qkv)
        self._attention_core(lw, kv_slot, qkv, p, rows)
        qd = cfg.q_heads * cfg.head_dim
        q8, sc = F.act_prep(ws.attn, None, None, self._signs(lw.o), rows=rows, q_out=ws.q8[qd],
                            scale_out=ws.scale)
        return self._row_parallel("o", lw.o, q8, sc, rows)

    def _attention_core(self, lw: LayerWeights, kv_slot: int, qkv, p: Packet, rows: int):
        """q/k head norm + RoPE + INT8 KV write, then attention into ``ws.attn``."""
        cfg, ws = self.cfg, self.ws
        F.qk_rope_kv(qkv, lw.q_norm if cfg.qk_norm else None, lw.k_norm if cfg.qk_norm else None,
                     ws.cos, ws.sin, p.row_req, p.row_pos, p.page_table, self.kv.k[kv_slot],
                     self.kv.v[kv_slot], self.kv.ks[kv_slot], self.kv.vs[kv_slot],
                     qh=cfg.q_heads, kvh=cfg.kv_heads, head_dim=cfg.head_dim,
                     gated=cfg.gated_attention and lw.qkv.n == cfg.q_dim + 2 * cfg.kv_dim,
                     eps=cfg.eps, zero_centered=cfg.zero_centered_norm, q_out=ws.q,
                     gate_out=ws.gate, rows=rows)
        gated = cfg.gated_attention and lw.qkv.n == cfg.q_dim + 2 * cfg.kv_dim
        gate = ws.gate if gated else None
        row_rows = rows
        if p.chunks is not None and p.attend_pos is None and cfg.head_dim in (64, 128, 256):
            done = F.attention_prefill(ws.q, gate, p.chunks, p.max_q_len, p.page_table,
                                       self.kv.k[kv_slot], self.kv.v[kv_slot],
                                       self.kv.ks[kv_slot], self.kv.vs[kv_slot], out=ws.attn,
                                       total_rows=rows)
            if done:
                row_rows = p.decode_rows
        if row_rows > 0:
            splits = min(F.attention_splits(p.max_kv_len, row_rows, cfg.kv_heads),
                         max(ws.SPLIT_ROWS // row_rows, 1))
            scratch = ws.attn_scratch if splits > 1 else None
            see = p.row_pos if p.attend_pos is None else p.attend_pos
            F.attention(ws.q, gate, p.row_req, see, p.page_table, self.kv.k[kv_slot],
                        self.kv.v[kv_slot], self.kv.ks[kv_slot], self.kv.vs[kv_slot],
                        splits=splits, scratch=scratch, out=ws.attn, rows=row_rows)

    def _fused_layer(self, lw: LayerWeights, kv_slot: int, p: Packet, rows: int) -> bool:
        """One dense decoder layer of a decode-sized packet with the row kernels fused into
        the projections.  The residual stream (``ws.resid``) already holds every earlier
        branch output: each prologue only reads it and the o / down projections add their
        FP16-rounded results into it.  False when a shape does not fit the fused kernel."""
        cfg, ws = self.cfg, self.ws
        h, eps, zc = cfg.hidden, cfg.eps, cfg.zero_centered_norm
        fuse = F.qgemv_fused
        qd = cfg.q_heads * cfg.head_dim
        f = lw.gate_up.n // 2
        gu = ws.gate_up.view(-1)[: ws.max_rows * 2 * f].view(ws.max_rows, 2 * f)
        with trace.span("attn"):
            if not fuse(F.PRE_NORM, None, ws.resid, lw.in_norm, lw.qkv.signs, lw.qkv.codes,
                        lw.qkv.scale, lw.qkv.fmt, lw.qkv.n, h, rows, eps=eps, zero_centered=zc,
                        out=ws.qkv):
                return False
            self._attention_core(lw, kv_slot, ws.qkv, p, rows)
            ok = fuse(F.PRE_PLAIN, ws.attn, None, None, lw.o.signs, lw.o.codes, lw.o.scale,
                      lw.o.fmt, h, qd, rows, resid_accum=ws.resid)
        with trace.span("ffn"):
            ok = ok and fuse(F.PRE_NORM, None, ws.resid, lw.post_norm, lw.gate_up.signs,
                             lw.gate_up.codes, lw.gate_up.scale, lw.gate_up.fmt, 2 * f, h, rows,
                             eps=eps, zero_centered=zc, out=gu)
            ok = ok and fuse(F.PRE_SWIGLU, gu, None, None, lw.down.signs, lw.down.codes,
                             lw.down.scale, lw.down.fmt, h, f, rows, resid_accum=ws.resid)
        if not ok:
            raise RuntimeError("a projection of this model does not fit the fused decode kernel")
        return True

    def _fused_fits(self, rows: int) -> bool:
        """Shared memory of the fused projection kernel: decode tables, the INT8 rows, one
        FP32 row and the partial sums must fit one CTA for the widest input of a layer."""
        cfg = self.cfg
        mt = 1 if rows == 1 else (2 if rows == 2 else (4 if rows <= 4 else 8))
        k = max(cfg.hidden, cfg.q_heads * cfg.head_dim, cfg.ffn)
        return 65536 + mt * k + 4 * k + 8192 <= 220 * 1024

    def _gdn_state(self, slots: int):
        """Recurrent pools, one entry per page-table row: FP32 state [slots, HV, D, D] and the
        FP16 three-row convolution history [slots, 3, conv_dim] of every GDN layer."""
        st = getattr(self, "_gdn", None)
        if st is None or st["slots"] < slots:
            cfg = self.cfg
            hk, hv, d = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
            conv_dim = (2 * hk + hv) * d
            n = sum(lw.kind == "gdn" for lw in self.w.layers)
            ws, dev = self.ws, self.device
            st = self._gdn = dict(
                slots=slots,
                index={i: j for j, i in enumerate(i for i, lw in enumerate(self.w.layers)
                                                  if lw.kind == "gdn")},
                state=torch.zeros(n, slots, hv, d, d, dtype=torch.float32, device=dev),
                hist=torch.zeros(n, slots, 3, conv_dim, dtype=torch.float16, device=dev),
                proj=torch.empty(ws.max_rows, conv_dim + hv * d, dtype=torch.float16, device=dev),
                conv=torch.empty(ws.max_rows, conv_dim, dtype=torch.float16, device=dev),
                ab=torch.empty(ws.max_rows, 2 * hv, dtype=torch.float32, device=dev),
                o=torch.empty(ws.max_rows, hv, d, dtype=torch.float32, device=dev),
                mix=torch.empty(ws.max_rows, hv * d, dtype=torch.float16, device=dev),
                layers=n, t_rows=0)
        return st

    TENTATIVE_ROWS = 512

    def _gdn_tentative(self, st):
        """Per-layer records of a verification pass: the pre-convolution rows and the
        (decay, k, delta) factors of every step."""
        if "t_proj" not in st:
            cfg = self.cfg
            hk, hv, d = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
            conv_dim = (2 * hk + hv) * d
            n, r, dev = st["layers"], self.TENTATIVE_ROWS, self.device
            st["t_proj"] = torch.empty(n, r, conv_dim, dtype=torch.float16, device=dev)
            st["t_fac"] = torch.empty(n, r, hv, 2 * d + 1, dtype=torch.float32, device=dev)
        return st

    def gdn_snapshot(self, slot: int):
        """Copy of the recurrent state of one request slot (every GDN layer): what a cached
        prefix needs besides its KV pages."""
        st = self._gdn
        return st["state"][:, slot].clone(), st["hist"][:, slot].clone()

    def gdn_restore(self, slot: int, snap, slots: int) -> None:
        """``slots``: rows of the page table (sizes the pools on first use)."""
        st = self._gdn_state(slots)
        st["state"][:, slot].copy_(snap[0])
        st["hist"][:, slot].copy_(snap[1])

    def gdn_commit(self, p: Packet, accepted_rows) -> None:
        """Keeps the first ``accepted_rows[s]`` rows of every segment of the tentative packet
        ``p`` in every recurrent layer (state and convolution history)."""
        st = getattr(self, "_gdn", None)
        if st is None or "t_proj" not in st:
            return
        cfg = self.cfg
        hk, hv, d = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
        acc = torch.tensor(list(accepted_rows), dtype=torch.int32, device=self.device)
        for j in range(st["layers"]):
            F.gdn_commit(st["t_proj"][j], st["t_fac"][j], p.segments, p.n_segments, acc,
                         p.row_req, p.row_pos, hk, hv, d, st["hist"][j], st["state"][j])

    def _gdn_block(self, lw: LayerWeights, layer: int, x, p: Packet, rows: int):
        """Gated-delta-rule mixer: norm+rotate+A8 -> q|k|v|z projection (tensor cores) and the
        fp16 a/b gate projection -> conv4+SiLU+L2 with per-request history -> sequential FP32
        recurrence -> gated RMSNorm -> rotate+A8 -> output projection."""
        cfg = self.cfg
        hk, hv, d = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
        conv_dim = (2 * hk + hv) * d
        p.ensure_segments()
        st = self._gdn_state(p.page_table.shape[0])
        j = st["index"][layer]
        y16 = self.ws.attn_norm(rows, cfg.hidden)
        q8, sc = self._prep(x, lw.in_norm, self._signs(lw.gdn_qkvz), rows, y_out=y16)
        proj = self._linear(lw.gdn_qkvz, q8, sc, rows, st["proj"])
        F.small_proj(y16, lw.gdn_ab, rows=rows, out=st["ab"])
        factors = None
        if p.tentative:
            if rows > self.TENTATIVE_ROWS:
                raise ValueError("verification packet larger than the recurrent journal")
            self._gdn_tentative(st)
            st["t_proj"][j, :rows].copy_(proj[:rows, :conv_dim])
            factors = st["t_fac"][j]
        F.gdn_conv(proj, lw.gdn_conv, st["hist"][j], p.row_first, p.row_req, p.row_pos,
                   p.segments, p.n_segments, rows, hk, hv, d, out=st["conv"],
                   update_history=not p.tentative)
        F.gdn_scan(st["conv"], st["ab"], lw.gdn_a_log, lw.gdn_dt_bias, p.segments, p.n_segments,
                   p.row_req, p.row_pos, hk, hv, d, st["state"][j], out=st["o"], factors=factors)
        F.gdn_gated_norm(st["o"], proj[:, conv_dim:], lw.gdn_norm, cfg.eps, rows, hv, d,
                         out=st["mix"])
        q8, sc = F.act_prep(st["mix"], None, None, self._signs(lw.gdn_out), rows=rows,
                            q_out=self.ws.q8[hv * d], scale_out=self.ws.scale)
        return self._row_parallel("gdn_out", lw.gdn_out, q8, sc, rows)

    def _reduce(self, x, rows: int):
        """Completes a row-parallel projection (no-op without tensor parallelism)."""
        return x

    def _prep(self, x, norm_w, signs, rows: int, y_out=None):
        """Residual add + RMSNorm + rotation + A8 of a branch output ``x`` (a tensor here;
        tensor-parallel runners may hand over a pending all-reduce instead)."""
        cfg, ws = self.cfg, self.ws
        return F.act_prep(x, ws.resid, norm_w, signs, eps=cfg.eps,
                          zero_centered=cfg.zero_centered_norm, rows=rows,
                          q_out=ws.q8[cfg.hidden], scale_out=ws.scale, y_out=y_out)

    def _row_parallel(self, name: str, lin: QLinear, q8, sc, rows: int):
        """Row-parallel projection into the hidden buffer (then reduced across ranks)."""
        return self._reduce(self._linear(lin, q8, sc, rows, self.ws.hidden), rows)

    def _dense_ffn(self, lw: LayerWeights, x, rows: int):
        cfg, ws = self.cfg, self.ws
        h = cfg.hidden
        q8, sc = self._prep(x, lw.post_norm, self._signs(lw.gate_up), rows)
        f = lw.gate_up.n // 2
        gu = self._linear(lw.gate_up, q8, sc, rows, ws.gate_up.view(-1)[: ws.max_rows * 2 * f]
                          .view(ws.max_rows, 2 * f))
        q8, sc = F.act_prep(gu, None, None, self._signs(lw.down), swiglu=True, rows=rows,
                            q_out=ws.q8[f], scale_out=ws.scale)
        return self._row_parallel("down", lw.down, q8, sc, rows)

    # ---------------------------------------------------------------- forward
    def forward_hidden(self, p: Packet):
        """Runs embedding + all layers; leaves the last branch output in ws.hidden and
        the running residual in ws.resid (final residual = resid + hidden)."""
        cfg, ws, rows = self.cfg, self.ws, p.rows
        if rows > ws.max_rows:
            raise ValueError(f"packet of {rows} rows exceeds workspace ({ws.max_rows})")
        x = F.embed_w8(p.ids, self.w.embed_q, self.w.embed_s, out=ws.hidden)
        if p.overlay_rows is not None:
            x.index_copy_(0, p.overlay_rows, p.overlay.to(x.dtype))
        ws.resid[:rows].zero_()
        self._rope(p, rows)
        hook, self.stage_hook = getattr(self, "stage_hook", None), None
        if (self._fused_decode and rows <= 2 and hook is None and p.attend_pos is None
                and not self.layer_hooks and self._fused_fits(rows)):
            ws.resid[:rows].copy_(x[:rows])             # the stream starts as the embedding
            if self._fused_layer(self.w.layers[0], self._attn_index[0], p, rows):
                for i, lw in enumerate(self.w.layers[1:], 1):
                    self._fused_layer(lw, self._attn_index[i], p, rows)
                return None                             # everything is in ws.resid
            ws.resid[:rows].zero_()                     # shapes do not fit: separate kernels
        pauses = set()
        if hook is not None:
            n = len(self.w.layers)
            pauses = {n * s // hook[0] for s in range(1, hook[0])} - {0}
        for i, lw in enumerate(self.w.layers):
            if i in pauses:
                x = self._pause(p, x, rows, hook[1])
            with trace.span("attn" if lw.kind == "attn" else "gdn"):
                if lw.kind == "attn":
                    x = self._attention_block(lw, self._attn_index[i], x, p, rows, True)
                else:
                    x = self._gdn_block(lw, i, x, p, rows)
            with trace.span("moe_ffn" if cfg.experts else "ffn"):
                if cfg.experts:
                    x = self._moe_ffn(lw, x, rows)
                else:
                    x = self._dense_ffn(lw, x, rows)
        return x

    def enable_expert_pager(self, resident: int):
        """Keeps ``resident`` experts of every MoE layer on the device and the rest in pinned
        host memory (see ``engine.expert_pager``).  The layers' full banks leave the device."""
        from ..engine.expert_pager import ExpertPager
        if getattr(self.w, "tp", None) is not None:
            raise ValueError("expert paging and expert parallelism are exclusive")
        banks = {}
        for lw in self.w.layers:
            if lw.expert_gate_up is not None:
                banks[id(lw)] = (lw.expert_gate_up, lw.expert_down)
        self.pager = ExpertPager(banks, resident, self.device)
        for lw in self.w.layers:                      # free the device copies
            if lw.expert_gate_up is not None:
                res = self.pager.layers[id(lw)]
                lw.expert_gate_up, lw.expert_down = res.host
        torch.cuda.empty_cache() if self.device.type == "cuda" else None
        return self.pager

    supports_stages = True

    def _pause(self, p: Packet, x, rows: int, between):
        """Layer boundary of a layered prefill (``stage_hook = (stages, callback)`` set by the
        caller before the forward): everything a later layer needs from the earlier ones is
        the pending branch output ``x`` and the FP32 residual, so those rows are set aside,
        ``between()`` is free to run other packets through this runner, and the rows and the
        packet's RoPE table are put back.
        Same contract as the reference's resumable prefill stages
        (crates/orinfer-engine/src/runtime/requests/prefill.rs:7-70)."""
        cfg, ws = self.cfg, self.ws
        keep_x, keep_r = x[:rows].clone(), ws.resid[:rows].clone()
        between()
        x[:rows].copy_(keep_x)
        ws.resid[:rows].copy_(keep_r)
        self._rope(p, rows)
        return x

    supports_media = True

    def _rope(self, p: Packet, rows: int) -> None:
        """Fill the rotary tables of the packet: the table kernel for ordinary positions,
        PyTorch for (t, h, w) positions and for partially rotated heads."""
        cfg, ws = self.cfg, self.ws
        if p.mrope is None and not cfg.rotary_dim:
            F.rope_table(p.row_pos, cfg.head_dim, cfg.rope_theta, ws.cos, ws.sin, rows=rows)
            return
        if p.mrope is not None:
            from .vision import mrope_tables
            cos, sin = mrope_tables(p.mrope[:, :rows], cfg.head_dim, cfg.rope_theta)
        else:
            from ..ref.ops_ref import rope_tables
            cos, sin = rope_tables(p.row_pos[:rows], cfg.head_dim, cfg.rope_theta, cfg.rotary_dim)
        ws.cos[:rows].copy_(cos)
        ws.sin[:rows].copy_(sin)

    def _moe_ffn(self, lw: LayerWeights, x, rows: int):
        """norm+rotate+quantise once -> router top-k -> dispatch rows to expert-contiguous
        slots -> grouped gate_up GEMM -> SwiGLU+rotate+quantise -> grouped down GEMM ->
        weighted combine (+ sigmoid-gated shared expert)."""
        cfg, ws = self.cfg, self.ws
        h, f = cfg.hidden, cfg.expert_ffn
        if getattr(ws, "moe", None) is None:
            ws.moe = F.MoeScratch(ws.max_rows, cfg.top_k, cfg.experts, h, f, self.device)
            ws.moe_out = torch.empty(ws.max_rows, h, dtype=torch.float16, device=self.device)
            ws.shared_out = torch.empty(ws.max_rows, h, dtype=torch.float16, device=self.device)
        sc = ws.moe
        bank_up, bank_dn = lw.expert_gate_up, lw.expert_down
        y16 = ws.attn_norm(rows, h)
        q8, s8 = self._prep(x, lw.post_norm, bank_up.signs, rows, y_out=y16)
        F.router_topk(y16, lw.router, cfg.experts, cfg.top_k, renorm=cfg.renormalize, rows=rows,
                      ids=sc.ids, probs=sc.probs, gate=sc.gate)
        pager = getattr(self, "pager", None)
        if pager is not None:
            # bounded residency: the routed experts are paged into slot banks and the ids
            # become slot ids; everything after the router runs on the slot banks
            bank_up, bank_dn, slot_ids = pager.page_in(id(lw), sc.ids, rows)
            F.moe_dispatch(slot_ids, q8, s8, bank_up.experts, sc, rows, 0, bank_up.experts)
        else:
            F.moe_dispatch(sc.ids, q8, s8, cfg.experts, sc, rows, bank_up.base, bank_up.experts)
        total = rows * cfg.top_k
        F.qgemm_grouped(sc.q8, sc.scale, bank_up.codes, bank_up.scale, bank_up.fmt, 2 * f,
                        sc.gate_up, sc, total)
        # offsets[n_local_experts] = rows actually routed to this rank's experts
        F.act_prep_limited(sc.gate_up, bank_dn.signs, sc.offsets[bank_up.experts:], swiglu=True,
                           rows=total, q_out=sc.q8_mid, scale_out=sc.scale_mid)
        F.qgemm_grouped(sc.q8_mid, sc.scale_mid, bank_dn.codes, bank_dn.scale, bank_dn.fmt, h,
                        sc.down, sc, total)
        shared = None
        tp = getattr(self.w, "tp", None)
        if lw.shared_gate_up is not None and (tp is None or lw.shared_owner in (-1, tp.rank)):
            fs = lw.shared_gate_up.n // 2
            gu = self._linear(lw.shared_gate_up, q8, s8, rows,
                              ws.gate_up.view(-1)[: ws.max_rows * 2 * fs].view(ws.max_rows, 2 * fs))
            q8s, s8s = F.act_prep(gu, None, None, self._signs(lw.shared_down), swiglu=True,
                                  rows=rows, q_out=ws.q8[fs], scale_out=ws.scale)
            shared = self._linear(lw.shared_down, q8s, s8s, rows, ws.shared_out)
        has_gate = lw.router.shape[0] == cfg.experts + 1
        return self._moe_combine(sc, shared, sc.gate if has_gate and shared is not None else None,
                                 rows)

    def _moe_combine(self, sc, shared, gate, rows: int):
        """Weighted sum of the routed expert rows (+ gated shared expert) into the hidden
        buffer; expert-parallel runners complete it across ranks."""
        F.moe_combine(sc.down, sc.slots, sc.probs, shared, gate, self.ws.hidden, rows)
        return self._reduce(self.ws.hidden, rows)

    def logits(self, p: Packet, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """fp32 logits [n_sel, vocab] of the selected rows (final norm + W8 head)."""
        return self._head(self.forward_hidden(p), p, out)

    def _head(self, x, p: Packet, out: Optional[torch.Tensor]) -> torch.Tensor:
        cfg, ws = self.cfg, self.ws
        rows = p.rows
        if p.logit_rows is not None or not isinstance(x, torch.Tensor):
            # final norm over every row (fp16 result), then pick the rows that need logits
            self._prep(x, self.w.final_norm, None, rows, y_out=ws.attn_norm(rows, cfg.hidden))
            y = ws.attn_norm(rows, cfg.hidden)[:rows]
            if p.logit_rows is not None:
                y = y.index_select(0, p.logit_rows).contiguous()
                rows = p.logit_rows.shape[0]
            q8, sc = F.act_prep(y, None, None, self.w.head.signs, rows=rows,
                                q_out=ws.q8[cfg.hidden], scale_out=ws.scale)
        else:
            q8, sc = self._prep(x, self.w.final_norm, self.w.head.signs, rows)
        if out is None:
            out = torch.empty(rows, self.w.head.n, dtype=torch.float32, device=self.device)
        return F.qgemm(q8, sc, self.w.head.codes, self.w.head.scale, self.w.head.fmt,
                       self.w.head.n, out=out, out_f32=True, rows=rows)

    def greedy(self, p: Packet, logits_out=None, token_out=None, need_logits: bool = True):
        lg = self.logits(p, logits_out)
        return F.argmax(lg, out=token_out), lg

    # ---------------------------------------------------------------- MTP draft head
    def final_hidden(self, rows: int) -> torch.Tensor:
        """Residual stream entering the final norm, for the rows of the last packet."""
        return self.ws.resid[:rows]

    def mtp_rows(self, tokens: torch.Tensor, hidden: torch.Tensor, p: Packet):
        """One pass of the draft head over ``p.rows`` rows: row i combines the embedding of
        ``tokens[i]`` (the token that FOLLOWS position ``p.row_pos[i]``) with the target
        model's hidden state at that position, writes the draft layer's KV at that position
        and predicts the token after next.  Returns (draft tokens, draft hidden fp32).
        concat(norm_e(embed), norm_h(hidden)) -> fc -> one decoder layer -> norm -> shared head
        (kernels/cuda/model/speculation.py:31 mtp_norm_concat of the reference)."""
        cfg, ws, m, rows = self.cfg, self.ws, self.w.mtp, p.rows
        h = cfg.hidden
        if getattr(ws, "mtp_buf", None) is None:
            e = lambda *s, dt=torch.float16: torch.empty(*s, dtype=dt, device=self.device)
            ws.mtp_buf = dict(e=e(ws.max_rows, h), ye=e(ws.max_rows, h), yh=e(ws.max_rows, h),
                              r=e(ws.max_rows, h, dt=torch.float32),
                              resid=e(ws.max_rows, h, dt=torch.float32))
        b = ws.mtp_buf
        F.embed_w8(tokens, self.w.embed_q, self.w.embed_s, out=b["e"])
        F.act_prep(b["e"], None, m.norm_e, None, eps=cfg.eps, rows=rows, q_out=ws.q8[h],
                   scale_out=ws.scale, y_out=b["ye"])
        b["r"][:rows].copy_(hidden[:rows])
        F.act_prep(None, b["r"], m.norm_h, None, eps=cfg.eps, rows=rows, q_out=ws.q8[h],
                   scale_out=ws.scale, y_out=b["yh"])
        cat = torch.cat([b["ye"][:rows], b["yh"][:rows]], dim=1).contiguous()
        q8, sc = F.act_prep(cat, None, None, m.fc.signs, rows=rows)
        x = F.qgemm(q8, sc, m.fc.codes, m.fc.scale, m.fc.fmt, m.fc.n, out=ws.hidden, rows=rows)
        saved = ws.resid
        ws.resid = b["resid"]
        try:
            ws.resid[:rows].zero_()
            self._rope(p, rows)
            x = self._attention_block(m.layer, self.mtp_kv_index, x, p, rows, True)
            if m.layer.router is not None:       # a draft layer with routed experts
                x = self._moe_ffn(m.layer, x, rows)
            else:
                x = self._dense_ffn(m.layer, x, rows)
            q8, sc = self._prep(x, m.final_norm, self.w.head.signs, rows)
            lg = F.qgemm(q8, sc, self.w.head.codes, self.w.head.scale, self.w.head.fmt,
                         self.w.head.n, out_f32=True, rows=rows)
            hid = ws.resid[:rows].clone()
        finally:
            ws.resid = saved
        return self._draft_tokens(lg[:rows]), hid

    def _draft_tokens(self, logits: torch.Tensor) -> torch.Tensor:
        """Greedy draft tokens from the head's logits (tensor-parallel runners merge the
        ranks' vocabulary shards here)."""
        return F.argmax(logits)
