"""Packed-row forward in plain PyTorch over the same paged INT8 KV layout.

Drop-in stand-in for :class:`ModelRunner` on machines without a GPU (engine tests,
the timed CPU baseline) and the batch-invariance oracle for the CUDA path: it is
built from ``ops_ref`` only, so it computes what the kernels are specified to
compute.  Plays the role of the reference's single-request generation path used as
isolation oracle (crates/orinfer-engine/src/runtime/reference_generation.rs:5-6).
"""

from __future__ import annotations

from typing import Optional

import torch

from ..config import ModelConfig
from ..ref import ops_ref as R
from .runner import KVPool, Packet
from .weights import LayerWeights, ModelWeights, QLinear


class TorchRunner:
    def __init__(self, weights: ModelWeights, kv: KVPool, max_rows: int):
        self.w, self.cfg, self.kv = weights, weights.config, kv
        self.device = weights.embed_q.device
        self.max_rows = max_rows
        self._ints = {}
        self._attn_index = {}
        n = 0
        for i in range(self.cfg.layers):
            if self.cfg.is_full_attention(i):
                self._attn_index[i] = n
                n += 1
        self.mtp_kv_index = n
        self.layer_hooks = {}

    def _w(self, lin: QLinear) -> torch.Tensor:
        key = id(lin.codes)
        if key not in self._ints:
            self._ints[key] = lin.integers()
        return self._ints[key]

    def _linear(self, lin: QLinear, y: torch.Tensor, out_f32: bool = False) -> torch.Tensor:
        z = R.hadamard_rotate(y, lin.signs) if lin.signs is not None else y
        q, s = R.a8(z)
        return R.qgemm(q, s, self._w(lin), lin.scale, out_f32)

    def _attention(self, lw: LayerWeights, slot: int, y: torch.Tensor, p: Packet, cos, sin):
        cfg = self.cfg
        rows, d, qh, kvh = p.rows, cfg.head_dim, cfg.q_heads, cfg.kv_heads
        proj = self._linear(lw.qkv, y)
        gated = cfg.gated_attention and lw.qkv.n == cfg.q_dim + 2 * cfg.kv_dim
        qw = qh * d * (2 if gated else 1)
        gate = None
        if gated:
            qg = proj[:, :qw].reshape(rows, qh, 2 * d)
            q, gate = qg[..., :d], qg[..., d:]
        else:
            q = proj[:, :qw].reshape(rows, qh, d)
        k = proj[:, qw:qw + kvh * d].reshape(rows, kvh, d)
        v = proj[:, qw + kvh * d:].reshape(rows, kvh, d)
        qn = R.qk_norm_rope(q, lw.q_norm if cfg.qk_norm else None, cos, sin, cfg.eps,
                            cfg.zero_centered_norm)
        kn = R.qk_norm_rope(k, lw.k_norm if cfg.qk_norm else None, cos, sin, cfg.eps,
                            cfg.zero_centered_norm)
        kq, ks = R.kv_quant(kn)
        vq, vs = R.kv_quant(R.f16(v.float()))
        req, pos = p.row_req[:rows].long(), p.row_pos[:rows].long()
        page = p.page_table[req, pos // 128].long()
        off = pos % 128
        self.kv.k[slot][page, off] = kq
        self.kv.v[slot][page, off] = vq
        self.kv.ks[slot][page, off] = ks.to(torch.float16)
        self.kv.vs[slot][page, off] = vs.to(torch.float16)
        out = torch.empty(rows, qh * d)
        see = pos if p.attend_pos is None else p.attend_pos[:rows].long()
        for r in torch.unique(req).tolist():
            idx = (req == r).nonzero().flatten()
            rp = see[idx]
            kv_len = int(rp.max()) + 1
            allpos = torch.arange(kv_len)
            pg = p.page_table[r, allpos // 128].long()
            kk = R.kv_dequant(self.kv.k[slot][pg, allpos % 128], self.kv.ks[slot][pg, allpos % 128])
            vv = R.kv_dequant(self.kv.v[slot][pg, allpos % 128], self.kv.vs[slot][pg, allpos % 128])
            for j, i in enumerate(idx.tolist()):
                n = int(rp[j]) + 1
                out[i] = R.causal_gqa(qn[i:i + 1], kk[:n], vv[:n], n - 1,
                                      None if gate is None else gate[i:i + 1])[0]
        return out

    def _gdn(self, lw: LayerWeights, layer: int, y: torch.Tensor, p: Packet) -> torch.Tensor:
        """Gated-delta-rule mixer per run of rows of one request; the recurrent state and the
        convolution history live per page-table row and restart when a run begins at
        position 0."""
        from ..ref import gdn_ref as G
        cfg = self.cfg
        hk, hv, d = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
        dk, conv_dim = hk * d, (2 * hk + hv) * d
        if not hasattr(self, "_gdn_pool"):
            self._gdn_pool = {}
        proj = self._linear(lw.gdn_qkvz, y)
        ab = R.f16(y).float() @ lw.gdn_ab.float().t()
        g, beta = G.gates(ab, lw.gdn_a_log, lw.gdn_dt_bias)
        p.ensure_segments()
        out = torch.empty(p.rows, hv * d)
        if p.tentative:
            self._gdn_journal = getattr(self, "_gdn_journal", {})
        for si, (start, n, _a, _b) in enumerate(p.segments.tolist()):
            slot, pos0 = int(p.row_req[start]), int(p.row_pos[start])
            key = (layer, slot)
            if pos0 == 0 or key not in self._gdn_pool:
                self._gdn_pool[key] = (torch.zeros(hv, d, d), torch.zeros(3, conv_dim))
            state, hist = self._gdn_pool[key]
            sl = slice(start, start + n)
            if p.tentative:                      # verification pass: remember how to redo a prefix
                self._gdn_journal[(layer, si)] = (key, proj[sl, :conv_dim].clone(), g[sl].clone(),
                                                  beta[sl].clone(), lw)
            yc, hist = G.conv_silu_l2(proj[sl, :conv_dim], hist, lw.gdn_conv, dk, d)
            o, state = G.recurrence(yc[:, :dk].reshape(n, hk, d), yc[:, dk:2 * dk].reshape(n, hk, d),
                                    yc[:, 2 * dk:].reshape(n, hv, d), g[sl], beta[sl], state)
            if not p.tentative:
                self._gdn_pool[key] = (state, hist)
            out[sl] = G.gated_norm(o, proj[sl, conv_dim:].reshape(n, hv, d), lw.gdn_norm, cfg.eps)
        return out

    def gdn_snapshot(self, slot: int):
        """Copy of the recurrent state of one request slot (every GDN layer)."""
        keys = sorted(k for k in self._gdn_pool if k[1] == slot)
        return ([k[0] for k in keys], [self._gdn_pool[k][0].clone() for k in keys],
                [self._gdn_pool[k][1].clone() for k in keys])

    def gdn_restore(self, slot: int, snap, slots: int = 0) -> None:
        for layer, state, hist in zip(*snap):
            self._gdn_pool[(layer, slot)] = (state.clone(), hist.clone())

    def gdn_commit(self, p: Packet, accepted_rows) -> None:
        """Keeps the first ``accepted_rows[s]`` rows of every segment of a tentative packet."""
        from ..ref import gdn_ref as G
        cfg = self.cfg
        hk, hv, d = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
        dk = hk * d
        accepted_rows = list(accepted_rows)
        for (layer, si), (key, x, g, beta, lw) in getattr(self, "_gdn_journal", {}).items():
            a = min(accepted_rows[si], x.shape[0])
            if a <= 0:
                continue
            state, hist = self._gdn_pool[key]
            yc, hist = G.conv_silu_l2(x[:a], hist, lw.gdn_conv, dk, d)
            _, state = G.recurrence(yc[:, :dk].reshape(a, hk, d), yc[:, dk:2 * dk].reshape(a, hk, d),
                                    yc[:, 2 * dk:].reshape(a, hv, d), g[:a], beta[:a], state)
            self._gdn_pool[key] = (state, hist)
        self._gdn_journal = {}

    def _reduce(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def _ffn(self, lw: LayerWeights, y: torch.Tensor) -> torch.Tensor:
        gu = self._linear(lw.gate_up, y)
        f = gu.shape[-1] // 2
        return self._reduce(self._linear(lw.down, R.silu_mul(gu[:, :f], gu[:, f:])))

    supports_stages = True
    supports_media = True

    def forward_hidden(self, p: Packet):
        cfg = self.cfg
        rows = p.rows
        x = R.embed_w8(p.ids[:rows], self.w.embed_q, self.w.embed_s)
        if p.overlay_rows is not None:
            x = x.index_copy(0, p.overlay_rows, p.overlay.to(x.dtype))
        resid = torch.zeros(rows, cfg.hidden)
        if p.mrope is None:
            cos, sin = R.rope_tables(p.row_pos[:rows], cfg.head_dim, cfg.rope_theta, cfg.rotary_dim)
        else:
            from .vision import mrope_tables
            cos, sin = mrope_tables(p.mrope[:, :rows], cfg.head_dim, cfg.rope_theta)
        zc = cfg.zero_centered_norm
        hook, self.stage_hook = getattr(self, "stage_hook", None), None
        pauses = set()
        if hook is not None:                     # layered prefill: see ModelRunner._pause
            n = len(self.w.layers)
            pauses = {n * s // hook[0] for s in range(1, hook[0])} - {0}
        for i, lw in enumerate(self.w.layers):
            if i in pauses:
                hook[1]()                        # x and resid are private to this call
            resid = resid + x
            y = R.rms_norm(resid, lw.in_norm, cfg.eps, zc)
            if lw.kind == "attn":
                mix = self._attention(lw, self._attn_index[i], y, p, cos, sin)
                x = self._reduce(self._linear(lw.o, mix))
            else:
                x = self._reduce(self._linear(lw.gdn_out, self._gdn(lw, i, y, p)))
            resid = resid + x
            y = R.rms_norm(resid, lw.post_norm, cfg.eps, zc)
            if cfg.experts:
                from ..ref.cpu_forward import moe_ffn
                tp = getattr(self.w, "tp", None)       # replicated shared expert: owner adds it
                lw._add_shared = tp is None or lw.shared_owner in (-1, tp.rank)
                x = self._reduce(moe_ffn(cfg, lw, y, True))
            else:
                x = self._ffn(lw, y)
        return x, resid

    def logits(self, p: Packet, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        x, resid = self.forward_hidden(p)
        final = resid + x
        self._final = final
        if p.logit_rows is not None:
            final = final.index_select(0, p.logit_rows.long())
        h = R.rms_norm(final, self.w.final_norm, self.cfg.eps, self.cfg.zero_centered_norm)
        lg = self._linear(self.w.head, h, out_f32=True)
        if out is not None:
            out[:lg.shape[0]].copy_(lg)
        return lg

    def greedy(self, p: Packet, logits_out=None, token_out=None, need_logits: bool = True):
        lg = self.logits(p, logits_out)
        tok = R.argmax_lowest(lg)
        if token_out is not None:
            token_out[:tok.shape[0]].copy_(tok)
        return tok, lg

    # ---------------------------------------------------------------- MTP draft head
    def final_hidden(self, rows: int) -> torch.Tensor:
        return self._final[:rows]

    def mtp_rows(self, tokens: torch.Tensor, hidden: torch.Tensor, p: Packet):
        """Same contract as ModelRunner.mtp_rows, in plain PyTorch."""
        cfg, m, rows = self.cfg, self.w.mtp, p.rows
        zc = cfg.zero_centered_norm
        e = R.embed_w8(tokens[:rows], self.w.embed_q, self.w.embed_s)
        ye = R.rms_norm(e, m.norm_e, cfg.eps, zc)
        yh = R.rms_norm(hidden[:rows].float(), m.norm_h, cfg.eps, zc)
        x = self._linear(m.fc, torch.cat([ye, yh], dim=1))
        cos, sin = R.rope_tables(p.row_pos[:rows], cfg.head_dim, cfg.rope_theta, cfg.rotary_dim)
        resid = x
        y = R.rms_norm(resid, m.layer.in_norm, cfg.eps, zc)
        mix = self._attention(m.layer, self.mtp_kv_index, y, p, cos, sin)
        x = self._reduce(self._linear(m.layer.o, mix))
        resid = resid + x
        y = R.rms_norm(resid, m.layer.post_norm, cfg.eps, zc)
        if m.layer.router is not None:           # a draft layer with routed experts
            from ..ref.cpu_forward import moe_ffn
            tp = getattr(self.w, "tp", None)
            m.layer._add_shared = tp is None or m.layer.shared_owner in (-1, tp.rank)
            x = self._reduce(moe_ffn(cfg, m.layer, y, True))
        else:
            x = self._ffn(m.layer, y)
        final = resid + x
        lg = self._linear(self.w.head, R.rms_norm(final, m.final_norm, cfg.eps, zc), out_f32=True)
        return self._draft_tokens(lg), final

    def _draft_tokens(self, logits: torch.Tensor) -> torch.Tensor:
        """Greedy draft tokens from the head's logits (tensor-parallel runners merge the
        ranks' vocabulary shards here)."""
        return R.argmax_lowest(logits)
