"""Tensor-parallel runners: one process per GPU, ``torch.distributed`` for plumbing.

``TPRunner`` is the NCCL-only arm (all-reduce after every row-parallel projection,
all-gather of per-rank (max, argmax) for the vocabulary-sharded head): it is the
*baseline* that the fused compute+collective kernels in ``fused.py`` are measured
against, and the fallback when peer memory cannot be mapped.  ``TPTorchRunner`` is the
same arithmetic on CPU ranks (gloo) for tests.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..models.runner import KVPool, ModelRunner, Packet
from ..models.torch_runner import TorchRunner
from ..models.weights import ModelWeights
from ..ops import functional as F
from ..ref import ops_ref as R


def merge_sharded_argmax(values: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """values/tokens: [world, rows] per-rank maxima and *global* token ids (-1 = invalid
    row on that rank).  Global greedy token = largest value, lowest id on ties; any
    invalid shard invalidates the row."""
    best = values.max(dim=0).values
    big = torch.iinfo(torch.int32).max
    cand = torch.where(values == best[None], tokens, torch.full_like(tokens, big))
    tok = cand.min(dim=0).values
    return torch.where((tokens < 0).any(dim=0), torch.full_like(tok, -1), tok)


class _TPMixin:
    group: Optional[dist.ProcessGroup]

    def _init_tp(self, weights: ModelWeights, group):
        self.group = group
        self.tp = weights.tp
        self.world = self.tp.world
        self.vocab0 = self.tp.vocab[0]
        self.global_vocab = weights.global_config.vocab

    def _gather_logits(self, local: torch.Tensor) -> torch.Tensor:
        """[rows, V/tp] -> [rows, V] (ranks own contiguous vocabulary ranges; the shards
        may differ by one 128-block in width, so gather padded and trim)."""
        rows = local.shape[0]
        widths = [b - a for a, b in
                  (self._vocab_range(r) for r in range(self.world))]
        wmax = max(widths)
        pad = torch.full((rows, wmax), float("-inf"), dtype=local.dtype, device=local.device)
        pad[:, :local.shape[1]] = local
        parts = [torch.empty_like(pad) for _ in range(self.world)]
        dist.all_gather(parts, pad, group=self.group)
        return torch.cat([p[:, :w] for p, w in zip(parts, widths)], dim=1)

    def sample_sharded(self, rows, options, uniforms):
        """Tokens for the selected rows of the last forward, drawn from the sharded logits
        (only top-k candidates cross ranks).  Collective: every rank calls it alike."""
        from . import sharded_sampling
        idx = torch.tensor(list(rows), dtype=torch.int64, device=self._last_local.device)
        return sharded_sampling.sample_rows(self._last_local.index_select(0, idx), self.vocab0,
                                            options, uniforms, self.group)

    def _vocab_range(self, rank: int):
        from .tp import split_blocks
        a, b = split_blocks(self.global_vocab // 128, self.world)[rank]
        return a * 128, b * 128

    def _merge_tokens(self, local_logits: torch.Tensor, local_tok: torch.Tensor) -> torch.Tensor:
        rows = local_tok.shape[0]
        safe = local_tok.clamp(min=0).long()
        val = local_logits.gather(1, safe[:, None])[:, 0]
        tok = torch.where(local_tok >= 0, local_tok + self.vocab0, local_tok)
        pack = torch.stack([val, tok.to(val.dtype)], dim=1)            # ids < 2^24: exact
        parts = [torch.empty_like(pack) for _ in range(self.world)]
        dist.all_gather(parts, pack, group=self.group)
        allp = torch.stack(parts)                                      # [world, rows, 2]
        return merge_sharded_argmax(allp[..., 0], allp[..., 1].to(torch.int32)).to(torch.int32)


class TPRunner(_TPMixin, ModelRunner):
    # NOTE: the draft head (``mtp_rows``) of a sharded model runs the inherited code: its
    # row-parallel projections end in ``_reduce`` and its tokens go through ``_draft_tokens``.

    """NCCL-only tensor-parallel runner (baseline arm)."""

    def __init__(self, weights: ModelWeights, kv: KVPool, max_rows: int, group=None):
        ModelRunner.__init__(self, weights, kv, max_rows)
        self._init_tp(weights, group)
        import os
        self._exact_reduce = os.environ.get("ORINFER_TP_EXACT_REDUCE") == "1"

    def _reduce(self, x, rows: int):
        if self._exact_reduce:
            # same arithmetic as the fused path's consumer: FP16 partials summed in FP32 in
            # rank order, rounded once; lets tests compare the two arms bit for bit
            parts = [torch.empty_like(x[:rows]) for _ in range(self.world)]
            dist.all_gather(parts, x[:rows].contiguous(), group=self.group)
            acc = parts[0].float()
            for p in parts[1:]:
                acc += p.float()
            x[:rows].copy_(acc.to(x.dtype))
            return x
        dist.all_reduce(x[:rows], group=self.group)
        return x

    def _draft_tokens(self, logits: torch.Tensor) -> torch.Tensor:
        return self._merge_tokens(logits, F.argmax(logits))

    def greedy(self, p: Packet, logits_out=None, token_out=None, need_logits: bool = True):
        local = self._last_local = self.logits(p)                      # [n_sel, V/tp]
        tok = self._merge_tokens(local, F.argmax(local))
        if token_out is not None:
            token_out[:tok.shape[0]].copy_(tok)
            tok = token_out
        full = None
        if need_logits:
            full = self._gather_logits(local)
            if logits_out is not None:
                logits_out[:full.shape[0]].copy_(full)
                full = logits_out
        return tok, full


class TPTorchRunner(_TPMixin, TorchRunner):
    """CPU ranks over gloo: same sharded arithmetic, for tests without GPUs."""

    def __init__(self, weights: ModelWeights, kv: KVPool, max_rows: int, group=None):
        TorchRunner.__init__(self, weights, kv, max_rows)
        self._init_tp(weights, group)

    def _reduce(self, x: torch.Tensor) -> torch.Tensor:
        # ranks add FP16-rounded partials in fp32, then round once (as the device path does)
        y = x.float().contiguous()
        dist.all_reduce(y, group=self.group)
        return R.f16(y)

    def _draft_tokens(self, logits: torch.Tensor) -> torch.Tensor:
        return self._merge_tokens(logits, R.argmax_lowest(logits))

    def greedy(self, p: Packet, logits_out=None, token_out=None, need_logits: bool = True):
        local = self._last_local = self.logits(p)
        tok = self._merge_tokens(local, R.argmax_lowest(local))
        full = self._gather_logits(local) if need_logits else None
        return tok, full
