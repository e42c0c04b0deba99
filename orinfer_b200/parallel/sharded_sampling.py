"""Sampling over a vocabulary-sharded head without gathering the logits.

Every rank holds the logits of its own vocabulary range.  For a request whose law is a
temperature / top-k / top-p categorical with ``1 <= top_k <= 64`` and no host-side score
rewriting, the global top-k is contained in the union of the ranks' local top-k lists, so
ranks exchange ``rows x k`` (logit, token id) pairs instead of ``rows x vocab / tp`` logits.
Each rank then applies the ordinary host law (``core.sampling.sample``) to the merged
candidates with the request's counter-RNG uniform: the token is the very one a single device
would have drawn from the full row, ties included (candidates keep ascending-id order, the
order in which the law breaks ties).

Counterpart of the reference's TP-sharded sampler, where only log-sum-exp terms and selected
candidates cross ranks (crates/orinfer-engine/src/backend/ascend/sampling*.rs,
kernels/ascend/sampling*.py).
"""

from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch
import torch.distributed as dist

from ..core import sampling as S

MAX_K = 64


def local_candidates(local: torch.Tensor, k: int, vocab0: int):
    """Top ``k`` of every row of this rank's shard: (values fp32 [rows, k], global ids int32
    [rows, k]); among equal logits the lowest id comes first (stable sort)."""
    k = min(k, local.shape[1])
    order = torch.sort(local.float(), dim=1, descending=True, stable=True)
    return order.values[:, :k].contiguous(), (order.indices[:, :k] + vocab0).to(torch.int32)


def merge_candidates(values: torch.Tensor, ids: torch.Tensor, k: int):
    """values / ids: [rows, n] candidates of all ranks.  -> the k best per row by (logit
    descending, id ascending), returned in ascending-id order."""
    # sort by id first, then stably by value: equal values stay in ascending-id order
    by_id = torch.sort(ids, dim=1, stable=True)
    v = values.gather(1, by_id.indices)
    by_val = torch.sort(v, dim=1, descending=True, stable=True)
    top_ids = by_id.values.gather(1, by_val.indices)[:, :k]
    top_val = by_val.values[:, :k]
    again = torch.sort(top_ids, dim=1)
    return top_val.gather(1, again.indices), again.values


def sample_rows(local: torch.Tensor, vocab0: int, options: Sequence[S.SamplingOptions],
                uniforms: Sequence[float], group=None) -> List[int]:
    """One token per row of ``local`` [rows, V/tp] (this rank's logits), identical on every
    rank.  All options must satisfy ``SamplingOptions.device_topk``."""
    for o in options:
        if not o.device_topk:
            raise ValueError("sharded sampling serves temperature/top-k/top-p laws only")
    k = max(o.top_k for o in options)
    vals, ids = local_candidates(local, k, vocab0)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world > 1:
        width = torch.tensor([vals.shape[1]], dtype=torch.int64, device=vals.device)
        widths = [torch.empty_like(width) for _ in range(world)]
        dist.all_gather(widths, width, group=group)
        wmax = max(int(w) for w in widths)                 # shards may differ in width
        pv = torch.full((vals.shape[0], wmax), float("-inf"), device=vals.device)
        pi = torch.full((vals.shape[0], wmax), torch.iinfo(torch.int32).max, dtype=torch.int32,
                        device=vals.device)
        pv[:, :vals.shape[1]], pi[:, :ids.shape[1]] = vals, ids
        gv = [torch.empty_like(pv) for _ in range(world)]
        gi = [torch.empty_like(pi) for _ in range(world)]
        dist.all_gather(gv, pv, group=group)
        dist.all_gather(gi, pi, group=group)
        vals, ids = torch.cat(gv, dim=1), torch.cat(gi, dim=1)
    vals, ids = merge_candidates(vals, ids, k)
    vals, ids = vals.cpu().numpy(), ids.cpu().numpy()
    out = []
    for row, (o, u) in enumerate(zip(options, uniforms)):
        keep = np.isfinite(vals[row])
        pick = S.sample(vals[row][keep], [], o, u)
        out.append(int(ids[row][keep][pick]))
    return out
