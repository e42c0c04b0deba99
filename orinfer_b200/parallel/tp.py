"""Tensor-parallel sharding of a quantised model (Megatron layout).

* qkv and gate_up are column-parallel: every rank keeps the output rows of its own
  query / KV heads and its own slice of the FFN width;
* o and down are row-parallel: every rank keeps a slice of the input channels (whole
  128-channel rotation blocks, so the block Hadamard stays rank-local) and produces a
  partial sum that a reduce-scatter / all-reduce completes;
* the head is vocabulary-sharded; ranks exchange only (max, argmax) per row for greedy
  decoding, as the reference's TP head does (kernels/ascend/topk.py:74-100).

The reference shards its Ascend TP8 plans the same way: ``wo_a`` by output rows,
``wo_b`` by input columns, the head by vocabulary
(python/orinfer_build/models/deepseek_v41/build.py:1086-1110,1498).
"""

from __future__ import annotations

import dataclasses
from typing import List, Optional, Tuple

import torch

from ..config import ModelConfig
from ..models.weights import LayerWeights, ModelWeights, MtpWeights, QLinear


def split_blocks(total_blocks: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous, near-even split of ``total_blocks`` into ``world`` ranges."""
    base, extra = divmod(total_blocks, world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((start, start + n))
        start += n
    return out


def _rows(lin: QLinear, idx: torch.Tensor) -> QLinear:
    """Keep output rows ``idx`` (column-parallel shard)."""
    if lin.fmt == "w8":
        codes = lin.codes.index_select(0, idx).contiguous()
    else:
        codes = lin.codes.index_select(1, idx).contiguous()
    dense = None if lin.dense is None else lin.dense.index_select(0, idx.cpu())
    return QLinear(lin.fmt, int(idx.numel()), lin.k, codes, lin.scale.index_select(0, idx),
                   lin.signs, dense)


def _cols(lin: QLinear, lo: int, hi: int) -> QLinear:
    """Keep input channels [lo, hi) (row-parallel shard); lo, hi multiples of 128."""
    if lin.fmt == "w8":
        codes = lin.codes[:, lo:hi].contiguous()
    else:
        codes = lin.codes[lo // 128:hi // 128].contiguous()
    signs = None if lin.signs is None else lin.signs[lo:hi].contiguous()
    dense = None if lin.dense is None else lin.dense[:, lo:hi].contiguous()
    return QLinear(lin.fmt, lin.n, hi - lo, codes, lin.scale, signs, dense)


@dataclasses.dataclass
class TPLayout:
    rank: int
    world: int
    q_heads: int                 # local query heads
    kv_heads: int                # local KV heads (>= 1; replicated when kv_heads < world)
    ffn: Tuple[int, int]         # local slice of the FFN width (channels)
    vocab: Tuple[int, int]       # local slice of the vocabulary


def layout(cfg: ModelConfig, rank: int, world: int) -> TPLayout:
    if cfg.q_heads % world:
        raise ValueError(f"{cfg.q_heads} query heads do not split over {world} ranks")
    if cfg.kv_heads % world and world % cfg.kv_heads:
        raise ValueError("KV heads must divide or be divided by the TP degree")
    blocks = split_blocks((cfg.ffn or 128) // 128, world)[rank]
    v = split_blocks(cfg.vocab // 128, world)[rank]
    return TPLayout(rank, world, cfg.q_heads // world, max(cfg.kv_heads // world, 1),
                    (blocks[0] * 128, blocks[1] * 128), (v[0] * 128, v[1] * 128))


def _shard_attention(cfg: ModelConfig, lw: LayerWeights, lay: TPLayout, dev) -> None:
    d = cfg.head_dim
    qs = d * (2 if cfg.gated_attention and lw.qkv.n == cfg.q_dim + 2 * cfg.kv_dim else 1)
    q_total = cfg.q_heads * qs
    q0 = lay.rank * lay.q_heads
    kv0 = (lay.rank * cfg.kv_heads) // lay.world if cfg.kv_heads < lay.world \
        else lay.rank * lay.kv_heads
    ar = lambda a, b: torch.arange(a, b, device=dev)
    idx = torch.cat([ar(q0 * qs, (q0 + lay.q_heads) * qs),
                     ar(q_total + kv0 * d, q_total + (kv0 + lay.kv_heads) * d),
                     ar(q_total + cfg.kv_dim + kv0 * d,
                        q_total + cfg.kv_dim + (kv0 + lay.kv_heads) * d)])
    lw.qkv = _rows(lw.qkv, idx)
    lw.o = _cols(lw.o, q0 * d, (q0 + lay.q_heads) * d)


def _shard_ffn(lw: LayerWeights, lay: TPLayout, dev) -> None:
    f = lw.gate_up.n // 2
    lo, hi = lay.ffn
    idx = torch.cat([torch.arange(lo, hi, device=dev), torch.arange(f + lo, f + hi, device=dev)])
    lw.gate_up = _rows(lw.gate_up, idx)
    lw.down = _cols(lw.down, lo, hi)


def shard_model(weights: ModelWeights, rank: int, world: int) -> ModelWeights:
    """Returns this rank's shard; ``weights.config`` becomes the *local* geometry
    (local head counts, local FFN width) while ``vocab`` stays global."""
    cfg = weights.config
    if cfg.arch != "dense":
        raise NotImplementedError("tensor parallelism is implemented for dense decoders")
    lay = layout(cfg, rank, world)
    dev = weights.embed_q.device
    layers = []
    for lw in weights.layers:
        lw = dataclasses.replace(lw)
        _shard_attention(cfg, lw, lay, dev)
        _shard_ffn(lw, lay, dev)
        layers.append(lw)
    v0, v1 = lay.vocab
    head = _rows(weights.head, torch.arange(v0, v1, device=dev))
    local = dataclasses.replace(cfg, q_heads=lay.q_heads, kv_heads=lay.kv_heads,
                                ffn=lay.ffn[1] - lay.ffn[0], mtp_layers=0)
    out = ModelWeights(local, weights.embed_q, weights.embed_s, layers, weights.final_norm, head,
                       weights.signs, None, weights.embed_dense)
    out.tp = lay                       # type: ignore[attr-defined]
    out.global_config = cfg            # type: ignore[attr-defined]
    return out
