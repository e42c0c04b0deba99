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
from ..models.weights import ExpertBank, LayerWeights, ModelWeights, MtpWeights, QLinear


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


def _shard_gdn(cfg: ModelConfig, lw: LayerWeights, lay: TPLayout, dev) -> None:
    """Linear-attention heads are split over the ranks (no collective inside the mixer):
    q|k|v|z projection rows, gate rows, convolution channels and per-head scalars follow
    their heads; the output projection is row-parallel."""
    w, r = lay.world, lay.rank
    hk, hv, d = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
    if hk % w or hv % w or (hv // w * d) % 128:
        raise ValueError(f"GDN heads ({hk} key, {hv} value) do not split over {w} ranks")
    lk, lv = hk // w, hv // w
    ar = lambda a, n: torch.arange(a, a + n, device=dev)
    q_i = ar(r * lk * d, lk * d)
    k_i = ar(hk * d + r * lk * d, lk * d)
    v_i = ar(2 * hk * d + r * lv * d, lv * d)
    z_i = ar(2 * hk * d + hv * d + r * lv * d, lv * d)
    lw.gdn_qkvz = _rows(lw.gdn_qkvz, torch.cat([q_i, k_i, v_i, z_i]))
    conv_i = torch.cat([q_i, k_i, v_i]).to(lw.gdn_conv.device)
    lw.gdn_conv = lw.gdn_conv.index_select(0, conv_i).contiguous()
    heads = torch.arange(r * lv, (r + 1) * lv, device=lw.gdn_ab.device)
    lw.gdn_ab = lw.gdn_ab.index_select(0, torch.cat([heads, hv + heads])).contiguous()
    lw.gdn_a_log = lw.gdn_a_log[r * lv:(r + 1) * lv].contiguous()
    lw.gdn_dt_bias = lw.gdn_dt_bias[r * lv:(r + 1) * lv].contiguous()
    lw.gdn_out = _cols(lw.gdn_out, r * lv * d, (r + 1) * lv * d)


def _slice_bank(bank: ExpertBank, lo: int, hi: int) -> ExpertBank:
    dense = None if bank.dense is None else bank.dense[lo:hi]
    return ExpertBank(bank.fmt, hi - lo, bank.n, bank.k, bank.codes[lo:hi].contiguous(),
                      bank.scale[lo:hi].contiguous(), bank.signs, dense, base=lo)


def _shard_moe(cfg: ModelConfig, lw: LayerWeights, layer: int, lay: TPLayout, dev) -> None:
    """Expert parallelism: a contiguous range of experts per rank; tokens and the router stay
    replicated for decode-sized packets, so every rank computes its own experts' share of each
    token and the partial sums meet in the all-reduce that follows (the reference's TP8 plans
    do the same: python/orinfer_build/models/deepseek_v41/build.py:1199-1226,1355-1364);
    prefill-sized packets shard the tokens and exchange rows with all-to-alls."""
    w, r = lay.world, lay.rank
    lo, hi = split_blocks(cfg.experts, w)[r]
    lw.expert_gate_up = _slice_bank(lw.expert_gate_up, lo, hi)
    lw.expert_down = _slice_bank(lw.expert_down, lo, hi)
    # The shared expert stays whole on every rank (it is small): with sharded tokens each rank
    # applies it to the rows it owns; with replicated tokens only its owner rank adds it.
    lw.shared_owner = layer % w


def _draft_ffn_slice(width: int, lay: TPLayout) -> Tuple[int, int]:
    """This rank's channels of the draft layer's FFN (its width is the model's FFN width for
    dense models and a width of its own for expert models)."""
    if width % 128 or width // 128 < lay.world:
        raise ValueError(f"a draft FFN of {width} channels does not split over {lay.world} ranks")
    lo, hi = split_blocks(width // 128, lay.world)[lay.rank]
    return lo * 128, hi * 128


def _shard_draft_head(cfg: ModelConfig, mtp, lay: TPLayout, dev):
    """The draft head's decoder layer is sharded like any full-attention layer (heads, FFN
    channels); its input projection and norms are small and stay whole on every rank; the
    vocabulary head it shares with the model is sharded already."""
    from ..models.weights import MtpWeights
    lw = dataclasses.replace(mtp.layer)
    _shard_attention(cfg, lw, lay, dev)
    if lw.router is not None:
        _shard_moe(cfg, lw, 0, lay, dev)
    else:
        _shard_ffn(lw, dataclasses.replace(lay, ffn=_draft_ffn_slice(lw.gate_up.n // 2, lay)),
                   dev)
    return MtpWeights(mtp.norm_e, mtp.norm_h, mtp.fc, lw, mtp.final_norm)


def shard_model(weights: ModelWeights, rank: int, world: int,
                draft_head: bool = False) -> ModelWeights:
    """Returns this rank's shard; ``weights.config`` becomes the *local* geometry
    (local head counts, local FFN width) while ``vocab`` and the expert count stay global.
    ``draft_head``: keep (and shard) the model's draft head; without it the shard has none."""
    cfg = weights.config
    lay = layout(cfg, rank, world)
    dev = weights.embed_q.device
    layers = []
    for i, lw in enumerate(weights.layers):
        lw = dataclasses.replace(lw)
        if lw.kind == "attn":
            _shard_attention(cfg, lw, lay, dev)
        else:
            _shard_gdn(cfg, lw, lay, dev)
        if cfg.experts:
            _shard_moe(cfg, lw, i, lay, dev)
        else:
            _shard_ffn(lw, lay, dev)
        layers.append(lw)
    v0, v1 = lay.vocab
    head = _rows(weights.head, torch.arange(v0, v1, device=dev))
    local = dataclasses.replace(cfg, q_heads=lay.q_heads, kv_heads=lay.kv_heads,
                                ffn=(lay.ffn[1] - lay.ffn[0]) if cfg.ffn else cfg.ffn,
                                gdn_k_heads=cfg.gdn_k_heads // world if cfg.gdn_k_heads else 0,
                                gdn_v_heads=cfg.gdn_v_heads // world if cfg.gdn_v_heads else 0,
                                mtp_layers=0)
    mtp = None
    if draft_head and weights.mtp is not None:
        mtp = _shard_draft_head(cfg, weights.mtp, lay, dev)
        local = dataclasses.replace(local, mtp_layers=cfg.mtp_layers)
    out = ModelWeights(local, weights.embed_q, weights.embed_s, layers, weights.final_norm, head,
                       weights.signs, mtp, weights.embed_dense)
    out.tp = lay                       # type: ignore[attr-defined]
    out.global_config = cfg            # type: ignore[attr-defined]
    return out


def local_config(cfg: ModelConfig, lay: TPLayout) -> ModelConfig:
    """The geometry one rank computes: its heads, its FFN slice; vocabulary and expert
    count stay global."""
    world = lay.world
    return dataclasses.replace(
        cfg, q_heads=lay.q_heads, kv_heads=lay.kv_heads,
        ffn=(lay.ffn[1] - lay.ffn[0]) if cfg.ffn else cfg.ffn,
        gdn_k_heads=cfg.gdn_k_heads // world if cfg.gdn_k_heads else 0,
        gdn_v_heads=cfg.gdn_v_heads // world if cfg.gdn_v_heads else 0, mtp_layers=0)


def random_shard(cfg: ModelConfig, rank: int, world: int, device, seed: int = 0,
                 draft_head: bool = False) -> ModelWeights:
    """Random-init N(0, 0.02) weights of ONE rank's shard, quantised to the configured
    formats, created directly in the sharded geometry: no rank ever holds the whole model
    (``shard_model(random_model(...))`` would need all of an 80B-class model on every GPU).

    Tensors that tensor parallelism replicates (embedding, norms, router, shared expert) come
    from a generator seeded alike on every rank, so all ranks route and embed identically;
    sharded tensors come from a rank-specific generator.  The result has the same fields as
    ``shard_model`` gives (``tp`` layout, ``global_config``).  ``draft_head``: also create this
    rank's shard of the draft head when the geometry has one."""
    from ..models.weights import MtpWeights, _Init, _mtp_layer, quantize_linear
    lay = layout(cfg, rank, world)
    local = local_config(cfg, lay)
    dev = torch.device(device)
    own = _Init(local, seed + 7919 * (rank + 1), dev, False)
    shared = _Init(local, seed, dev, False)
    own.signs = shared.signs                         # one sign vector per width, rank-independent
    lo, hi = split_blocks(cfg.experts, world)[rank] if cfg.experts else (0, 0)

    def make_layer(i: int, full_attention: bool) -> LayerWeights:
        dense_cfg = dataclasses.replace(local, experts=0, ffn=local.ffn or 128)
        own.cfg = dense_cfg if cfg.experts else local
        lw = own.layer(i, full_attention)
        own.cfg = local
        if cfg.experts:
            lw.gate_up = lw.down = None
            rows = cfg.experts + (1 if cfg.shared_expert_ffn else 0)
            lw.router = shared.normal(rows, cfg.hidden).to(torch.float16)
            lw.expert_gate_up = own.bank(hi - lo, 2 * cfg.expert_ffn, cfg.hidden, cfg.expert_format)
            lw.expert_down = own.bank(hi - lo, cfg.hidden, cfg.expert_ffn, cfg.expert_format)
            lw.expert_gate_up.base = lw.expert_down.base = lo
            if cfg.shared_expert_ffn:
                lw.shared_gate_up = shared.linear(2 * cfg.shared_expert_ffn, cfg.hidden,
                                                  cfg.proj_format)
                lw.shared_down = shared.linear(cfg.hidden, cfg.shared_expert_ffn, cfg.proj_format)
            lw.shared_owner = i % world
        return lw

    layers: List[LayerWeights] = [make_layer(i, cfg.is_full_attention(i))
                                  for i in range(cfg.layers)]
    emb = quantize_linear(shared.normal(cfg.vocab, cfg.hidden), "w8", None)
    v0, v1 = lay.vocab
    if cfg.tied_embeddings:
        head = QLinear("w8", v1 - v0, cfg.hidden, emb.codes[v0:v1].contiguous(),
                       emb.scale[v0:v1].contiguous(), None)
    else:
        head = own.linear(v1 - v0, cfg.hidden, cfg.head_format, rotate=False)
    mtp = None
    if draft_head and cfg.mtp_layers:
        if cfg.draft_layer == "model":
            draft = make_layer(cfg.layers, True)
        else:
            full_f = cfg.ffn or max(cfg.expert_ffn * 4, 512)
            f0, f1 = _draft_ffn_slice(full_f, lay)
            own.cfg = dataclasses.replace(local, experts=0, ffn=f1 - f0)
            draft = _mtp_layer(own)
            own.cfg = local
        mtp = MtpWeights(shared.ones(cfg.hidden), shared.ones(cfg.hidden),
                         shared.linear(cfg.hidden, 2 * cfg.hidden, "w8", rotate=False),
                         draft, shared.ones(cfg.hidden))
        local = dataclasses.replace(local, mtp_layers=cfg.mtp_layers)
    out = ModelWeights(local, emb.codes, emb.scale, layers, shared.ones(cfg.hidden), head,
                       shared.signs, mtp, None)
    out.tp = lay                       # type: ignore[attr-defined]
    out.global_config = cfg            # type: ignore[attr-defined]
    return out
