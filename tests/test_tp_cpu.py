"""Tensor-parallel sharding on CPU ranks (gloo, world_size 2): the sharded model must
reproduce the unsharded quantised forward up to the per-shard activation scales."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir, preset):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from orinfer_b200.config import PRESETS
    from orinfer_b200.models.runner import KVPool, Packet
    from orinfer_b200.models.weights import random_model
    from orinfer_b200.parallel.tp import shard_model
    from orinfer_b200.parallel.tp_runner import TPTorchRunner
    cfg = PRESETS[preset]
    full = random_model(cfg, seed=0)
    shard = shard_model(full, rank, world)
    assert shard.config.q_heads == cfg.q_heads // world
    if cfg.experts:
        assert shard.layers[0].expert_gate_up.experts == cfg.experts // world
        assert shard.layers[0].expert_gate_up.base == rank * (cfg.experts // world)
    else:
        assert shard.config.ffn == cfg.ffn // world
    runner = TPTorchRunner(shard, KVPool.allocate(shard.config, 4, "cpu"), 64)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab, (24,), generator=g, dtype=torch.int32)
    t = lambda v: torch.tensor(v, dtype=torch.int32)
    p = Packet(ids, t([0] * 24), t(list(range(24))), t([[1]]), 24, 24, torch.tensor([23]))
    tok, logits = runner.greedy(p)
    torch.save({"tok": tok, "logits": logits}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.destroy_process_group()


@pytest.mark.parametrize("preset", ["tiny", "tiny-moe", "tiny-hybrid"])
def test_tp2_matches_unsharded(tmp_path, preset):
    """Dense: Megatron sharding.  MoE: experts split over the ranks (expert parallelism with
    replicated tokens).  Hybrid: linear-attention heads split over the ranks."""
    from orinfer_b200.config import PRESETS
    from orinfer_b200.models.weights import random_model
    from orinfer_b200.ref import cpu_forward as ref
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path), preset), nprocs=2, join=True)
    r0 = torch.load(tmp_path / "r0.pt")
    r1 = torch.load(tmp_path / "r1.pt")
    assert torch.equal(r0["logits"], r1["logits"]) and torch.equal(r0["tok"], r1["tok"])
    cfg = PRESETS[preset]
    full = random_model(cfg, seed=0)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab, (24,), generator=g, dtype=torch.int32)
    want = ref.forward_request(full, ids, 0, ref.RefKV(cfg.layers), True)[-1]
    got = r0["logits"][0]
    assert got.shape == want.shape
    cos = torch.nn.functional.cosine_similarity(got, want, dim=0)
    assert cos > 0.995, cos
    assert int(r0["tok"][0]) == int(got.argmax())


def test_merge_sharded_argmax_rules():
    from orinfer_b200.parallel.tp_runner import merge_sharded_argmax
    vals = torch.tensor([[1.0, 5.0, 2.0], [3.0, 5.0, 2.0]])
    toks = torch.tensor([[4, 900, 7], [600, 20, -1]], dtype=torch.int32)
    assert merge_sharded_argmax(vals, toks).tolist() == [600, 20, -1]


def test_split_blocks_uneven():
    from orinfer_b200.parallel.tp import split_blocks
    parts = split_blocks(76, 8)
    assert parts[0] == (0, 10) and parts[-1] == (67, 76)
    assert sum(b - a for a, b in parts) == 76
