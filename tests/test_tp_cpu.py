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


def test_sharded_sampling_equals_the_host_law_on_the_full_row():
    """World 1 (no process group): merged candidates + host law = host law on all logits,
    ties at the top-k boundary included."""
    from orinfer_b200.core import sampling as S
    from orinfer_b200.parallel import sharded_sampling as SS
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(6, 640, generator=g)
    logits[0, [5, 300, 17]] = 4.0                      # ties inside and at the boundary
    logits[1, 100:140] = 2.5
    opts = [S.SamplingOptions(temperature=0.7, top_k=2, seed=1),
            S.SamplingOptions(temperature=1.3, top_k=16, top_p=0.8, seed=2),
            S.SamplingOptions(temperature=1.0, top_k=64, seed=3),
            S.SamplingOptions(temperature=0.2, top_k=1, seed=4),
            S.SamplingOptions(temperature=2.0, top_k=40, top_p=0.5, seed=5),
            S.SamplingOptions(temperature=1.0, top_k=8, seed=6)]
    for step in range(40):
        us = [S.counter_uniform(o.seed, 0, step) for o in opts]
        got = SS.sample_rows(logits, 0, opts, us)
        want = [S.sample(logits[i].numpy(), [], o, u) for i, (o, u) in enumerate(zip(opts, us))]
        assert got == want, step
    # two shards merged by hand: same answer as one shard
    a, b = logits[:, :384], logits[:, 384:]
    va, ia = SS.local_candidates(a, 64, 0)
    vb, ib = SS.local_candidates(b, 64, 384)
    v, i = SS.merge_candidates(torch.cat([va, vb], 1), torch.cat([ia, ib], 1), 64)
    v1, i1 = SS.merge_candidates(*SS.local_candidates(logits, 64, 0), 64)
    assert torch.equal(v, v1) and torch.equal(i, i1)


def _sampling_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from orinfer_b200.config import PRESETS, LoadOptions, SchedulerOptions
    from orinfer_b200.core.sampling import SamplingOptions
    from orinfer_b200.engine.engine import Engine
    from orinfer_b200.models.runner import KVPool
    from orinfer_b200.models.weights import random_model
    from orinfer_b200.parallel.tp import shard_model
    from orinfer_b200.parallel.tp_runner import TPTorchRunner
    cfg = PRESETS["tiny"]
    shard = shard_model(random_model(cfg, seed=0), rank, world)
    eng = Engine(shard, kv_pages=12, max_context=256,
                 load=LoadOptions(prefix_cache_bytes=0),
                 sched=SchedulerOptions(max_active=4, prefill_chunk=64))
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (20, 9, 14)]
    opts = [SamplingOptions(temperature=0.9, top_k=8, seed=11), None,
            SamplingOptions(temperature=1.2, top_k=32, top_p=0.9, seed=12)]
    assert isinstance(eng.runner, TPTorchRunner)
    reqs = [eng.submit(p, 10, sampling=o) for p, o in zip(prompts, opts)]
    while eng.has_work():
        eng.step()
    torch.save({"out": [r.generated for r in reqs], "sharded": eng.stats.sharded_samples},
               os.path.join(out_dir, f"s{rank}.pt"))
    dist.destroy_process_group()


def test_tp2_engine_samples_from_sharded_candidates(tmp_path):
    """Sampled requests on two ranks: both ranks commit the same tokens, drawn without
    gathering the logits; a greedy request in the same batch is unaffected."""
    port = 31500 + os.getpid() % 2000
    mp.spawn(_sampling_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = torch.load(tmp_path / "s0.pt"), torch.load(tmp_path / "s1.pt")
    assert r0["out"] == r1["out"]
    assert all(len(o) == 10 for o in r0["out"])
    assert r0["sharded"] == 20                       # two sampled requests x 10 tokens


def _draft_cfg(preset):
    import dataclasses
    from orinfer_b200.config import PRESETS
    return dataclasses.replace(PRESETS[preset], mtp_layers=1,
                               draft_layer="dense" if preset == "tiny" else "model")


def _draft_worker(rank, world, port, out_dir, preset):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    from orinfer_b200.models.runner import KVPool, Packet
    from orinfer_b200.models.weights import random_model
    from orinfer_b200.parallel.tp import shard_model
    from orinfer_b200.parallel.tp_runner import TPTorchRunner
    cfg = _draft_cfg(preset)
    shard = shard_model(random_model(cfg, seed=0), rank, world, draft_head=True)
    assert shard.config.mtp_layers == 1
    if cfg.experts:
        assert shard.mtp.layer.expert_down.experts == cfg.experts // world
    else:
        assert shard.mtp.layer.gate_up.n == cfg.ffn * 2 // world
    assert shard.mtp.layer.o.k == cfg.q_heads * cfg.head_dim // world
    runner = TPTorchRunner(shard, KVPool.allocate(shard.config, 4, "cpu", 1), 64)
    ids, p = _draft_inputs(cfg, Packet)
    runner.greedy(p)
    tok, hid = runner.mtp_rows(torch.roll(ids, -1), runner.final_hidden(p.rows), p)
    torch.save({"tok": tok, "hid": hid}, os.path.join(out_dir, f"d{rank}.pt"))
    dist.destroy_process_group()


def _draft_inputs(cfg, Packet):
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, cfg.vocab, (16,), generator=g, dtype=torch.int32)
    t = lambda v: torch.tensor(v, dtype=torch.int32)
    return ids, Packet(ids, t([0] * 16), t(list(range(16))), t([[1]]), 16, 16)


@pytest.mark.parametrize("preset", ["tiny", "tiny-moe"])
def test_sharded_draft_head_matches_the_whole_one(tmp_path, preset):
    """The draft head split over two ranks (heads, FFN channels or experts, vocabulary) gives
    the hidden rows and draft tokens of the unsplit head, up to the per-shard activation
    scales."""
    from orinfer_b200.models.runner import KVPool, Packet
    from orinfer_b200.models.torch_runner import TorchRunner
    from orinfer_b200.models.weights import random_model
    port = 31500 + os.getpid() % 2000
    mp.spawn(_draft_worker, args=(2, port, str(tmp_path), preset), nprocs=2, join=True)
    r0, r1 = torch.load(tmp_path / "d0.pt"), torch.load(tmp_path / "d1.pt")
    assert torch.equal(r0["tok"], r1["tok"]) and torch.equal(r0["hid"], r1["hid"])
    cfg = _draft_cfg(preset)
    full = random_model(cfg, seed=0)
    runner = TorchRunner(full, KVPool.allocate(cfg, 4, "cpu", 1), 64)
    ids, p = _draft_inputs(cfg, Packet)
    runner.greedy(p)
    tok, hid = runner.mtp_rows(torch.roll(ids, -1), runner.final_hidden(p.rows), p)
    cos = torch.nn.functional.cosine_similarity(r0["hid"].float(), hid.float(), dim=1)
    assert cos.min() > 0.995, cos
    assert (r0["tok"].long() == tok.long()).float().mean() >= 0.75


def test_random_shards_carry_a_draft_head_only_when_asked():
    from orinfer_b200.parallel.tp import random_shard
    for preset in ("tiny", "tiny-moe"):
        cfg = _draft_cfg(preset)
        assert random_shard(cfg, 0, 2, "cpu").mtp is None
        shards = [random_shard(cfg, r, 2, "cpu", draft_head=True) for r in range(2)]
        for r, s in enumerate(shards):
            assert s.config.mtp_layers == 1 and s.mtp.fc.k == 2 * cfg.hidden
            assert s.mtp.layer.o.k == cfg.q_heads * cfg.head_dim // 2
            if cfg.experts:
                assert s.mtp.layer.expert_down.base == r * cfg.experts // 2
                assert torch.equal(s.mtp.layer.router, shards[0].mtp.layer.router)
            else:
                assert s.mtp.layer.gate_up.n == cfg.ffn
        assert torch.equal(shards[0].mtp.fc.codes, shards[1].mtp.fc.codes)     # replicated
