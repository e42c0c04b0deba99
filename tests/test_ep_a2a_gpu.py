"""Expert-parallel dispatch / combine all-to-alls over peer memory against the single-rank
MoE arithmetic.  world_size 1 runs the whole protocol with the rank as its own peer."""
import os
import sys
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from orinfer_b200.models.weights import ExpertBank
    from orinfer_b200.ops import functional as F
    from orinfer_b200.ops import native
    from orinfer_b200.parallel.ep_a2a import ExpertA2A
    native.init()
    experts, top_k, hidden, ffn, rows = 8, 2, 256, 256, 150
    g = torch.Generator().manual_seed(5)                      # same weights on every rank
    codes = lambda e, n, k: torch.randint(-2 ** 31, 2 ** 31 - 1, (e, k // 128, n, 16),
                                          generator=g, dtype=torch.int32).to(dev)
    scales = lambda e, n: (torch.rand(e, n, generator=g) * 0.01 + 1e-3).half().to(dev)
    signs = (torch.randint(0, 2, (ffn,), generator=g, dtype=torch.int8) * 2 - 1).to(dev)
    up = ExpertBank("q4", experts, 2 * ffn, hidden, codes(experts, 2 * ffn, hidden),
                    scales(experts, 2 * ffn), None)
    dn = ExpertBank("q4", experts, hidden, ffn, codes(experts, hidden, ffn),
                    scales(experts, hidden), signs)
    gr = torch.Generator().manual_seed(100 + rank)            # this rank's own tokens
    q8 = torch.randint(-127, 128, (rows, hidden), generator=gr, dtype=torch.int8).to(dev)
    sa = (torch.rand(rows, generator=gr) * 0.05 + 1e-3).to(dev)
    ids = torch.stack([torch.randperm(experts, generator=gr)[:top_k] for _ in range(rows)]) \
        .to(torch.int32).to(dev)
    if rank == 0:
        ids[:60] = torch.tensor([7, 3], dtype=torch.int32)    # skew: many rows to one expert
    probs = torch.rand(rows, top_k, generator=gr).to(dev)
    # single-rank arithmetic over this rank's tokens with every expert local
    sc = F.MoeScratch(rows, top_k, experts, hidden, ffn, dev)
    F.moe_dispatch(ids, q8, sa, experts, sc, rows)
    F.qgemm_grouped(sc.q8, sc.scale, up.codes, up.scale, "q4", 2 * ffn, sc.gate_up, sc,
                    rows * top_k)
    F.act_prep(sc.gate_up, None, None, signs, swiglu=True, rows=rows * top_k, q_out=sc.q8_mid,
               scale_out=sc.scale_mid)
    F.qgemm_grouped(sc.q8_mid, sc.scale_mid, dn.codes, dn.scale, "q4", hidden, sc.down, sc,
                    rows * top_k)
    want = torch.zeros(rows, hidden, dtype=torch.float16, device=dev)
    F.moe_combine(sc.down, sc.slots, probs, None, None, want, rows)
    # expert parallel: this rank keeps experts [lo, hi)
    per = experts // world
    lo, hi = rank * per, (rank + 1) * per
    a2a = ExpertA2A(ExpertBank("q4", per, 2 * ffn, hidden, up.codes[lo:hi].contiguous(),
                               up.scale[lo:hi].contiguous(), None, base=lo),
                    ExpertBank("q4", per, hidden, ffn, dn.codes[lo:hi].contiguous(),
                               dn.scale[lo:hi].contiguous(), signs, base=lo),
                    experts, top_k, max_rows=rows)
    got = torch.zeros(rows, hidden, dtype=torch.float16, device=dev)
    for _ in range(3):                                        # buffers and counters are reused
        got.zero_()
        a2a.forward(q8, sa, ids, probs, got)
    torch.cuda.synchronize()
    ok = bool(torch.equal(got, want)) and native.read_status() == 0
    torch.save({"ok": ok, "diff": float((got.float() - want.float()).abs().max())},
               os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


def _check(tmp_path, world):
    port = 29800 + os.getpid() % 1000 + world
    ctx = mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=False)
    deadline = time.time() + 180
    while not ctx.join(timeout=5):
        if time.time() > deadline:
            for proc in ctx.processes:
                if proc.is_alive():
                    proc.kill()
            pytest.fail("expert-parallel ranks did not finish within 180 s")
    for r in range(world):
        res = torch.load(tmp_path / f"r{r}.pt")
        assert res["ok"], res


def test_expert_all_to_all_world1(cuda, tmp_path):
    _check(tmp_path, 1)


def test_expert_all_to_all_world2(cuda, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _check(tmp_path, 2)
