"""Gated-delta-rule kernels and the hybrid model on the device against the PyTorch oracle."""
import pytest
import torch

from orinfer_b200.config import PRESETS
from orinfer_b200.models.weights import random_model
from orinfer_b200.ref import gdn_ref as G

pytestmark = pytest.mark.gpu


def _segments(lens, cuda):
    segs, first, start = [], [], 0
    for n in lens:
        segs.append([start, n, 0, 0])
        first += [start] * n
        start += n
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=cuda)
    return t(segs), t(first)


@pytest.mark.parametrize("d", [64, 128])
def test_conv_scan_norm_match_reference_across_chunks(cuda, d):
    from orinfer_b200.ops import functional as F
    torch.manual_seed(d)
    hk, hv = 2, 4
    dk, conv_dim = hk * d, (2 * hk + hv) * d
    lens, slots = [5, 1, 9], [2, 0, 3]
    rows = sum(lens)
    w = (torch.randn(conv_dim, 4) * 0.5).half()
    a_log, dt_bias = torch.randn(hv) * 0.3, torch.randn(hv) * 0.3
    norm_w = (1 + 0.1 * torch.randn(d)).half()
    hist = torch.zeros(4, 3, conv_dim, dtype=torch.float16, device=cuda)
    state = torch.zeros(4, hv, d, d, device=cuda)
    ref_state = {s: (torch.zeros(hv, d, d), torch.zeros(3, conv_dim)) for s in slots}
    segs, first = _segments(lens, cuda)
    row_slot = torch.tensor([s for s, n in zip(slots, lens) for _ in range(n)], dtype=torch.int32,
                            device=cuda)
    pos0 = [0, 0, 0]
    for step in range(3):                     # the second and third pass continue the state
        x = torch.randn(rows, conv_dim + hv * d).half()
        ab = torch.randn(rows, 2 * hv)
        row_pos = torch.tensor([p + i for p, n in zip(pos0, lens) for i in range(n)],
                               dtype=torch.int32, device=cuda)
        yc = F.gdn_conv(x.to(cuda), w.to(cuda), hist, first, row_slot, row_pos, segs, len(lens),
                        rows, hk, hv, d)
        o = F.gdn_scan(yc, ab.to(cuda), a_log.to(cuda), dt_bias.to(cuda), segs, len(lens),
                       row_slot, row_pos, hk, hv, d, state)
        y = F.gdn_gated_norm(o, x.to(cuda)[:, conv_dim:], norm_w.to(cuda), 1e-6, rows, hv, d)
        torch.cuda.synchronize()
        start = 0
        for s, n in zip(slots, lens):
            sl = slice(start, start + n)
            st, hs = ref_state[s]
            yr, hs = G.conv_silu_l2(x[sl, :conv_dim].float(), hs, w, dk, d)
            g, beta = G.gates(ab[sl], a_log, dt_bias)
            orf, st = G.recurrence(yr[:, :dk].reshape(n, hk, d), yr[:, dk:2 * dk].reshape(n, hk, d),
                                   yr[:, 2 * dk:].reshape(n, hv, d), g, beta, st)
            ref_state[s] = (st, hs)
            want = G.gated_norm(orf, x[sl, conv_dim:].float().reshape(n, hv, d), norm_w, 1e-6)
            assert (yc[sl].cpu().float() - yr).abs().max() < 2e-3
            assert torch.equal(hist[s].cpu().float(), hs)
            assert (o[sl].cpu() - orf).abs().max() < 2e-3 * max(1.0, float(orf.abs().max()))
            assert (state[s].cpu() - st).abs().max() < 2e-3 * max(1.0, float(st.abs().max()))
            assert (y[sl].cpu().float() - want).abs().max() < 2e-2
            start += n
        pos0 = [p + n for p, n in zip(pos0, lens)]


def test_small_projection(cuda):
    from orinfer_b200.ops import functional as F
    torch.manual_seed(3)
    x, w = torch.randn(37, 512).half(), torch.randn(8, 512).half()
    got = F.small_proj(x.to(cuda), w.to(cuda)).cpu()
    assert torch.allclose(got, x.float() @ w.float().t(), atol=2e-3, rtol=1e-4)


def test_tiny_hybrid_matches_torch_runner_prefill_and_decode(cuda):
    from orinfer_b200.models.runner import KVPool, ModelRunner, Packet
    from orinfer_b200.models.torch_runner import TorchRunner
    cfg = PRESETS["tiny-hybrid"]
    w_cpu = random_model(cfg, seed=7)
    dev = ModelRunner(w_cpu.to(cuda), KVPool.allocate(cfg, 6, cuda), 256)
    cpu = TorchRunner(w_cpu, KVPool.allocate(cfg, 6, "cpu"), 256)
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (40, 13)]

    def packet(device, toks, starts):
        ids, req, pos, last = [], [], [], []
        for r, (tk, st) in enumerate(zip(toks, starts)):
            ids += tk
            req += [r] * len(tk)
            pos += list(range(st, st + len(tk)))
            last.append(len(ids) - 1)
        t = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
        return Packet(t(ids), t(req), t(pos), t([[1, 2], [3, 4]]), len(ids), max(pos) + 1,
                      torch.tensor(last, dtype=torch.int64, device=device))

    tok_d, lg_d = dev.greedy(packet(cuda, prompts, [0, 0]))
    tok_c, lg_c = cpu.greedy(packet("cpu", prompts, [0, 0]))
    for r in range(2):
        cos = torch.nn.functional.cosine_similarity(lg_d[r].cpu(), lg_c[r], dim=0)
        assert cos > 0.998, cos
    cur = tok_c.tolist()
    lens = [40, 13]
    for step in range(6):                      # teacher-forced decode continues the state
        toks = [[cur[0]], [cur[1]]]
        starts = [lens[0] + step, lens[1] + step]
        _, lg_d = dev.greedy(packet(cuda, toks, starts))
        tok_c, lg_c = cpu.greedy(packet("cpu", toks, starts))
        for r in range(2):
            cos = torch.nn.functional.cosine_similarity(lg_d[r].cpu(), lg_c[r], dim=0)
            assert cos > 0.998, (step, cos)
        cur = tok_c.tolist()


def test_hybrid_engine_graph_decode_matches_direct(cuda):
    from orinfer_b200.config import GraphMode, LoadOptions, SchedulerOptions
    from orinfer_b200.engine.engine import Engine
    cfg = PRESETS["tiny-hybrid"]
    w = random_model(cfg, seed=9).to(cuda)
    g = torch.Generator().manual_seed(10)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (30, 11, 19)]
    outs = []
    for mode in (GraphMode.OFF, GraphMode.DECODE_ONLY):
        eng = Engine(w, load=LoadOptions(cuda_graph=mode),
                     sched=SchedulerOptions(max_active=4, prefill_chunk=16), kv_pages=16,
                     max_context=256)
        outs.append(eng.generate(prompts, max_new=10))
    assert outs[0] == outs[1]


@pytest.mark.parametrize("d", [64, 128])
def test_tentative_scan_then_commit_is_bit_identical_to_plain_prefix(cuda, d):
    """A verification pass records (decay, k, delta) and leaves state and history alone; the
    commit of a[s] rows per segment gives the very bits a plain pass over those rows gives."""
    from orinfer_b200.ops import functional as F
    torch.manual_seed(100 + d)
    hk, hv = 2, 4
    conv_dim = (2 * hk + hv) * d
    lens, slots, keep = [4, 3, 5], [1, 3, 0], [2, 0, 5]
    rows = sum(lens)
    w = (torch.randn(conv_dim, 4) * 0.5).half().to(cuda)
    a_log, dt_bias = (torch.randn(hv) * 0.3).to(cuda), (torch.randn(hv) * 0.3).to(cuda)
    hist0 = torch.randn(4, 3, conv_dim, device=cuda).half()
    state0 = torch.randn(4, hv, d, d, device=cuda) * 0.1
    x = torch.randn(rows, conv_dim, device=cuda).half()
    ab = torch.randn(rows, 2 * hv, device=cuda)
    segs, first = _segments(lens, cuda)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=cuda)
    row_slot = t([s for s, n in zip(slots, lens) for _ in range(n)])
    row_pos = t([7 + i for n in lens for i in range(n)])

    hist, state = hist0.clone(), state0.clone()
    fac = torch.zeros(rows, hv, 2 * d + 1, device=cuda)
    yc = F.gdn_conv(x, w, hist, first, row_slot, row_pos, segs, len(lens), rows, hk, hv, d,
                    update_history=False)
    o_t = F.gdn_scan(yc, ab, a_log, dt_bias, segs, len(lens), row_slot, row_pos, hk, hv, d, state,
                     factors=fac)
    torch.cuda.synchronize()
    assert torch.equal(hist, hist0) and torch.equal(state, state0)
    F.gdn_commit(x, fac, segs, len(lens), t(keep), row_slot, row_pos, hk, hv, d, hist, state)

    # plain pass over the kept rows only
    kept = [i for st, (n, a) in zip([0, 4, 7], zip(lens, keep)) for i in range(st, st + a)]
    klens = [a for a in keep if a > 0]
    kslots = [s for s, a in zip(slots, keep) if a > 0]
    ksegs, kfirst = _segments(klens, cuda)
    idx = torch.tensor(kept, device=cuda)
    hist_p, state_p = hist0.clone(), state0.clone()
    kslot = t([s for s, n in zip(kslots, klens) for _ in range(n)])
    kpos = row_pos[idx].contiguous()
    xk = x[idx].contiguous()
    yk = F.gdn_conv(xk, w, hist_p, kfirst, kslot, kpos, ksegs, len(klens), len(kept), hk, hv, d)
    o_p = F.gdn_scan(yk, ab[idx].contiguous(), a_log, dt_bias, ksegs, len(klens), kslot, kpos,
                     hk, hv, d, state_p)
    torch.cuda.synchronize()
    assert torch.equal(o_t[idx], o_p)
    assert torch.equal(hist, hist_p)
    assert torch.equal(state, state_p)


def test_hybrid_engine_speculation_on_device_matches_plain(cuda, monkeypatch):
    from orinfer_b200.config import GraphMode, LoadOptions, SchedulerOptions
    from orinfer_b200.engine.engine import Engine
    monkeypatch.setenv("ORINFER_SINGLE_MTP_POLICY", "fixed3")
    cfg = PRESETS["tiny-hybrid"]
    w = random_model(cfg, seed=11).to(cuda)
    g = torch.Generator().manual_seed(12)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (25, 9)]
    mk = lambda **kw: Engine(w, load=LoadOptions(cuda_graph=GraphMode.OFF, **kw),
                             sched=SchedulerOptions(max_active=4, prefill_chunk=16),
                             kv_pages=16, max_context=256)
    plain = mk().generate(prompts, max_new=12)
    for kind in ("oracle", "half"):
        eng = mk(prompt_lookup=True, mtp_drafts=3)
        reqs = [eng.submit(p, 12) for p in prompts]
        text = {r.rid: t for r, t in zip(reqs, plain)}

        def drafts(r, c, kind=kind, text=text):
            dr = list(text[r.rid][len(r.generated):len(r.generated) + c])
            if kind == "half" and len(dr) > 1:
                dr[1:] = [(x + 1) % cfg.vocab for x in dr[1:]]
            return dr

        eng.spec.drafts_for = drafts
        while eng.has_work():
            eng.step()
        assert [r.generated for r in reqs] == plain, kind
        assert eng.spec.statistics()["accepted_draft_tokens"] > 0


def test_hybrid_prefix_reuse_restores_recurrent_state_on_device(cuda):
    from orinfer_b200.config import PAGE_TOKENS, LoadOptions, SchedulerOptions
    from orinfer_b200.engine.engine import Engine
    cfg = PRESETS["tiny-hybrid"]
    w = random_model(cfg, seed=13).to(cuda)
    g = torch.Generator().manual_seed(14)
    prompt = torch.randint(0, cfg.vocab, (2 * PAGE_TOKENS + 9,), generator=g).tolist()
    longer = prompt[:2 * PAGE_TOKENS] + torch.randint(0, cfg.vocab, (20,), generator=g).tolist()
    mk = lambda cache: Engine(w, load=LoadOptions(prefix_cache_bytes=cache),
                              sched=SchedulerOptions(max_active=2, prefill_chunk=96),
                              kv_pages=24, max_context=512)
    # cold runs with the same chunk boundaries as the warm ones (chunks end at the endpoints)
    want = [mk(64 << 20).generate([p], max_new=6)[0] for p in (prompt, longer)]
    eng = mk(64 << 20)
    assert eng.generate([prompt], max_new=6)[0] == want[0]
    assert eng.stats.stored_snapshots == 1
    for p, text in zip((prompt, longer), want):
        r = eng.submit(p, 6)
        while eng.has_work():
            eng.step()
        assert r.generated == text and r.cached_tokens == 2 * PAGE_TOKENS
    assert eng.stats.restored_snapshots == 2
