"""Hybrid (gated-delta-rule + attention) model through the engine on the CPU runner."""
import torch

from orinfer_b200.config import PRESETS, SchedulerOptions
from orinfer_b200.engine.engine import Engine
from orinfer_b200.models.weights import random_model
from orinfer_b200.ref import cpu_forward as ref
from orinfer_b200.ref import gdn_ref as G


def test_recurrence_matches_closed_form_single_step():
    torch.manual_seed(0)
    hk, hv, d = 1, 2, 8
    q, k = torch.randn(1, hk, d), torch.randn(1, hk, d)
    v, g, beta = torch.randn(1, hv, d), -torch.rand(1, hv), torch.rand(1, hv)
    s0 = torch.randn(hv, d, d)
    o, s1 = G.recurrence(q, k, v, g, beta, s0)
    for h in range(hv):
        sd = s0[h] * torch.exp(g[0, h])
        want = sd + torch.outer(k[0, 0], beta[0, h] * (v[0, h] - sd.t() @ k[0, 0]))
        assert torch.allclose(s1[h], want, atol=1e-5)
        assert torch.allclose(o[0, h], want.t() @ (q[0, 0] * d ** -0.5), atol=1e-5)


def test_conv_history_makes_chunking_exact():
    torch.manual_seed(1)
    c = 3 * 16
    x = torch.randn(10, c).half().float()
    w = torch.randn(c, 4).half().float()
    full, hist_full = G.conv_silu_l2(x, torch.zeros(3, c), w, 16, 16)
    a, h = G.conv_silu_l2(x[:4], torch.zeros(3, c), w, 16, 16)
    b, h = G.conv_silu_l2(x[4:], h, w, 16, 16)
    assert torch.equal(torch.cat([a, b]), full) and torch.equal(h, hist_full)


def test_hybrid_engine_matches_single_request_reference():
    cfg = PRESETS["tiny-hybrid"]
    w = random_model(cfg, seed=0)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (21, 9)]
    eng = Engine(w, sched=SchedulerOptions(max_active=4, prefill_chunk=8), kv_pages=12,
                 max_context=256)
    assert eng.prefix is None and not eng.spec.enabled      # recurrent state: no reuse, no drafts
    r0 = eng.submit(prompts[0], 5)
    eng.step()
    r1 = eng.submit(prompts[1], 5)                           # joins while r0 is mid-prefill
    while eng.has_work():
        eng.step()
    for r, p in zip((r0, r1), prompts):
        want, _ = ref.generate_greedy(w, torch.tensor(p), 5, quantized=True)
        assert r.generated == want
    # a slot reused by a later request starts from a zero state
    r2 = eng.submit(prompts[1], 5)
    while eng.has_work():
        eng.step()
    assert r2.generated == r1.generated
