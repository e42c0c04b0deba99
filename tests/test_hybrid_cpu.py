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
    assert eng.prefix is not None                            # endpoints carry recurrent snapshots
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


def test_tentative_pass_then_commit_equals_plain_prefix():
    """A verification packet leaves the recurrent state alone; committing a rows of it gives
    what a plain pass over those a rows gives."""
    from orinfer_b200.models.runner import Packet
    from orinfer_b200.models.torch_runner import TorchRunner
    cfg = PRESETS["tiny-hybrid"]
    w = random_model(cfg, seed=3)
    t = lambda v: torch.tensor(v, dtype=torch.int32)

    def prefilled():
        from orinfer_b200.models.runner import KVPool
        r = TorchRunner(w, KVPool.allocate(cfg, 4, torch.device("cpu")), max_rows=64)
        n = 6
        r.logits(Packet(t(list(range(3, 3 + n))), t([0] * n), t(list(range(n))), t([[1, 2]]), n, n))
        return r

    toks = [11, 12, 13, 14]
    a, b = prefilled(), prefilled()
    p = Packet(t(toks), t([0] * 4), t([6, 7, 8, 9]), t([[1, 2]]), 4, 10)
    p.tentative = True
    a.logits(p)
    a.gdn_commit(p, [2])
    b.logits(Packet(t(toks[:2]), t([0] * 2), t([6, 7]), t([[1, 2]]), 2, 8))
    nxt = Packet(t([20]), t([0]), t([8]), t([[1, 2]]), 1, 9)
    assert torch.allclose(a.logits(nxt), b.logits(nxt), atol=1e-5)


def test_hybrid_engine_speculates_and_matches_plain_greedy(monkeypatch):
    """Right, wrong and half-right drafts: the recurrent state keeps exactly the accepted rows."""
    from orinfer_b200.config import LoadOptions
    monkeypatch.setenv("ORINFER_SINGLE_MTP_POLICY", "fixed3")
    cfg = PRESETS["tiny-hybrid"]
    w = random_model(cfg, seed=0)
    prompts = [[5, 6, 7, 8, 9, 5, 6, 7, 8, 9, 5, 6, 7], [3, 1, 4, 1, 5, 9, 2, 6]]
    want = [ref.generate_greedy(w, torch.tensor(p), 12, quantized=True)[0] for p in prompts]
    for kind in ("oracle", "wrong", "half"):
        eng = Engine(w, load=LoadOptions(prompt_lookup=True, mtp_drafts=3),
                     sched=SchedulerOptions(max_active=2, prefill_chunk=8), kv_pages=12,
                     max_context=256)
        assert eng.spec.enabled
        reqs = [eng.submit(p, 12) for p in prompts]
        text = {r.rid: t for r, t in zip(reqs, want)}

        def drafts(r, c, kind=kind, text=text):
            d = list(text[r.rid][len(r.generated):len(r.generated) + c])
            if kind == "wrong":
                d = [(t + 1) % cfg.vocab for t in d]
            elif kind == "half" and len(d) > 1:
                d[1:] = [(t + 1) % cfg.vocab for t in d[1:]]
            return d

        eng.spec.drafts_for = drafts
        while eng.has_work():
            eng.step()
        assert [r.generated for r in reqs] == want, kind
        st = eng.spec.statistics()
        assert st["proposed_tokens"] > 0
        if kind == "oracle":
            assert st["acceptance_rate"] == 1.0
        if kind == "half":
            assert 0 < st["accepted_draft_tokens"] < st["proposed_tokens"]


def test_hybrid_prefix_reuse_restores_recurrent_state():
    """A second request with the same prompt (or one that extends it) starts from the cached KV
    pages and the snapshotted recurrent state, and produces the text of a cold run."""
    from orinfer_b200.config import LoadOptions
    from orinfer_b200.config import PAGE_TOKENS
    cfg = PRESETS["tiny-hybrid"]
    w = random_model(cfg, seed=0)
    g = torch.Generator().manual_seed(5)
    n = 2 * PAGE_TOKENS + 9
    prompt = torch.randint(0, cfg.vocab, (n,), generator=g).tolist()
    longer = prompt[:2 * PAGE_TOKENS] + torch.randint(0, cfg.vocab, (20,), generator=g).tolist()
    mk = lambda cache: Engine(w, load=LoadOptions(prefix_cache_bytes=cache),
                              sched=SchedulerOptions(max_active=2, prefill_chunk=96),
                              kv_pages=24, max_context=512)
    cold = mk(0)
    want = [cold.generate([p], max_new=6)[0] for p in (prompt, longer)]
    eng = mk(64 << 20)
    assert eng.prefix is not None
    assert eng.generate([prompt], max_new=6)[0] == want[0]
    assert eng.stats.stored_snapshots == 1 and eng.stats.restored_snapshots == 0
    r = eng.submit(prompt, 6)
    while eng.has_work():
        eng.step()
    assert r.generated == want[0] and r.cached_tokens == 2 * PAGE_TOKENS
    r2 = eng.submit(longer, 6)                    # shares the first two pages only
    while eng.has_work():
        eng.step()
    assert r2.generated == want[1] and r2.cached_tokens == 2 * PAGE_TOKENS
    assert eng.stats.restored_snapshots == 2
    # a prompt that diverges inside the snapshotted span cannot use the endpoint
    other = prompt[:PAGE_TOKENS + 3] + [(t + 1) % cfg.vocab for t in prompt[PAGE_TOKENS + 3:]]
    r3 = eng.submit(other, 4)
    while eng.has_work():
        eng.step()
    assert r3.cached_tokens == 0
    assert r3.generated == cold.generate([other], max_new=4)[0]


def test_chunked_gdn_recurrence_equals_the_sequential_one():
    """The WY (chunkwise) form and the token-by-token scan are the same function, for any
    chunk size, ragged last chunks, grouped heads and a non-zero starting state."""
    import torch
    from orinfer_b200.ref import gdn_ref as G
    gen = torch.Generator().manual_seed(5)
    t, hk, hv, d = 45, 2, 4, 16
    q = torch.nn.functional.normalize(torch.randn(t, hk, d, generator=gen), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(t, hk, d, generator=gen), dim=-1)
    v = torch.randn(t, hv, d, generator=gen)
    g = -torch.rand(t, hv, generator=gen) * 0.5
    beta = torch.rand(t, hv, generator=gen)
    s0 = torch.randn(hv, d, d, generator=gen) * 0.3
    want_o, want_s = G.recurrence(q, k, v, g, beta, s0)
    for chunk in (1, 16, 64, 7):
        o, s = G.recurrence_chunked(q, k, v, g, beta, s0, chunk)
        assert torch.allclose(o, want_o, atol=2e-5, rtol=1e-5), chunk
        assert torch.allclose(s, want_s, atol=2e-5, rtol=1e-5), chunk
    # chunk boundaries may fall anywhere: two calls carry the state like one
    o1, s1 = G.recurrence_chunked(q[:20], k[:20], v[:20], g[:20], beta[:20], s0)
    o2, s2 = G.recurrence_chunked(q[20:], k[20:], v[20:], g[20:], beta[20:], s1)
    assert torch.allclose(torch.cat([o1, o2]), want_o, atol=2e-5, rtol=1e-5)
    assert torch.allclose(s2, want_s, atol=2e-5, rtol=1e-5)
