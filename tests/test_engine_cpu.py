"""Continuous engine on the CPU reference runner (tiny model)."""
import pytest
import torch

from orinfer_b200.config import PRESETS, LoadOptions, SchedulerOptions
from orinfer_b200.core.sampling import SamplingOptions
from orinfer_b200.engine.engine import Engine
from orinfer_b200.engine.request import Phase
from orinfer_b200.models.weights import random_model
from orinfer_b200.ref import cpu_forward as ref


@pytest.fixture(scope="module")
def weights():
    return random_model(PRESETS["tiny"], seed=0)


def _prompts(n, length, seed=1, vocab=1024):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def _engine(weights, **kw):
    sched = SchedulerOptions(max_active=kw.pop("max_active", 4),
                             prefill_chunk=kw.pop("prefill_chunk", 64))
    return Engine(weights, sched=sched, kv_pages=kw.pop("kv_pages", 24), max_context=512,
                  load=kw.pop("load", LoadOptions()), **kw)


def test_greedy_matches_single_request_reference(weights):
    prompts = _prompts(2, 32)
    eng = _engine(weights)
    out = eng.generate(prompts, max_new=8)
    for p, o in zip(prompts, out):
        want, _ = ref.generate_greedy(weights, torch.tensor(p), 8, quantized=True)
        assert o == want
    assert eng.stats.finished == 2 and eng.pool.available == 23 - eng.prefix.statistics().device_pages


def test_continuous_batching_is_batch_invariant(weights):
    prompts = _prompts(3, 20, seed=2)
    solo = [_engine(weights).generate([p], max_new=6)[0] for p in prompts]
    eng = _engine(weights, prefill_chunk=8)          # chunked prefill + staggered arrivals
    r0 = eng.submit(prompts[0], 6)
    eng.step(); eng.step()
    r1 = eng.submit(prompts[1], 6)
    eng.step()
    r2 = eng.submit(prompts[2], 6)
    while eng.has_work():
        eng.step()
    assert [r0.generated, r1.generated, r2.generated] == solo
    assert eng.stats.prefill_tokens == 60


def test_prefix_cache_reuses_pages_and_keeps_output(weights):
    base = _prompts(1, 140, seed=3)[0]
    eng = _engine(weights, prefill_chunk=256)
    first = eng.generate([base + [5, 6, 7]], max_new=4)[0]
    r = eng.submit(base + [5, 6, 7], 4)
    while not r.finished:
        eng.step()
    assert r.cached_tokens == 128 and r.generated == first
    other = eng.submit(base[:130] + [9, 9], 4)
    while not other.finished:
        eng.step()
    assert other.cached_tokens == 128
    st = eng.prefix.statistics()
    assert st.hit_tokens >= 256 and st.device_pages >= 1
    cold = _engine(weights, prefill_chunk=256, load=LoadOptions(prefix_cache_bytes=0))
    assert cold.generate([base[:130] + [9, 9]], max_new=4)[0] == other.generated


def test_admission_waits_for_pages_and_evicts_prefixes(weights):
    prompts = _prompts(4, 100, seed=4)
    eng = _engine(weights, kv_pages=4, max_active=4)       # 3 usable pages, 1 page per request
    reqs = [eng.submit(p, 8) for p in prompts]
    steps = 0
    while eng.has_work():
        eng.step()
        steps += 1
        assert steps < 200
    assert all(len(r.generated) == 8 for r in reqs)
    assert eng.stats.deferred_admissions > 0
    solo = _engine(weights).generate([prompts[3]], max_new=8)[0]
    assert reqs[3].generated == solo


def test_seeded_sampling_is_independent_of_batch(weights):
    prompts = _prompts(2, 16, seed=5)
    opt = SamplingOptions(temperature=0.9, top_p=0.95, seed=1234)
    alone = _engine(weights).generate([prompts[0]], max_new=6, sampling=opt)[0]
    both = _engine(weights).generate(prompts, max_new=6, sampling=opt)
    assert both[0] == alone
    again = _engine(weights).generate([prompts[0]], max_new=6, sampling=opt)[0]
    assert again == alone
    other_seed = _engine(weights).generate(
        [prompts[0]], max_new=6, sampling=SamplingOptions(temperature=0.9, top_p=0.95, seed=99))[0]
    assert other_seed != alone


def test_cancel_stop_and_logprobs(weights):
    prompts = _prompts(2, 12, seed=6)
    eng = _engine(weights)
    a = eng.submit(prompts[0], 50)
    b = eng.submit(prompts[1], 5, SamplingOptions(temperature=0.0, top_logprobs=3))
    eng.step(); eng.step()
    eng.cancel(a)
    while eng.has_work():
        eng.step()
    assert a.finish_reason == "cancelled" and a.phase is Phase.FINISHED
    assert b.finish_reason == "length" and len(b.logprobs) == 5
    tok, lp, top = b.logprobs[0]
    assert top[0][0] == tok and abs(top[0][1] - lp) < 1e-12 and lp <= 0
    first = b.generated[0]
    c = eng.submit(prompts[1], 5, stop_ids=(first,))
    while eng.has_work():
        eng.step()
    assert c.generated == [first] and c.finish_reason == "stop"
    assert eng.pool.available + eng.prefix.statistics().device_pages == 23


def test_context_limit_is_rejected(weights):
    eng = _engine(weights)
    with pytest.raises(ValueError, match="exceeds the context window"):
        eng.submit([1] * 500, 100)


def test_speculation_preserves_output(weights):
    """Verification rounds commit exactly the tokens plain decoding produces, whether the
    drafts are all right (oracle), all wrong, or come from prompt lookup; greedy and seeded
    sampling (exact rejection sampling with point-mass proposals)."""
    import os
    base = [5, 6, 7, 8, 9, 10, 11, 12] * 6
    for opt in (None, SamplingOptions(temperature=0.8, seed=3)):
        ref_eng = _engine(weights)
        plain = ref_eng.generate([base], max_new=24, sampling=opt)[0]
        os.environ["ORINFER_SINGLE_MTP_POLICY"] = "fixed3"
        try:
            for kind in ("oracle", "wrong", "lookup"):
                eng = _engine(weights, load=LoadOptions(prompt_lookup=True, mtp_drafts=3))
                if kind == "oracle":
                    eng.spec.drafts_for = lambda r, c: plain[len(r.generated):len(r.generated) + c]
                elif kind == "wrong":
                    eng.spec.drafts_for = lambda r, c: [(t + 1) % 1024 for t in
                                                        plain[len(r.generated):len(r.generated) + c]]
                out = eng.generate([base], max_new=24, sampling=opt)[0]
                if opt is None:
                    assert out == plain, kind
                else:
                    # sampled rounds preserve the law, not the sample path; they must be
                    # reproducible for a fixed seed
                    eng2 = _engine(weights, load=LoadOptions(prompt_lookup=True, mtp_drafts=3))
                    eng2.spec.drafts_for = eng.spec.drafts_for
                    assert eng2.generate([base], max_new=24, sampling=opt)[0] == out
                    assert len(out) == 24
                    continue
                st = eng.spec.statistics()
                if kind == "oracle":
                    assert st["acceptance_rate"] == 1.0 and eng.stats.iterations < ref_eng.stats.iterations
                if kind == "wrong":
                    assert st["rounds"] > 0 and st["accepted_draft_tokens"] == 0
        finally:
            del os.environ["ORINFER_SINGLE_MTP_POLICY"]
    # adaptive controller path (width chosen from measured costs and acceptance)
    eng = _engine(weights, load=LoadOptions(prompt_lookup=True))
    greedy = _engine(weights).generate([base], max_new=24)[0]
    eng.spec.drafts_for = lambda r, c: greedy[len(r.generated):len(r.generated) + c]
    assert eng.generate([base], max_new=24)[0] == greedy


def test_draft_rows_go_to_the_requests_whose_drafts_survive(weights, monkeypatch):
    """A round's draft rows are placed by each request's own acceptance history: with two
    requests whose drafts are always right and two whose drafts are always wrong, the same row
    budget commits more tokens than equal shares do, and every text stays the plain one."""
    from orinfer_b200.core import policy as P
    assert P.mtp_allocate([0.9, 0.9, 0.1, 0.5], [3, 3, 3, 3], 6) == [3, 3, 0, 0]
    assert P.mtp_allocate([0.7, 0.7, 0.7], [3, 3, 3], 4) == [2, 1, 1]      # ties: fewest rows first
    assert P.mtp_allocate([0.9, 0.2], [3, 3], 6, 0.1) == [3, 1]            # 0.2^2 is under the floor
    assert P.mtp_allocate([0.9, 0.8], [2, 0], 6) == [2, 0]                 # caps
    assert P.mtp_allocate([], [], 4) == []
    monkeypatch.setenv("ORINFER_SINGLE_MTP_POLICY", "fixed2")
    prompts = _prompts(4, 16, seed=21)
    plain = _engine(weights).generate(prompts, max_new=24)
    text = {tuple(p): t for p, t in zip(prompts, plain)}

    def drafts(r, c):
        d = list(text[tuple(r.prompt)][len(r.generated):len(r.generated) + c])
        return d if tuple(r.prompt) in (tuple(prompts[0]), tuple(prompts[1])) else \
            [(t + 1) % 1024 for t in d]

    stats = {}
    for mode in ("uniform", "adaptive"):
        monkeypatch.setenv("ORINFER_MTP_ALLOCATION", mode)
        eng = _engine(weights, load=LoadOptions(prompt_lookup=True, mtp_drafts=3))
        eng.spec.drafts_for = drafts
        assert eng.generate(prompts, max_new=24) == plain, mode
        stats[mode] = eng.spec.statistics()
    uni, ada = stats["uniform"], stats["adaptive"]
    assert ada["acceptance_rate"] > uni["acceptance_rate"] + 0.15
    assert ada["rounds"] <= uni["rounds"]


def test_mtp_head_speculation_preserves_greedy_output():
    """Draft-head rounds (catch-up over the prompt, draft loop, verify, commit) leave the
    greedy text unchanged; the head of a random-init model rarely guesses right."""
    import dataclasses, os
    cfg = dataclasses.replace(PRESETS["tiny"], mtp_layers=1)
    w = random_model(cfg, seed=4)
    prompts = _prompts(2, 20, seed=8)
    plain = _engine(w, load=LoadOptions(mtp_drafts=0)).generate(prompts, max_new=10)
    os.environ["ORINFER_SINGLE_MTP_POLICY"] = "fixed2"
    try:
        eng = _engine(w, load=LoadOptions(mtp_drafts=2))
        assert eng.runner_has_mtp() and eng.spec.enabled
        out = eng.generate(prompts, max_new=10)
        # a contract whose largest draft profile is one request: the draft head runs once per
        # request instead of once per batch, with the same result
        split = _engine(w, load=LoadOptions(mtp_drafts=2))
        split.spec.contract = dataclasses.replace(split.spec.contract, batch_draft_profiles=(1,))
        assert split.generate(prompts, max_new=10) == plain
        assert split.spec.statistics()["rounds"] > 0
    finally:
        del os.environ["ORINFER_SINGLE_MTP_POLICY"]
    assert out == plain
    st = eng.spec.statistics()
    assert st["rounds"] > 0 and st["proposed_tokens"] >= 2 * st["rounds"]


def test_drafts_are_verified_inside_packets_that_carry_prompt_chunks(monkeypatch):
    """A prompt that arrives while others decode does not stop their speculation: the greedy
    decoders' verification rows travel in the same packets as its chunks.  Texts equal plain
    decoding for right, wrong and half-right drafts and for the draft head; a sampled decoder
    rides along with one row."""
    import dataclasses
    monkeypatch.setenv("ORINFER_SINGLE_MTP_POLICY", "fixed3")
    cfg = dataclasses.replace(PRESETS["tiny"], mtp_layers=1)
    w = random_model(cfg, seed=4)
    early = _prompts(2, 12, seed=5)
    late = _prompts(1, 150, seed=6)[0]
    sampled = SamplingOptions(temperature=0.7, seed=9)

    def run(load, drafts=None, sampler=None):
        eng = _engine(w, load=load, prefill_chunk=32, max_active=4)
        if drafts is not None:
            eng.spec.drafts_for = lambda r, c: drafts(r, c)
        reqs = [eng.submit(early[0], 40), eng.submit(early[1], 40, sampling=sampler)]
        for _ in range(2):
            eng.step()
        reqs.append(eng.submit(late, 6))              # five 32-row chunks beside the decoders
        while eng.has_work():
            eng.step()
        return eng, reqs

    _, want = run(LoadOptions(mtp_drafts=0))
    text = {tuple(r.prompt): r.generated for r in want}
    oracle = lambda r, c: text[tuple(r.prompt)][len(r.generated):len(r.generated) + c]
    wrong = lambda r, c: [(t + 1) % cfg.vocab for t in oracle(r, c)]
    half = lambda r, c: oracle(r, c)[:1] + wrong(r, c)[1:]
    for name, drafts in (("oracle", oracle), ("wrong", wrong), ("half", half)):
        eng, got = run(LoadOptions(prompt_lookup=True, mtp_drafts=3), drafts)
        assert [r.generated for r in got] == [r.generated for r in want], name
        assert eng.stats.mixed_verify_packets >= 2, name
        st = eng.spec.statistics()
        if name == "oracle":
            assert st["acceptance_rate"] == 1.0
        if name == "wrong":
            assert st["accepted_draft_tokens"] == 0 and st["proposed_tokens"] > 0
    # the draft head proposes (its backlog stays whole across mixed packets)
    eng, got = run(LoadOptions(mtp_drafts=2))
    assert eng.runner_has_mtp() and eng.stats.mixed_verify_packets >= 2
    assert [r.generated for r in got] == [r.generated for r in want]
    # a sampled decoder keeps its sample path: it never drafts inside a mixed packet
    _, want_s = run(LoadOptions(mtp_drafts=0), sampler=sampled)
    eng, got_s = run(LoadOptions(prompt_lookup=True, mtp_drafts=3), oracle_s := (
        lambda r, c: {tuple(q.prompt): q.generated for q in want_s}[tuple(r.prompt)]
        [len(r.generated):len(r.generated) + c]), sampler=sampled)
    assert got_s[0].generated == want_s[0].generated and got_s[2].generated == want_s[2].generated
    assert len(got_s[1].generated) == 40


def test_host_kv_offload_restores_evicted_prefix(weights):
    """With a host tier, prefixes evicted under page pressure come back from pinned host memory
    instead of being recomputed, and the restored KV gives the same tokens."""
    base = _prompts(3, 130, seed=11)
    load = LoadOptions(kv_offload_bytes=64 << 20)
    eng = _engine(weights, kv_pages=4, max_active=1, prefill_chunk=256, load=load)
    first = [eng.generate([p], max_new=4)[0] for p in base]       # 3 usable pages: must evict
    assert eng.stats.offloaded_pages >= 1 and eng.prefix.statistics().host_pages >= 1
    r = eng.submit(base[0], 4)
    while not r.finished:
        eng.step()
    assert eng.stats.restored_pages >= 1 and r.cached_tokens == 128
    assert r.generated == first[0]
    cold = _engine(weights, load=LoadOptions(prefix_cache_bytes=0))
    assert cold.generate([base[0]], max_new=4)[0] == first[0]


def test_host_tier_slots_are_all_accounted_for_under_traffic(weights):
    """Prompt families that share pages, far more of them than device pages: pages go to the
    host tier, come back, are re-adopted by recomputed prompts and dropped.  Every slot of the
    host slab is then either free or owned by a node the tree still indexes."""
    import random
    rng = random.Random(3)
    load = LoadOptions(kv_offload_bytes=8 * 4 * 2 * 128 * 2 * 32 * 2)      # a handful of slots
    eng = _engine(weights, kv_pages=5, max_active=1, prefill_chunk=256, load=load)
    assert 2 <= eng.host_kv.slots <= 64
    stems = [_prompts(1, 128, seed=20 + i)[0] for i in range(3)]
    tails = [_prompts(1, 130, seed=40 + i)[0] for i in range(4)]
    for _ in range(40):
        stem = rng.choice(stems)
        prompt = stem + rng.choice(tails) if rng.random() < 0.6 else stem + [7, 8, 9]
        eng.generate([prompt], max_new=2)
        live = eng.prefix.statistics().host_pages
        assert eng.host_kv.available + live == eng.host_kv.slots
    assert eng.stats.offloaded_pages > 0 and eng.stats.restored_pages > 0


def test_layered_prefill_lets_decoders_step_inside_a_long_prompt(weights):
    """A prompt that joins while another request decodes is run as a paused packet: the
    decoder takes a step at every layer-boundary pause and both texts stay what they were."""
    short, long_ = _prompts(1, 16)[0], _prompts(1, 96)[0]
    plain = _engine(weights, prefill_chunk=128)
    want = [plain.generate([p], max_new=n)[0] for p, n in ((short, 12), (long_, 4))]
    eng = Engine(weights, kv_pages=24, max_context=512,
                 sched=SchedulerOptions(max_active=4, prefill_chunk=128, prefill_stages=2,
                                        layered_min_rows=64))
    a = eng.submit(short, 12)
    eng.step()                                   # a is decoding when the long prompt arrives
    eng.step()
    at = len(a.generated)
    b = eng.submit(long_, 4)
    eng.step()                                   # one iteration: whole prompt + one pause
    assert eng.stats.layered_decode_steps == 1
    assert len(a.generated) == at + 1 and len(b.generated) == 1
    while eng.has_work():
        eng.step()
    assert [a.generated, b.generated] == want


def test_packed_uploads_equal_single_uploads_and_reuse_the_ring(weights, monkeypatch):
    """All index arrays of a packet travel in one staged copy; the views must hold what
    separate uploads hold, through many wrap-arounds of the ring, with empty arrays, and fall
    back for a packet that is too large for a region."""
    import random
    eng = _engine(weights)
    rng = random.Random(0)
    for step in range(300):
        parts = {"ids": [rng.randrange(1000) for _ in range(rng.randrange(0, 700))],
                 "req": [rng.randrange(4) for _ in range(rng.randrange(0, 700))],
                 "none": None, "sel": [rng.randrange(9)], "empty": []}
        got = eng._upload_many(parts)
        assert set(got) == {"ids", "req", "sel", "empty"}
        for k, v in got.items():
            assert v.dtype == torch.int32 and v.tolist() == parts[k] and v.is_contiguous()
    assert eng.stats.packed_uploads == 300
    big = {"ids": list(range(eng.STAGE_BYTES // 8))}          # over a quarter of the ring
    assert eng._upload_many(big)["ids"].tolist() == big["ids"]
    assert eng.stats.packed_uploads == 300
    # a ring much smaller than the traffic: regions are reused only after they were retired
    monkeypatch.setattr(type(eng), "STAGE_BYTES", 1 << 14)
    small = _engine(weights)
    for step in range(200):
        parts = {"a": [step] * 500, "b": [step + 1] * 300}
        got = small._upload_many(parts)
        assert got["a"].tolist() == parts["a"] and got["b"].tolist() == parts["b"]
    st = small._stage_ring.stats()
    assert st["live"] == 0 and st["peak"] <= 1 << 14 and small.stats.packed_uploads == 200
    # a failure inside the packed path switches it off and the plain path carries on
    from orinfer_b200.core import transfers
    broken = _engine(weights)
    monkeypatch.setattr(transfers, "pack_inputs", lambda *a, **k: 1 / 0)
    assert broken._upload_many({"a": [4, 5], "b": [6]})["b"].tolist() == [6]
    assert broken._packed_uploads is False
    monkeypatch.undo()
    monkeypatch.setenv("ORINFER_PACKED_UPLOAD", "0")
    plain = _engine(weights)
    assert plain._upload_many({"a": [1, 2, 3]})["a"].tolist() == [1, 2, 3]
    assert plain.stats.packed_uploads == 0 and plain._stage is None


def test_follower_commands_check_what_they_can(weights):
    """``Engine.apply`` is what a follower rank runs: a host-tier save must land in the slot
    the leader announced, a host-tier command needs a store, unknown commands are refused."""
    from orinfer_b200.engine.offload import HostKvStore
    eng = _engine(weights, load=LoadOptions(prefix_cache_bytes=0))
    with pytest.raises(ValueError, match="without a host KV store"):
        eng.apply("host_kv", ("save", 1, 0))
    eng.host_kv = HostKvStore(eng.kv, 8 << 20)
    first = eng.host_kv._free[-1]
    eng.apply("host_kv", ("save", 1, first))                  # the slot the store hands out next
    with pytest.raises(ValueError, match="out of step"):
        eng.apply("host_kv", ("save", 2, first))              # the leader says an occupied slot
    eng.apply("host_kv", ("load", first, 3))
    eng.apply("host_kv", ("free", first))
    eng.apply("host_kv", ("sync",))
    eng.apply("page_row", (0, [1, 2]))
    eng.apply("verify", ([5, 6, 7], [0, 0, 0], [0, 1, 2], 3, False))      # runs, returns nothing
    with pytest.raises(ValueError, match="do not add up"):
        eng.apply("verify", ([5, 6, 7], [0, 0, 0], [0, 1, 2], 3, False, [2, 2]))
    with pytest.raises(ValueError, match="without a tentative"):
        eng.apply("verify_commit", [1])
    with pytest.raises(ValueError, match="no recurrent-state copy"):
        eng.apply("state_copy", ("restore", 7, 0))
    eng.apply("state_copy", ("drop", 7, -1))                  # dropping twice is harmless
    with pytest.raises(ValueError, match="unknown device command"):
        eng.apply("reboot", None)


def test_a_request_whose_constraint_breaks_fails_alone(weights):
    """What goes wrong while one request's token is chosen ends that request with an error;
    the engine keeps serving the others and the text of a bystander is unchanged."""
    class Breaks:
        def __init__(self, after):
            self.left = after

        def mask(self, vocab):
            return None

        def consume(self, token):
            self.left -= 1
            if self.left < 0:
                raise ValueError("grammar cannot follow this token\nlong state dump")

        def finished(self):
            return False

    prompts = _prompts(2, 20, seed=31)
    want = _engine(weights).generate([prompts[1]], max_new=8)[0]
    eng = _engine(weights)
    bad = eng.submit(prompts[0], 8)
    bad.constraint = Breaks(after=3)
    good = eng.submit(prompts[1], 8)
    while eng.has_work():
        eng.step()                                        # never raises
    assert bad.finished and bad.finish_reason == "error" and len(bad.generated) == 3
    assert bad.error == "ValueError: grammar cannot follow this token"
    assert good.generated == want and good.error is None
    assert eng.stats.failed_requests == 1 and eng.failed is None
    again = eng.generate([prompts[0]], max_new=4)         # its slot and pages came back
    assert len(again[0]) == 4
