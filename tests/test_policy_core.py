"""Scheduler policy math, adaptive MTP control, prompt lookup, error taxonomy (C++ core)."""
import math

import pytest

from orinfer_b200.core import policy as P


def test_queue_ordering_cost_aging_and_hard_fcfs():
    W = P.Waiting
    assert P.select_waiting([W(0, 5.0), W(0, 1.0), W(0, 3.0)]) == 1
    # smooth aging: cost / (1 + age/2)
    assert P.select_waiting([W(10, 5.0), W(0, 1.0)]) == 0
    # after 30 s the oldest wins whatever it costs
    assert P.select_waiting([W(31, 100.0), W(29, 0.001), W(40, 50.0)]) == 2
    assert P.select_waiting([]) is None


def test_throughput_ranking_prefers_cohort_match_then_long_work():
    W = P.Waiting
    reqs = [W(0, 1), W(0, 1), W(0, 1), W(35, 1)]
    order = P.rank_throughput_waiting(reqs, [10, 100, 1000, 5], cohort_remaining=90)
    assert order[0] == 3 and order[1] == 1
    assert P.rank_throughput_waiting(reqs[:3], [10, 100, 1000], None) == [2, 1, 0]


def test_estimators():
    t = P.Timing()
    t.observe(5.0)                         # first use: capture / lazy load, discarded later
    assert t.samples == 0
    for s in (1.0, 1.0, 1.2):
        t.observe(s)
    assert t.samples == 3 and 1.0 <= t.mean <= 1.1 and t.upper >= t.mean
    t.observe(float("nan"))
    assert t.samples == 3
    o = P.OutputLengths()
    assert o.estimate(100, 50) == 50
    o.observe(128, 256)
    assert o.estimate(100, 1000) == pytest.approx(200) and o.estimate(4000, 1000) == 1000


def test_small_policy_functions():
    assert P.replenish([-0.25, -0.1], 0.2) == pytest.approx([-0.05, 0.1])
    assert P.replenish([0.1, -3.0], 0.2) == [0.1, -3.0]
    assert P.prefill_window(0.5, 0.1, 200) == pytest.approx(0.2)
    assert P.prefill_window(0.05, 0.1, 200) == 0
    assert P.joint_prefill_worthwhile(True, False, 1.0, 2.0) is False
    assert P.joint_prefill_worthwhile(True, True, 1.0, 2.0) is True
    assert P.decode_quantum_s(1.0, 200, 400) == pytest.approx(0.2)
    assert P.admission_should_yield(True, 1, 0.011, False)
    assert not P.admission_should_yield(False, 7, 0.1, False)
    assert P.admission_should_yield(False, 32, 0.0, True)
    text = "MemTotal: 1600 kB\nMemFree: 1 kB\nMemAvailable: 1000 kB\n"
    assert P.usable_host_bytes(text) == (1000 - 100) * 1024
    with pytest.raises(ValueError):
        P.usable_host_bytes("MemTotal: 10 kB\n")


def test_error_taxonomy():
    assert not P.ErrorKind.REQUEST.fatal and not P.ErrorKind.CAPACITY.fatal
    assert P.ErrorKind.CUDA.fatal and P.ErrorKind.NCCL.fatal and P.ErrorKind.INVARIANT.fatal
    assert P.EngineError(P.ErrorKind.OUT_OF_MEMORY, "oom").fatal


def test_acceptance_batch_update_is_order_independent():
    a = P.Acceptance()
    a.observe([(5, 5)] * 16)
    assert a.rate(0) == pytest.approx(1 - 0.3 * 0.8 ** 16)
    b, c = P.Acceptance(), P.Acceptance()
    b.observe([(5, 0), (5, 5)])
    c.observe([(5, 5), (5, 0)])
    assert b.rate(0) == c.rate(0)
    # a rejected prefix does not count its untested suffix as rejections
    d = P.Acceptance()
    d.observe([(3, 0)])
    assert d.rate(1) == 0.7 and d.rate(0) < 0.7
    assert P.Acceptance().expected(3) == pytest.approx(1 + 0.7 + 0.49 + 0.343)
    assert P.mtp_progress([2.0, 2.0], 2, True) == pytest.approx(4.0)
    assert P.mtp_progress([2.0, 3.0], 2, False) == 5.0


def test_mtp_select_prefers_cheaper_tokens_and_respects_slack():
    C = P.Candidate
    hot = dict(samples=5, remaining_tokens=1000)
    # plain decode 10 ms per token; width 4 yields 2.5 tokens in 15 ms = 6 ms per token
    cid, exploring, _ = P.mtp_select(0.010, 1, 1.0, [
        C(1, 2, 1.5, 2, mean_s=0.013, upper_s=0.014, **hot),
        C(2, 4, 2.5, 4, mean_s=0.015, upper_s=0.016, **hot)], allow_exploration=False)
    assert cid == 2 and not exploring
    # too slow for the slack -> plain decode
    assert P.mtp_select(0.010, 1, 0.012, [C(2, 4, 2.5, 4, mean_s=0.015, upper_s=0.016, **hot)],
                        allow_exploration=False)[0] is None
    # not better than baseline * 0.98 -> plain decode
    assert P.mtp_select(0.010, 1, 1.0, [C(2, 4, 1.4, 4, mean_s=0.0139, upper_s=0.015, **hot)],
                        allow_exploration=False)[0] is None
    # an uncalibrated candidate may be probed within the calibration budget
    cid, exploring, calibrating = P.mtp_select(
        0.010, 1, 1.0, [C(3, 3, 2.0, 3, remaining_tokens=1000, mean_s=0.012, upper_s=0.013,
                          samples=0)], calibration_s=1.0)
    assert (cid, exploring, calibrating) == (3, True, True)


def test_prompt_lookup_copies_continuation_and_cools_down():
    lk = P.PromptLookup()
    hist = [1, 2, 3, 4, 5, 6, 7, 8, 9, 1, 2, 3, 4]
    assert lk.propose(hist, 3) == [5, 6, 7]
    assert lk.propose(hist, 3, confident=True) == []        # only 4 tokens of context match
    assert lk.propose([1, 2, 3], 2) == []
    lk.observe(0, 3, len(hist))
    lk.observe(0, 3, len(hist))                             # two misses -> cooldown
    assert lk.propose(hist, 3) == []


def test_cost_curves_exact_interpolated_and_cold():
    from orinfer_b200.core.policy import DIRECT, REPLAY, CostCurves
    c = CostCurves(cold_tokens_per_s=10000.0)
    sec, up, n, path = c.estimate(tokens=500, context=500)
    assert abs(sec - 0.05) < 1e-9 and n == 0 and path == DIRECT          # cold prior
    for _ in range(5):
        c.observe(0.010, tokens=512, context=512)
        c.observe(0.030, tokens=2048, context=512)
        c.observe(0.018, tokens=1024, context=512)
    sec, up, n, _ = c.estimate(tokens=512, context=512)
    assert abs(sec - 0.010) < 1e-9 and n == 5 and up >= sec
    sec, _, n, _ = c.estimate(tokens=768, context=512)                     # between 512 and 1024
    assert 0.010 < sec < 0.018 and n == 0
    sec, _, _, _ = c.estimate(tokens=4096, context=400)                    # beyond the data: linear
    assert abs(sec - 0.060) < 1e-9
    assert c.estimate(tokens=4096, context=4096)[2] == 0                   # another family: cold
    # the family remembers its last path; a path without samples borrows the hot cost
    c.observe(0.008, tokens=512, context=512, path=REPLAY)
    assert c.estimate(tokens=512, context=512)[3] == REPLAY
    # a sample that paid for a capture only primes the cell, a clean one replaces it
    c.observe(0.5, tokens=256, context=256, setup_s=0.4)
    assert abs(c.estimate(tokens=256, context=256)[0] - 0.5) < 1e-9
    c.observe(0.004, tokens=256, context=256)
    assert abs(c.estimate(tokens=256, context=256)[0] - 0.004) < 1e-9
    # chunk sizing against a budget uses the upper estimate
    assert c.fit_tokens(0.012, 4096, 128, context=512) in (512, 640)
    assert c.fit_tokens(1e-6, 4096, 128, context=512) == 128              # never below a quantum


def test_cost_curves_are_bounded():
    from orinfer_b200.core.policy import CostCurves
    c = CostCurves()
    for t in range(1, 400):
        c.observe(0.001 * t, tokens=t, context=64)
    assert c.cells == 256
    assert c.estimate(tokens=399, context=64)[2] == 1 and c.estimate(tokens=1, context=64)[2] == 0
