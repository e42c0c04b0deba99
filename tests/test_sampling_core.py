"""Host sampling law and counter RNG (CPU)."""
import math

import numpy as np
import pytest

from orinfer_b200.core import sampling as S


def _splitmix_py(x):
    m = 2 ** 64 - 1
    x = (x + 0x9E3779B97F4A7C15) & m
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & m
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & m
    return x ^ (x >> 31)


def test_counter_rng_matches_definition():
    for seed, stream, step in [(0, 0, 0), (20261002, 0, 5), (2 ** 63 + 11, S.ACCEPT_STREAM, 999)]:
        bits = _splitmix_py(_splitmix_py(seed ^ stream) ^ step) >> 11
        assert S.counter_uniform(seed, stream, step) == bits / 2 ** 53
    assert S.splitmix64(0) == _splitmix_py(0)
    k = _splitmix_py(_splitmix_py(7) ^ 3)
    assert S.categorical_key(7, 3) == (k & 0xFFFFFFFF, k >> 32)


def test_philox_reference_vector():
    # Random123 known-answer test for philox2x32-10: counter (0,0), key 0
    assert S.philox2x32_10((0, 0), 0) == (0xFF1DAE59, 0x6CD10DF2)
    assert S.philox2x32_10((0xFFFFFFFF, 0xFFFFFFFF), 0xFFFFFFFF) == (0x2C3F628B, 0xAB4FD7AD)


def test_round_step_layout():
    assert S.round_step(0, 5) == (1 << 32) | 5
    with pytest.raises(ValueError):
        S.round_step(2 ** 32 - 1, 0)


def test_validation():
    S.SamplingOptions().validate()
    for bad in (dict(temperature=2.5), dict(top_p=0.0), dict(presence_penalty=3),
                dict(repetition_penalty=0.0), dict(logit_bias={1: 101.0}), dict(top_logprobs=21)):
        with pytest.raises(ValueError):
            S.SamplingOptions(**bad).validate()
    assert S.SamplingOptions(temperature=0).is_greedy
    assert not S.SamplingOptions(temperature=0, logit_bias={1: 1.0}).is_greedy
    assert S.SamplingOptions().device_categorical
    assert not S.SamplingOptions(top_k=5).device_categorical


def test_greedy_ties_go_to_lowest_id():
    lg = np.array([0.5, 2.0, 2.0, -1.0], np.float32)
    assert S.sample(lg, [], S.GREEDY, 0.3) == 1
    assert S.law(lg, [], S.GREEDY) == [(1, 1.0)]


def test_law_topk_topp_and_order():
    lg = np.log(np.array([0.1, 0.4, 0.2, 0.3], np.float64)).astype(np.float32)
    full = S.law(lg, [], S.SamplingOptions())
    assert [i for i, _ in full] == [1, 3, 2, 0]
    assert abs(sum(p for _, p in full) - 1) < 1e-12
    assert [i for i, _ in S.law(lg, [], S.SamplingOptions(top_k=2))] == [1, 3]
    nucleus = S.law(lg, [], S.SamplingOptions(top_p=0.65))
    assert [i for i, _ in nucleus] == [1, 3]
    assert abs(nucleus[0][1] - 0.4 / 0.7) < 1e-6
    assert S.sample(lg, [], S.SamplingOptions(), 0.39) == 1
    assert S.sample(lg, [], S.SamplingOptions(), 0.41) == 3
    assert S.sample(lg, [], S.SamplingOptions(), 0.999999) == 0


def test_penalties_bias_mask():
    lg = np.array([1.0, 1.0, -1.0, 0.0], np.float32)
    o = S.SamplingOptions(temperature=0, repetition_penalty=2.0, presence_penalty=0.5,
                          frequency_penalty=0.25)
    # token 0 seen twice: 1/2 - 0.5 - 0.5 = -0.5 ; token 1 unseen stays 1.0
    assert S.sample(lg, [0, 0, 2], o, 0.0) == 1
    lp, _ = S.logprobs(lg, [0, 0, 2], S.SamplingOptions(repetition_penalty=2.0), 2, 0)
    scores = np.array([0.5, 1.0, -2.0, 0.0])
    assert abs(lp - (scores[2] - math.log(np.exp(scores).sum()))) < 1e-12
    assert S.sample(lg, [], S.SamplingOptions(temperature=0, logit_bias={3: 5.0}), 0.0) == 3
    mask = np.array([0b1100], np.uint32)
    assert S.sample(lg, [], S.GREEDY, 0.0, mask) == 3
    with pytest.raises(ValueError):
        S.sample(lg, [], S.GREEDY, 0.0, np.array([0], np.uint32))
    with pytest.raises(ValueError):
        S.sample(np.array([np.nan, 1], np.float32), [], S.GREEDY, 0.0)


def test_logprobs_top_n_sorted():
    lg = np.array([0.0, 3.0, 1.0, 2.0], np.float32)
    lp, top = S.logprobs(lg, [], S.SamplingOptions(), 1, 3)
    assert [i for i, _ in top] == [1, 3, 2]
    assert abs(top[0][1] - lp) < 1e-15


def test_greedy_commit():
    assert S.greedy_commit([5, 6, 7], [5, 6, 9, 1]) == [5, 6, 9]
    assert S.greedy_commit([5, 6], [5, 6, 2]) == [5, 6, 2]
    assert S.greedy_commit([4], [5, 6]) == [5]
    with pytest.raises(ValueError):
        S.greedy_commit([1], [1])


def test_rejection_sampling_preserves_target_law():
    """First committed token of a speculative round follows the target law even when the
    draft law is different (statistical check over many independent seeds)."""
    rng = np.random.default_rng(0)
    vocab = 6
    target = rng.normal(size=(2, vocab)).astype(np.float32)
    p = np.exp(target[0].astype(np.float64)); p /= p.sum()
    q = np.array([0.4, 0.05, 0.05, 0.3, 0.1, 0.1])
    counts = np.zeros(vocab)
    n = 20000
    for seed in range(n):
        o = S.SamplingOptions(seed=seed)
        draft = int(np.searchsorted(np.cumsum(q), S.counter_uniform(seed, S.DRAFT_STREAM, 0)))
        out = S.sampled_commit([draft], q[None, :], target, [], o, 0)
        counts[out[0]] += 1
    assert np.abs(counts / n - p).max() < 0.012


def test_sampled_commit_point_mass_and_determinism():
    lg = np.zeros((3, 4), np.float32)
    lg[:, 2] = 20.0                      # target is (almost) a point mass on token 2
    o = S.SamplingOptions(seed=11)
    assert S.sampled_commit([2, 2], None, lg, [], o, 0) == [2, 2, 2]
    first = S.sampled_commit([1, 2], None, lg, [], o, 0)
    assert first == [2] and first == S.sampled_commit([1, 2], None, lg, [], o, 0)
