"""Paired next-token probe analysis and the score-model adapters."""
import json
import math

import numpy as np
import pytest

from orinfer_b200.bench import quality as Q


def logits(seed, positions=6, vocab=32):
    return np.random.default_rng(seed).standard_normal((positions, vocab)).astype(np.float32) * 3


TOKENS = [3, 9, 1, 4, 7, 2]


def test_identical_scorers_agree_exactly():
    lg = logits(0)
    base = Q.probes_from_logits(lg, TOKENS, "a")
    cand = Q.probes_from_logits(lg, TOKENS, "a", query=Q.queries_from(base))
    assert len(base) == 5 and base[0]["context_sha256"] == Q.context_sha256(TOKENS[:1])
    rep = Q.analyze(Q.pair(base, cand))["aggregate"]
    assert rep["positions"] == 5 and rep["top1_agreement"] == 1 and rep["top3_overlap"] == 1
    assert rep["mean_abs_probability_error"] == 0 and rep["delta_target_nll"] == 0
    p = base[2]
    assert math.isclose(sum(math.exp(x) for x in Q.log_softmax(lg[2])), 1.0, rel_tol=1e-9)
    assert p["top3"][0]["logprob"] >= p["top3"][1]["logprob"] >= p["top3"][2]["logprob"]
    assert p["reference_token_id"] == TOKENS[3]


def test_perturbed_candidate_is_measured():
    lg = logits(1)
    noisy = lg.copy()
    top = int(np.argmax(lg[0]))
    noisy[0, top] -= 50.0                                   # position 1 flips its top-1
    base = Q.probes_from_logits(lg, TOKENS, "a")
    cand = Q.probes_from_logits(noisy, TOKENS, "a", query=Q.queries_from(base))
    rep = Q.analyze(Q.pair(base, cand))
    agg = rep["aggregate"]
    assert agg["top1_agreement"] == pytest.approx(4 / 5) and agg["mean_abs_logprob_error"] > 1
    assert rep["by_case_and_mode"][0]["case_id"] == "a"
    tie = np.zeros((2, 8), dtype=np.float32)
    assert [t["token_id"] for t in Q.top3_of(Q.log_softmax(tie[0]))] == [0, 1, 2]   # lower id wins


def test_unpairable_or_incomplete_probes_are_refused():
    lg = logits(2)
    base = Q.probes_from_logits(lg, TOKENS, "a")
    other = Q.probes_from_logits(lg, [3, 8] + TOKENS[2:], "a", query=Q.queries_from(base))
    with pytest.raises(Q.ProbeError, match="history mismatch"):
        Q.pair(base, other)
    with pytest.raises(Q.ProbeError, match="no probe"):
        Q.pair(base, base[:2])
    with pytest.raises(Q.ProbeError, match="duplicate"):
        Q.pair(base + base[:1], base)
    shifted = lg.copy()
    shifted[:, :16] += 40.0 * (np.arange(16) % 2)          # candidate's top-3 elsewhere, no query
    cand = Q.probes_from_logits(shifted, TOKENS, "a")
    with pytest.raises(Q.ProbeError, match="query it"):
        Q.analyze(Q.pair(base, cand))
    broken = json.loads(json.dumps(base))
    broken[0]["top3"][0]["logprob"] = 0.5
    with pytest.raises(Q.ProbeError, match="full-vocabulary"):
        Q.analyze(Q.pair(broken, broken))
    with pytest.raises(Q.ProbeError, match="no scoring records"):
        Q.analyze([])


def test_score_model_adapters_and_cli(tmp_path, capsys):
    from orinfer_b200 import cli
    base, cand = tmp_path / "b.jsonl", tmp_path / "c.jsonl"
    toks = ",".join(map(str, range(1, 20)))
    common = ["score-model", "--preset", "tiny", "--device", "cpu", "--tokens", toks]
    assert cli.main(common + ["--jsonl", str(base)]) == 0
    assert cli.main(common + ["--jsonl", str(cand), "--query-from", str(base)]) == 0
    capsys.readouterr()
    assert cli.main(["bench", "quality", "--baseline", str(base), "--candidate", str(cand),
                     "--min-top1", "1.0"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["aggregate"]["positions"] == 18 and rep["aggregate"]["top1_agreement"] == 1.0
