"""The single-request reference path is the isolation oracle for batched / chunked runs."""
import pytest

from orinfer_b200.config import PRESETS, SchedulerOptions
from orinfer_b200.engine.engine import Engine
from orinfer_b200.models.weights import random_model


@pytest.mark.parametrize("preset", ["tiny", "tiny-moe", "tiny-hybrid"])
def test_batched_chunked_runs_match_the_isolated_reference(preset):
    weights = random_model(PRESETS[preset], seed=1)
    prompts = [[(7 * i + 3 * j) % 250 + 1 for j in range(n)] for i, n in enumerate((5, 37, 70, 19))]

    def engine(chunk):
        return Engine(weights, sched=SchedulerOptions(max_active=4, prefill_chunk=chunk),
                      kv_pages=24, max_context=256)

    ref = [engine(32).generate_reference(p, max_new=6, chunk=32) for p in prompts]
    assert all(len(r) == 6 for r in ref)
    assert engine(16).generate(prompts, max_new=6) == ref           # batched + other chunking
    eng = engine(32)
    assert [eng.generate_reference(p, max_new=6, chunk=8) for p in prompts] == ref
    assert eng.generate([prompts[1]], max_new=6)[0] == ref[1]       # slot and pages were returned
    eng.submit(prompts[0], 4)
    with pytest.raises(RuntimeError, match="idle"):
        eng.generate_reference(prompts[0])
    with pytest.raises(ValueError):
        engine(32).generate_reference([1] * 250, max_new=10)
