"""Media rows and the single-request reference path on the CUDA runner."""
import numpy as np
import pytest
import torch

from orinfer_b200.config import PRESETS, GraphMode, LoadOptions, SchedulerOptions
from orinfer_b200.engine.engine import Engine
from orinfer_b200.engine.request import MediaSpan
from orinfer_b200.models.weights import random_model
from orinfer_b200.ref import ops_ref as R

pytestmark = pytest.mark.gpu


def _engine(w, chunk=64, graph=GraphMode.DECODE_ONLY):
    return Engine(w, load=LoadOptions(cuda_graph=graph),
                  sched=SchedulerOptions(max_active=4, prefill_chunk=chunk),
                  kv_pages=40, max_context=1024)


def test_overlay_rows_equal_the_tokens_they_stand_for(cuda):
    """Placeholders overlaid with the embeddings of other tokens, at ordinary positions,
    generate what the prompt holding those tokens generates (chunk boundaries inside the span),
    and identity (t, h, w) positions give the ordinary rotary table."""
    cpu = random_model(PRESETS["tiny"], seed=0)
    w = random_model(PRESETS["tiny"], seed=0).to(cuda)
    real = [3, 7, 11] + list(range(40, 140)) + [5, 9, 2]
    masked = real[:3] + [900] * 100 + real[103:]
    feats = R.embed_w8(torch.tensor(real[3:103]), cpu.embed_q, cpu.embed_s)
    want = _engine(w).generate([real], max_new=8)[0]
    eng = _engine(w, chunk=32)
    pos = np.tile(np.arange(len(masked), dtype=np.int32), (3, 1))
    req = eng.submit(masked, max_new=8, media=[MediaSpan(3, 103, feats, 77)], rope_positions=pos)
    while eng.has_work():
        eng.step()
    assert req.generated == want
    assert eng.stats.graph_hits >= 1              # decode steps went back to the graph path
    shifted = _engine(w, chunk=32)
    req2 = shifted.submit(masked, max_new=8, media=[MediaSpan(3, 103, feats, 77)],
                          rope_positions=pos, rope_delta=-40)
    while shifted.has_work():
        shifted.step()
    assert len(req2.generated) == 8 and shifted.stats.graph_hits == 0


@pytest.mark.parametrize("preset", ["tiny", "tiny-hybrid"])
def test_reference_generation_matches_batched_runs(cuda, preset):
    w = random_model(PRESETS[preset], seed=1).to(cuda)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(1, 1000, (n,), generator=g).tolist() for n in (5, 150, 70)]
    ref = [_engine(w).generate_reference(p, max_new=6, chunk=64) for p in prompts]
    assert _engine(w, chunk=128, graph=GraphMode.OFF).generate(prompts, max_new=6) == ref


def test_bidirectional_encoder_matches_the_cpu_runner(cuda):
    """Encoder passes on the CUDA runner (row attention kernel with the last position as every
    row's horizon) against the PyTorch runner on the same weights."""
    cfg = PRESETS["tiny-embed"]
    cpu_w = random_model(cfg, seed=3)
    ids = torch.randint(1, 1000, (150,), generator=torch.Generator().manual_seed(8)).tolist()
    want, want_logits = Engine(cpu_w, sched=SchedulerOptions(max_active=2, prefill_chunk=256),
                               kv_pages=16, max_context=512).encode(ids)
    got, got_logits = _engine(random_model(cfg, seed=3).to(cuda)).encode(ids)
    assert torch.nn.functional.cosine_similarity(got, want, dim=0) > 0.999
    assert torch.nn.functional.cosine_similarity(got_logits, want_logits, dim=0) > 0.995
    causal = _engine(random_model(PRESETS["tiny"], seed=3).to(cuda)).encode(ids)[0]
    assert torch.nn.functional.cosine_similarity(causal, want, dim=0) < 0.999   # it matters
