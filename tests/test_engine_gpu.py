"""Engine on the CUDA runner: graph modes, batch invariance, prefix reuse."""
import pytest
import torch

from orinfer_b200.config import PRESETS, GraphMode, LoadOptions, SchedulerOptions
from orinfer_b200.core.sampling import SamplingOptions
from orinfer_b200.engine.engine import Engine
from orinfer_b200.models.weights import random_model

pytestmark = pytest.mark.gpu


def _prompts(n, length, seed=1, vocab=1024):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def _engine(w, graph=GraphMode.DECODE_ONLY, **kw):
    return Engine(w, load=LoadOptions(cuda_graph=graph, **kw.pop("load", {})),
                  sched=SchedulerOptions(max_active=8, prefill_chunk=kw.pop("chunk", 256)),
                  kv_pages=40, max_context=1024)


def test_graph_modes_agree_and_replay_changed_inputs(cuda):
    w = random_model(PRESETS["tiny"], seed=0).to(cuda)
    prompts = _prompts(3, 40)
    off = _engine(w, GraphMode.OFF).generate(prompts, max_new=12)
    eng = _engine(w, GraphMode.DECODE_ONLY)
    on = eng.generate(prompts, max_new=12)
    assert on == off
    assert eng.stats.graph_captures >= 1 and eng.stats.graph_hits >= 5
    # same captured graphs, different requests
    more = _prompts(3, 33, seed=9)
    assert eng.generate(more, max_new=12) == _engine(w, GraphMode.OFF).generate(more, max_new=12)


def test_full_graph_mode_replays_prefill_geometries(cuda):
    """FULL mode: a prefill geometry is captured at its second use and replayed with new
    token ids; outputs equal the graph-free engine."""
    w = random_model(PRESETS["tiny"], seed=0).to(cuda)
    prompts = _prompts(5, 150, seed=21)
    off = [_engine(w, GraphMode.OFF).generate([p], max_new=6)[0] for p in prompts]
    eng = _engine(w, GraphMode.FULL)
    on = [eng.generate([p], max_new=6)[0] for p in prompts]
    assert on == off
    assert len(eng._prefill_graphs) == 1 and eng.stats.graph_hits >= 3 + 5 * 3
    other = _prompts(1, 77, seed=22)                      # a new geometry runs direct first
    assert eng.generate(other, max_new=4) == _engine(w, GraphMode.OFF).generate(other, max_new=4)


def test_batch_invariance_and_chunked_prefill(cuda):
    w = random_model(PRESETS["tiny"], seed=1).to(cuda)
    prompts = _prompts(4, 150, seed=2)
    solo = [_engine(w).generate([p], max_new=10)[0] for p in prompts]
    eng = _engine(w, chunk=64)
    reqs = [eng.submit(prompts[0], 10)]
    eng.step()
    reqs += [eng.submit(p, 10) for p in prompts[1:]]
    while eng.has_work():
        eng.step()
    assert [r.generated for r in reqs] == solo


def test_prefix_reuse_on_device(cuda):
    w = random_model(PRESETS["tiny"], seed=2).to(cuda)
    base = _prompts(1, 300, seed=3)[0]
    eng = _engine(w)
    first = eng.generate([base], max_new=6)[0]
    r = eng.submit(base, 6)
    while not r.finished:
        eng.step()
    assert r.cached_tokens == 256 and r.generated == first


def test_sampled_rows_use_host_law(cuda):
    w = random_model(PRESETS["tiny"], seed=3).to(cuda)
    prompts = _prompts(2, 24, seed=4)
    opt = SamplingOptions(temperature=0.8, top_k=20, seed=7)
    eng = _engine(w)
    a = eng.generate(prompts, max_new=8, sampling=opt)
    b = _engine(w).generate(prompts[:1], max_new=8, sampling=opt)
    assert a[0] == b[0]
    assert eng.stats.device_samples == 16              # drawn by the device top-k sampler
    host = _engine(w)
    host._device_samples = lambda order, logits: {}    # same steps through the host law
    assert host.generate(prompts, max_new=8, sampling=opt) == a
    pen = SamplingOptions(temperature=0.8, top_k=20, seed=7, presence_penalty=0.5)
    eng2 = _engine(w)
    eng2.generate(prompts, max_new=4, sampling=pen)    # penalties need history: host law
    assert eng2.stats.device_samples == 0


def test_host_kv_offload_on_device(cuda):
    w = random_model(PRESETS["tiny"], seed=3).to(cuda)
    base = _prompts(3, 130, seed=11)
    eng = Engine(w, load=LoadOptions(cuda_graph=GraphMode.OFF, kv_offload_bytes=64 << 20),
                 sched=SchedulerOptions(max_active=1, prefill_chunk=256), kv_pages=4,
                 max_context=512)
    first = [eng.generate([p], max_new=4)[0] for p in base]
    assert eng.stats.offloaded_pages >= 1
    r = eng.submit(base[0], 4)
    while not r.finished:
        eng.step()
    assert eng.stats.restored_pages >= 1 and r.cached_tokens == 128 and r.generated == first[0]


def test_mtp_head_speculation_on_device(cuda, monkeypatch):
    import dataclasses
    cfg = dataclasses.replace(PRESETS["tiny"], mtp_layers=1)
    w = random_model(cfg, seed=4).to(cuda)
    prompts = _prompts(2, 20, seed=8)
    plain = _engine(w, load=dict(mtp_drafts=0)).generate(prompts, max_new=10)
    monkeypatch.setenv("ORINFER_SINGLE_MTP_POLICY", "fixed2")
    eng = _engine(w, load=dict(mtp_drafts=2))
    assert eng.runner_has_mtp()
    assert eng.generate(prompts, max_new=10) == plain
    assert eng.spec.statistics()["rounds"] > 0


@pytest.mark.parametrize("preset", ["tiny", "tiny-hybrid"])
def test_layered_prefill_pauses_keep_both_texts(cuda, preset):
    """The paused prompt packet gets its hidden rows, residual and RoPE table back after the
    decoders used the same workspace (graph replay included)."""
    w = random_model(PRESETS[preset], seed=0).to(cuda)
    short, long_ = _prompts(1, 16)[0], _prompts(1, 200, seed=4)[0]

    def run(stages):
        eng = Engine(w, load=LoadOptions(cuda_graph=GraphMode.DECODE_ONLY, prefix_cache_bytes=0),
                     sched=SchedulerOptions(max_active=4, prefill_chunk=256,
                                            prefill_stages=stages, layered_min_rows=64),
                     kv_pages=40, max_context=1024)
        a = eng.submit(short, 14)
        for _ in range(3):
            eng.step()
        b = eng.submit(long_, 5)
        while eng.has_work():
            eng.step()
        return eng, [a.generated, b.generated]

    plain_eng, plain = run(1)
    eng, layered = run(2)
    assert plain_eng.stats.layered_decode_steps == 0 and eng.stats.layered_decode_steps == 1
    # the prompt rows ran without the decode row in their packet; the short request's text
    # must be identical, the long one's first token comes from the same arithmetic per row
    assert layered == plain
