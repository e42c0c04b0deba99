"""Bounded expert residency: SLRU policy, slot contents, remapping, capacity refusal."""
import pytest
import torch

from orinfer_b200.config import PRESETS, GraphMode, LoadOptions, SchedulerOptions
from orinfer_b200.engine.expert_pager import ExpertCapacityError, ExpertPager
from orinfer_b200.models.weights import ExpertBank, random_model


def _bank(experts, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(-2 ** 31, 2 ** 31 - 1, (experts, k // 128, n, 16), generator=g,
                          dtype=torch.int64).to(torch.int32)
    scale = torch.rand(experts, n, generator=g).half()
    return ExpertBank("q4", experts, n, k, codes, scale, torch.ones(k, dtype=torch.int8))


def _ids(rows):
    return torch.tensor(rows, dtype=torch.int32)


def test_page_in_fills_slots_and_rewrites_ids():
    up, down = _bank(8, 32, 128, 1), _bank(8, 128, 128, 2)
    pager = ExpertPager({"l0": (up, down)}, resident=4, device="cpu")
    su, sd, slots = pager.page_in("l0", _ids([[5, 2], [2, 7], [0, 0]]), rows=2)   # row 2 unused
    assert su.experts == 4 and slots.shape == (2, 2) and slots.dtype == torch.int32
    assert slots[0, 1] == slots[1, 0]                      # expert 2 twice: one slot
    for e, s in ((5, slots[0, 0]), (2, slots[0, 1]), (7, slots[1, 1])):
        assert torch.equal(su.codes[s], up.codes[e]) and torch.equal(su.scale[s], up.scale[e])
        assert torch.equal(sd.codes[s], down.codes[e])
    st = pager.stats
    assert (st.lookups, st.hits, st.misses, st.evictions) == (1, 0, 3, 0)
    assert st.bytes_in == 3 * pager.layers["l0"].bytes_per_expert
    pager.page_in("l0", _ids([[2, 5]]), rows=1)
    assert (st.hits, st.misses) == (2, 3)
    assert pager.route_histogram("l0")[2] == 2 and pager.route_histogram("l0")[0] == 0


def test_segmented_lru_keeps_reused_experts_and_never_evicts_needed_ones():
    up, down = _bank(8, 32, 128, 3), _bank(8, 128, 128, 4)
    pager = ExpertPager({0: (up, down)}, resident=4, device="cpu")
    pager.page_in(0, _ids([[0, 1], [2, 3]]), 2)            # all probationary
    pager.page_in(0, _ids([[0, 1]]), 1)                    # 0 and 1 promoted to protected
    pager.page_in(0, _ids([[4, 5]]), 1)                    # evicts the probationary 2 and 3
    layer = pager.layers[0]
    assert layer.slot_of[0] >= 0 and layer.slot_of[1] >= 0
    assert layer.slot_of[2] == -1 and layer.slot_of[3] == -1
    assert int(layer.remap[2]) == -1 and int(layer.remap[4]) == layer.slot_of[4]
    # a packet that needs four others must evict protected experts too, but none of its own
    _su, _sd, slots = pager.page_in(0, _ids([[6, 7], [4, 5]]), 2)
    assert sorted(slots.flatten().tolist()) == [0, 1, 2, 3]
    assert layer.slot_of[0] == -1 and layer.slot_of[1] == -1
    assert pager.stats.evictions == 4
    for e in (4, 5, 6, 7):
        assert torch.equal(layer.slots[0].codes[layer.slot_of[e]], up.codes[e])


def test_packet_needing_more_experts_than_slots_is_refused():
    pager = ExpertPager({0: (_bank(8, 32, 128, 5), _bank(8, 128, 128, 6))}, 2, "cpu")
    with pytest.raises(ExpertCapacityError):
        pager.page_in(0, _ids([[0, 1], [2, 3]]), 2)
    pager.page_in(0, _ids([[0, 1], [2, 3]]), 1)            # the first row alone fits


def test_engine_bounds_packets_and_turns_graphs_off_when_paging():
    from orinfer_b200.engine.engine import Engine
    w = random_model(PRESETS["tiny-moe"], seed=0)
    eng = Engine(w, load=LoadOptions(resident_experts=4, prompt_lookup=True), kv_pages=8,
                 max_context=256, sched=SchedulerOptions(max_active=8, prefill_chunk=64))
    assert eng.paging and eng.row_cap == 2
    assert eng.sched.max_active == 2 and eng.sched.prefill_chunk == 2
    assert eng.load.cuda_graph is GraphMode.OFF and not eng.spec.enabled
    full = Engine(w, kv_pages=8, max_context=256)
    prompt = [3, 1, 4, 1, 5, 9, 2, 6, 5]
    assert eng.generate([prompt], max_new=4) == full.generate([prompt], max_new=4)
    with pytest.raises(ValueError):
        Engine(w, load=LoadOptions(resident_experts=1), kv_pages=8, max_context=256)


@pytest.mark.gpu
def test_paged_experts_reproduce_the_resident_model_on_device(cuda):
    from orinfer_b200.engine.engine import Engine
    cfg = PRESETS["tiny-moe"]
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (19, 7)]
    mk = lambda resident: Engine(random_model(cfg, seed=0).to(cuda),
                                 load=LoadOptions(resident_experts=resident,
                                                  cuda_graph=GraphMode.OFF),
                                 sched=SchedulerOptions(max_active=2, prefill_chunk=2),
                                 kv_pages=8, max_context=256)
    want = mk(0).generate(prompts, max_new=6)
    eng = mk(4)                                            # 4 of 8 experts, top-2: 2-row packets
    assert eng.runner.pager is not None
    assert not eng.runner.w.layers[0].expert_gate_up.codes.is_cuda
    assert eng.generate(prompts, max_new=6) == want
    st = eng.runner.pager.stats
    assert st.misses > 0 and st.evictions > 0 and st.hits > 0
