"""Launch-variant tables: parsing, validation, lookup, and that the kernel library honours them."""
import ctypes
import json

import pytest
import torch

from orinfer_b200.config import PRESETS
from orinfer_b200.tuning import gemm_tuner, tables
from orinfer_b200.tuning.tables import GemmVariant


def _table(entries):
    return json.dumps({"schema": 1, "device": "test", "gemm": entries})


def test_table_round_trip_lookup_and_merge():
    vs = [GemmVariant("q4", 19456, 2560, 9, 16, 1, 64, 1, 20.0, 25.0),
          GemmVariant("q4", 19456, 2560, 17, 32, 1, 64, 1, 21.0, 25.0),
          GemmVariant("q4", 19456, 2560, 33, 64, 1, 128, 2, 22.0, 25.0),
          GemmVariant("w8", 2560, 9728, 257, 512, 2, 128, 4)]
    merged = tables.merge_ranges(vs)
    assert [(v.m_lo, v.m_hi) for v in merged if v.fmt == "q4"] == [(9, 32), (33, 64)]
    back = tables.parse(tables.dump(merged, "test"))
    assert tables.lookup(back, "q4", 20, 19456, 2560).nb == 64
    assert tables.lookup(back, "q4", 40, 19456, 2560).splits == 2
    assert tables.lookup(back, "q4", 65, 19456, 2560) is None
    assert tables.lookup(back, "w8", 300, 2560, 9728).mt == 2


@pytest.mark.parametrize("entry, why", [
    (dict(fmt="q4", n=256, k=256, m_lo=9, m_hi=16, mt=3, nb=128, splits=1), "mt"),
    (dict(fmt="q4", n=256, k=256, m_lo=9, m_hi=16, mt=1, nb=96, splits=1), "nb"),
    (dict(fmt="q4", n=256, k=256, m_lo=9, m_hi=16, mt=1, nb=64, splits=2), "split-K needs"),
    (dict(fmt="q4", n=256, k=256, m_lo=9, m_hi=16, mt=1, nb=128, splits=3), "splits"),
    (dict(fmt="q9", n=256, k=256, m_lo=9, m_hi=16, mt=1, nb=128, splits=1), "format"),
    (dict(fmt="q4", n=256, k=256, m_lo=20, m_hi=16, mt=1, nb=128, splits=1), "row range"),
    (dict(fmt="q4", n=151936, k=2560, m_lo=9, m_hi=8192, mt=4, nb=128, splits=2), "workspace"),
])
def test_invalid_entries_are_refused(entry, why):
    with pytest.raises(ValueError, match=why):
        tables.parse(_table([entry]))


def test_overlapping_ranges_and_wrong_schema_are_refused():
    e = dict(fmt="q4", n=256, k=256, m_lo=9, m_hi=32, mt=1, nb=128, splits=1)
    with pytest.raises(ValueError, match="overlapping"):
        tables.parse(_table([e, dict(e, m_lo=32, m_hi=64)]))
    with pytest.raises(ValueError, match="schema"):
        tables.parse(json.dumps({"schema": 7, "gemm": []}))


def test_tuner_shapes_candidates_and_buckets():
    shapes = gemm_tuner.model_shapes(PRESETS["qwen3.5-4b-class"])
    assert ("q4", 2 * 9728, 2560) in shapes and ("q4", 2560, 9728) in shapes
    assert ("q4", 32 * 128 + 2 * 8 * 128, 2560) in shapes
    assert gemm_tuner.bucket_ranges(64) == [(9, 16), (17, 32), (33, 64)]
    assert gemm_tuner.bucket_ranges(0, rows=[512, 100]) == [(9, 100), (101, 512)]
    cs = gemm_tuner.candidates("q4", 64, 2560, 2560)
    assert all(c.mt == 1 for c in cs) and any(c.splits == 8 for c in cs)
    assert all(c.nb == 128 for c in cs if c.splits > 1)
    assert {c.mt for c in gemm_tuner.candidates("q4", 512, 2560, 2560)} == {1, 2, 4}


def test_kernel_library_plan_follows_the_table():
    """Host-only: the plan the GEMM launcher derives for a shape changes with the table."""
    from orinfer_b200.ops import native
    lib = native.lib()
    plan = lambda m, n, k: (lambda o: (lib.orinfer_qgemm_plan(1, m, n, k, 0, o), list(o))[1])(
        (ctypes.c_int * 4)())
    lib.orinfer_qgemm_clear_variants()
    try:
        base = plan(512, 19456, 2560)
        assert base[:3] == [4, 128, 1]
        assert plan(512, 2560, 9728)[2] > 1                      # narrow projection: split-K
        n = tables.apply([GemmVariant("q4", 19456, 2560, 257, 512, 2, 64, 1)], lib)
        assert n == 1
        assert plan(512, 19456, 2560) == [2, 64, 1, 0]
        assert plan(256, 19456, 2560) == plan(256, 19456, 2560) != [2, 64, 1, 0]
        assert lib.orinfer_qgemm_launches_fmt(1, 512, 19456, 2560, 0, 0) == 1
        assert lib.orinfer_qgemm_set_variant(1, 9, 16, 256, 256, 3, 128, 1) == -1
    finally:
        lib.orinfer_qgemm_clear_variants()


@pytest.mark.gpu
def test_variants_do_not_change_the_gemm_result(cuda):
    from orinfer_b200.ops import functional as F
    from orinfer_b200.ops import native
    from orinfer_b200.bench.kernel_probe import weights
    lib = native.lib()
    n, k = 2560, 2560
    w = weights("q4", n, k, cuda, 1)[0]
    sw = (torch.rand(n, device=cuda) * 0.01).half()
    try:
        for m in (40, 300, 700):
            a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=cuda)
            sa = torch.rand(m, device=cuda) * 0.01
            lib.orinfer_qgemm_clear_variants()
            want = F.qgemm(a, sa, w, sw, "q4", n, path=2).clone()
            for c in gemm_tuner.candidates("q4", m, n, k):
                tables.apply([c], lib)
                assert torch.equal(F.qgemm(a, sa, w, sw, "q4", n, path=2), want), c
        torch.cuda.synchronize()
        assert native.read_status() == 0
    finally:
        lib.orinfer_qgemm_clear_variants()


def test_launch_plan_is_valid_over_the_whole_row_domain():
    """Offline validation of the launch geometry, the way the reference validates its dynamic
    row contracts for every live row count (crates/orinfer-model-sdk/src/operators/dynamic.rs:
    75-146): for each projection shape of the benchmark models, at every tensor-parallel
    degree and with the packaged table loaded, every row count 1..4096 yields a plan the
    launcher has a kernel instance for and whose split-K partials fit the workspace."""
    from orinfer_b200.ops import native
    lib = native.lib()
    out = (ctypes.c_int * 4)()
    formats = tables.FORMATS
    workspace = 96 << 20                                   # split-K partials buffer
    checked = 0
    for table in (False, True):
        lib.orinfer_qgemm_clear_variants()
        if table:
            assert tables.load_default(lib) > 0
        for preset, degrees in (("qwen3.5-4b-class", (1, 2, 4, 8)), ("27b-class", (1, 8))):
            for tp in degrees:
                for fmt, n, k in gemm_tuner.model_shapes(PRESETS[preset], tp):
                    for m in list(range(1, 513)) + list(range(513, 4097, 7)) + [4096]:
                        lib.orinfer_qgemm_plan(formats[fmt], m, n, k, 0, out)
                        mt, nb, splits, tail = list(out)
                        assert mt in (1, 2, 4) and nb in (32, 64, 128), (fmt, m, n, k, list(out))
                        assert 1 <= splits <= 8 and splits <= max(k // 128, 1)
                        assert 0 <= tail <= 8 and (tail == 0 or (splits == 1 and nb == 128))
                        assert splits == 1 or splits * m * n * 4 <= workspace
                        checked += 1
    lib.orinfer_qgemm_clear_variants()
    assert checked > 40_000


def test_attention_split_table_overrides_the_heuristic():
    from orinfer_b200.ops import functional as F
    from orinfer_b200.tuning.tables import AttentionSplit
    saved = list(tables.ATTENTION)
    try:
        tables.set_attention([])
        base = F.attention_splits(512, 1, 8)
        assert base == 8                                         # 512 keys: at most 8 splits of 64
        assert F.attention_splits(100, 1, 8) == 1                # one page: never split
        doc = {"schema": 1, "gemm": [], "attention": [
            {"rows_lo": 1, "rows_hi": 2, "ctx_lo": 129, "ctx_hi": 1024, "kvh": 8, "splits": 4,
             "us": 10.0, "us_default": 12.0}]}
        import json
        entries = tables.parse_attention(json.dumps(doc))
        assert tables.set_attention(entries) == 1
        assert F.attention_splits(512, 1, 8) == 4                # tuned
        assert F.attention_splits(512, 2, 8) == 4
        assert F.attention_splits(512, 3, 8) == F.attention_splits(512, 3, 8) != 0   # outside: heuristic
        assert F.attention_splits(512, 1, 4) == min(148 * 3 // 4, 8)               # other head count
        assert F.attention_splits(200, 1, 8) == 4                # 200 keys: ceil(200/64) = 4 caps it
        assert tables.dump_attention(entries)[0]["splits"] == 4
        doc["attention"].append(dict(doc["attention"][0], rows_lo=2, rows_hi=4))
        with pytest.raises(ValueError, match="overlap"):
            tables.parse_attention(json.dumps(doc))
        doc["attention"] = [dict(doc["attention"][0], splits=64)]
        with pytest.raises(ValueError, match="splits"):
            tables.parse_attention(json.dumps(doc))
        assert AttentionSplit(1, 1, 129, 512, 8, 8).problems() == []
    finally:
        tables.set_attention(saved)


def test_attention_tuner_cells_and_choice():
    from orinfer_b200.tuning import attention_tuner as at
    assert at.candidates(512) == [1, 2, 3, 4, 6, 8]
    assert at.candidates(130) == [1, 2]                        # 130 keys over 3 splits: 44 each
    assert 32 in at.candidates(8192)
    cells = at.buckets([1, 8], [512])
    assert cells == [((1, 1), (129, 512)), ((5, 8), (129, 512))]
    assert len(at.buckets([], [])) == len(at.ROW_BUCKETS) * len(at.CTX_BUCKETS)
    # a candidate must beat the heuristic by more than the margin
    assert at.choose({4: 10.0, 8: 9.9}, 4, 0.03) == (4, 10.0, 10.0)
    assert at.choose({4: 10.0, 8: 9.0}, 4, 0.03) == (8, 9.0, 10.0)
    assert at.main(["--rows", "1", "--ctx", "512"]) == 2         # no GPU here: refuses to guess
