"""Plan validation before allocation: dimensions, sharding, descriptor and memory."""
import json

import pytest

from orinfer_b200.config import PRESETS, LoadOptions, SchedulerOptions
from orinfer_b200.engine.plan import PlanError, validate_plan, weight_shapes

L, S = LoadOptions(), SchedulerOptions()


def test_plans_of_the_presets_fit_one_b200():
    for name, low, high in (("qwen3.5-4b-class", 3.5e9, 4.5e9), ("27b-class", 24e9, 29e9),
                            ("35b-a3b-class", 28e9, 37e9), ("80b-a3b-class", 70e9, 90e9)):
        plan = validate_plan(PRESETS[name], L, S, max_context=8704, device_bytes=180 << 30)
        assert low < plan.weight_parameters < high, (name, plan.weight_parameters)
        assert plan.total_bytes == (plan.weight_bytes + plan.kv_bytes + plan.workspace_bytes
                                    + plan.table_bytes)
        sharded = validate_plan(PRESETS[name], L, S, max_context=8704, world=8,
                                device_bytes=180 << 30)
        assert sharded.weight_bytes < plan.weight_bytes / 3
        assert sharded.kv_bytes_per_page < plan.kv_bytes_per_page


def test_memory_that_does_not_fit_is_refused_with_numbers():
    with pytest.raises(PlanError) as err:
        validate_plan(PRESETS["80b-a3b-class"], L, S, max_context=8704, device_bytes=16 << 30)
    assert "GiB" in str(err.value) and "weights" in str(err.value)
    validate_plan(PRESETS["80b-a3b-class"], L, S, max_context=8704, world=8,
                  device_bytes=16 << 30)                      # split over 8 ranks it fits


def test_dimensions_and_sharding_rules():
    tiny = PRESETS["tiny"]
    with pytest.raises(PlanError, match="query heads"):
        validate_plan(tiny, L, S, max_context=256, world=8)
    with pytest.raises(PlanError, match="max_context"):
        validate_plan(tiny, L, S, max_context=tiny.max_context + 1)
    with pytest.raises(PlanError, match="KV pages"):
        validate_plan(tiny, L, S, max_context=512, kv_pages=3)
    with pytest.raises(PlanError, match="max_rows"):
        validate_plan(tiny, L, S, max_context=256, max_rows=8)
    validate_plan(PRESETS["qwen3.5-4b-class"], L, S, max_context=512, world=8)   # uneven FFN blocks


def test_descriptor_must_list_what_the_geometry_needs(tmp_path):
    import torch

    from orinfer_b200.engine.checkpoint import read_descriptor, save_model
    from orinfer_b200.models.weights import random_model
    cfg = PRESETS["tiny"]
    save_model(random_model(cfg, seed=0), tmp_path)
    desc = read_descriptor(tmp_path)
    validate_plan(cfg, L, S, max_context=256, descriptor=desc, exhaustive=True)
    stems = weight_shapes(cfg)
    assert "layers.0.qkv" in stems and stems["layers.0.qkv"][1] == cfg.hidden
    broken = json.loads(json.dumps(desc))
    del broken["tensors"]["layers.1.down.scale"]
    with pytest.raises(PlanError, match="layers.1.down"):
        validate_plan(cfg, L, S, max_context=256, descriptor=broken)
    broken = json.loads(json.dumps(desc))
    broken["tensors"]["final_norm"] = "not-a-hash"
    validate_plan(cfg, L, S, max_context=256, descriptor=broken)          # only when exhaustive
    with pytest.raises(PlanError, match="malformed hash"):
        validate_plan(cfg, L, S, max_context=256, descriptor=broken, exhaustive=True)


def test_plan_model_cli_reports_the_plan_and_refusals(capsys):
    from orinfer_b200 import cli
    assert cli.main(["plan-model", "--preset", "27b-class", "--tp", "8"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["ok"] and out["memory_plan"]["world"] == 8
    assert cli.main(["plan-model", "--preset", "80b-a3b-class", "--device-gib", "8"]) == 2
    out = json.loads(capsys.readouterr().out)
    assert not out["ok"] and "GiB" in out["error"]


def test_the_draft_head_is_part_of_the_plan(tmp_path):
    import dataclasses

    from orinfer_b200.engine.checkpoint import read_descriptor, save_model
    from orinfer_b200.models.weights import random_model
    for preset, kind in (("tiny", "dense"), ("tiny-moe", "model")):
        base = PRESETS[preset]
        cfg = dataclasses.replace(base, mtp_layers=1, draft_layer=kind)
        stems = weight_shapes(cfg)
        assert stems["mtp.fc"] == (cfg.hidden, 2 * cfg.hidden, "w8")
        assert ("mtp.layer.expert_down" in stems) == (kind == "model")
        with_head = validate_plan(cfg, L, S, max_context=256)
        without = validate_plan(base, L, S, max_context=256)
        assert with_head.weight_bytes > without.weight_bytes
        assert with_head.kv_bytes_per_page > without.kv_bytes_per_page       # its own KV layer
        out = tmp_path / preset
        save_model(random_model(cfg, seed=0), out)
        desc = read_descriptor(out)
        validate_plan(cfg, L, S, max_context=256, descriptor=desc, exhaustive=True)
        broken = json.loads(json.dumps(desc))
        del broken["tensors"]["mtp.fc.scale"]
        with pytest.raises(PlanError, match="mtp.fc"):
            validate_plan(cfg, L, S, max_context=256, descriptor=broken)
