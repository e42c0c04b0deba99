"""Device / memory / family contracts."""
import json

import pytest

from orinfer_b200 import contracts as C


def test_memory_ranges_are_checked_at_construction():
    r = C.MemoryRange(256, 1024, 4096)
    assert r.end == 1280 and r.aligned(256) and not r.aligned(512)
    s = r.slice(24, 100)
    assert (s.offset, s.length, s.capacity) == (280, 100, 4096)
    assert r.rows(64, 2, 3) == C.MemoryRange(256 + 128, 192, 4096)
    for bad in ((-1, 4, 8), (4, 8, 8), (0, 0, 1 << 62)):
        with pytest.raises(C.ContractError):
            C.MemoryRange(*bad)
    with pytest.raises(C.ContractError):
        r.slice(1000, 25)
    with pytest.raises(C.ContractError):
        r.rows(0, 0, 1)
    a, b, c = C.MemoryRange(0, 16, 64), C.MemoryRange(16, 16, 64), C.MemoryRange(8, 16, 64)
    assert not a.overlaps(b) and a.overlaps(c) and c.overlaps(b)
    assert not a.overlaps(C.MemoryRange(4, 0, 64))
    assert C.disjoint([b, a]) and not C.disjoint([a, b, c])


def test_owners_targets_and_dtypes():
    a, b = C.DeviceOwner.new(0), C.DeviceOwner.new(0)
    a.require(a)
    with pytest.raises(C.ContractError, match="different device or session"):
        a.require(b)                                   # same ordinal, another session
    assert C.parse_target("sm_100a") == "sm_100a"
    for other in ("sm_87", "sm_90a", "ascend910b"):
        with pytest.raises(C.ContractError, match="sm_100a only"):
            C.parse_target(other)
    assert C.Dtype.F16.bytes == 2 and C.Dtype("u64").bytes == 8


def test_gdn_policy_and_encoder_specs():
    C.GdnPolicy().validate_supported()
    with pytest.raises(C.ContractError):
        C.GdnPolicy(prefill=C.GdnPrefill.CHUNKED).validate_supported()
    with pytest.raises(C.ContractError):
        C.GdnPolicy(decode=C.GdnDecode(8)).validate_supported()
    with pytest.raises(C.ContractError):
        C.GdnDecode(65)
    e = C.EmbeddingSpec(256)
    assert e.output_dimensions(None) == 256 and e.output_dimensions(64) == 64
    with pytest.raises(C.ContractError):
        e.output_dimensions(257)
    assert C.RerankSpec(3, 5).score([0, 0, 0, 2.5, 0, -1.0]) == 3.5
    assert C.encoder_rows([3, 1, 4], 8) == [(0, 3), (3, 1), (4, 4)]
    with pytest.raises(C.ContractError, match="capacity"):
        C.encoder_rows([5, 4], 8)
    with pytest.raises(C.ContractError, match="empty"):
        C.encoder_rows([2, 0], 8)


def test_registry_guards_the_loader(tmp_path):
    from orinfer_b200.config import PRESETS
    from orinfer_b200.engine.checkpoint import CheckpointError, load_model, save_model
    from orinfer_b200.models.weights import random_model
    assert C.architectures() == ["orinfer_b200.dense", "orinfer_b200.hybrid", "orinfer_b200.moe"]
    with pytest.raises(C.ContractError, match="compute policy"):
        C.create("orinfer_b200.dense", "fp16_fast", PRESETS["tiny"])
    with pytest.raises(C.ContractError, match="unknown architecture"):
        C.create("qwen9", C.COMPUTE_POLICY, PRESETS["tiny"])
    with pytest.raises(C.ContractError, match="twice"):
        C.register("orinfer_b200.dense", lambda cfg: cfg)
    save_model(random_model(PRESETS["tiny"], seed=0), tmp_path)
    assert load_model(tmp_path).config.arch == "dense"
    path = tmp_path / "cache" / "model.json"
    desc = json.loads(path.read_text())
    for key, value, why in (("architecture", "orinfer_b200.moe", "describes `dense`"),
                            ("target", "sm_87", "sm_100a"),
                            ("compute_policy", "fast", "compute policy")):
        path.write_text(json.dumps(dict(desc, **{key: value})))
        with pytest.raises(CheckpointError, match=why):
            load_model(tmp_path)


def test_mtp_spec_contract():
    from orinfer_b200.config import PRESETS
    from orinfer_b200.contracts import ContractError, MtpSpec
    spec = MtpSpec.for_config(PRESETS["tiny"], 3, 32, 4128)
    assert spec.verification_widths == (2, 3, 4) and spec.max_drafts == 3
    assert spec.batch_draft_profiles == (1, 2, 4, 8, 16, 32) and not spec.commit_always
    assert spec.draft_capacity(3) == 4 and spec.draft_capacity(33) == 32
    assert spec.width_allowed(4, 100) and not spec.width_allowed(5, 1)
    assert not spec.width_allowed(4, 2000)                      # 8000 rows exceed the packet bound
    assert MtpSpec.for_config(PRESETS["tiny-hybrid"], 2, 4, 256).commit_always
    off = MtpSpec.for_config(PRESETS["tiny"], 0, 8, 256)
    assert off.verification_widths == () and off.max_drafts == 0
    with pytest.raises(ContractError):
        MtpSpec(verification_widths=(3, 2))
    with pytest.raises(ContractError):
        MtpSpec(batch_draft_profiles=(4, 4))
    with pytest.raises(ContractError):
        MtpSpec(max_drafts=2, verification_widths=(2, 3, 4))
    with pytest.raises(ContractError):
        MtpSpec(batch_verification_tokens=2)
