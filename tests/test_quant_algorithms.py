"""Offline quantiser algorithms: block LDL rounding, beam-8 search, the Paley x Walsh
rotation, scalar row Q4, lattice-coded embedding rows, precision promotion.  Where the
reference's own CPU implementation is installed (``baseline/_ref``) the formats are compared
with it bit for bit; the rest are property tests."""
import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from orinfer_b200.quant import e8p, embedding_vq, ldlq, rotation, row_q4, search

REF = Path(__file__).resolve().parent.parent / "baseline" / "_ref"


def _ref(module: str):
    if not (REF / "orinfer_build").exists():
        pytest.skip("reference toolchain not installed")
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    import importlib
    return importlib.import_module(module)


# ------------------------------------------------------------------ rotation
def test_paley20_is_a_hadamard_matrix():
    h = rotation.paley20()
    assert set(np.unique(h)) == {-1.0, 1.0}
    assert np.array_equal(h @ h.T, 20 * np.eye(20, dtype=np.float32))
    assert not np.array_equal(h, h.T)                   # forward and inverse differ


@pytest.mark.parametrize("k", [160, 640, 2560])
def test_full_rotation_is_orthogonal_and_inverts(k):
    rng = np.random.default_rng(k)
    signs = e8p.random_signs(k, seed=3)
    x = rng.standard_normal((5, k)).astype(np.float32)
    y = rotation.transform(x, signs, mode="full")
    assert np.allclose((y * y).sum(1), (x * x).sum(1), rtol=1e-4)
    back = rotation.transform(y, signs, mode="full", inverse=True)
    assert np.allclose(back, x, atol=2e-5)
    r = rotation.matrix(signs, mode="full")
    assert np.allclose(r @ r.T, np.eye(k), atol=1e-4)


def test_full_rotation_rejects_other_widths():
    with pytest.raises(ValueError):
        rotation.transform(np.zeros((1, 384), np.float32), np.ones(384, np.int8), mode="full")
    with pytest.raises(ValueError):
        rotation.transform(np.zeros((1, 160), np.float32), np.zeros(160, np.int8), mode="full")


def test_block128_mode_is_the_runtime_rotation():
    signs = e8p.random_signs(256, seed=1)
    x = np.random.default_rng(0).standard_normal((3, 256)).astype(np.float32)
    y = rotation.transform(x, signs, mode="block128")
    assert np.array_equal(y, e8p.hadamard_rotate(x, signs))
    assert np.allclose(rotation.transform(y, signs, mode="block128", inverse=True), x, atol=1e-5)


def test_rotation_matches_the_reference():
    ref = _ref("orinfer_build.quantization.rotation")
    signs = e8p.random_signs(640, seed=9)
    x = np.random.default_rng(1).standard_normal((4, 640)).astype(np.float32)
    assert np.array_equal(ref.hadamard20(), rotation.paley20())
    for inverse in (False, True):
        want = ref.transform(x, signs, mode="full", inverse=inverse)
        got = rotation.transform(x, signs, mode="full", inverse=inverse)
        assert np.allclose(got, want, atol=1e-5)


# ------------------------------------------------------------------ block LDL rounding
def _correlated_covariance(k, rng):
    a = rng.standard_normal((k, k)) * 0.15
    base = np.eye(k) + a @ a.T
    # a few strongly correlated directions, as real activations have
    u = rng.standard_normal((k, 3))
    return base + 4.0 * u @ u.T


def test_factor_reconstructs_and_has_unit_blocks():
    rng = np.random.default_rng(0)
    h = _correlated_covariance(64, rng)
    hn, lower, diag = ldlq.factor(h, block=8, damping=0.01)
    big = np.zeros_like(hn)
    for b in range(8):
        big[b * 8:(b + 1) * 8, b * 8:(b + 1) * 8] = diag[b]
    assert np.allclose(lower @ big @ lower.T, hn, atol=1e-9)
    for b in range(8):
        sl = slice(b * 8, (b + 1) * 8)
        assert np.allclose(lower[sl, sl], np.eye(8), atol=1e-9)
        assert np.allclose(lower[:b * 8, sl], 0)
    with pytest.raises(ValueError):
        ldlq.factor(h[:, :10])
    with pytest.raises(ValueError):
        ldlq.factor(h, damping=0.0)
    with pytest.raises(ValueError):
        ldlq.factor(h + np.triu(np.ones_like(h), 1))


def test_factor_matches_the_reference():
    ref = _ref("orinfer_build.quantization.block_ldlq")
    h = _correlated_covariance(32, np.random.default_rng(2))
    want = ref.factor(h, block_size=8, damping=0.02)
    got = ldlq.factor(h, block=8, damping=0.02)
    for a, b in zip(got, want):
        assert np.allclose(a, b, atol=1e-9)
    w = np.random.default_rng(3).standard_normal((6, 32))
    q = lambda t: np.round(t)
    assert np.allclose(ldlq.round_blocks(w, got[1], q), ref.round_blocks(w, want[1], q, block_size=8))


def test_ldl_rounding_lowers_the_proxy_loss():
    rng = np.random.default_rng(5)
    k = 128
    h = _correlated_covariance(k, rng)
    hn, lower, _ = ldlq.factor(h)
    w = rng.standard_normal((24, k)) * 3.0
    plain = np.round(w)
    fed = ldlq.round_blocks(w, lower, np.round)
    assert ldlq.proxy_loss(w, fed, hn) < 0.8 * ldlq.proxy_loss(w, plain, hn)


def test_e8p_codes_from_ldl_rounding_beat_nearest_rounding_on_the_proxy():
    rng = np.random.default_rng(6)
    k, n = 128, 16
    signs = e8p.random_signs(k, seed=2)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    h = _correlated_covariance(k, rng)                  # covariance of the rotated inputs
    hn, _, _ = ldlq.factor(h)
    wr = e8p.hadamard_rotate(w, signs)
    for fit_ldl, fit_plain in ((ldlq.fit_q2_ldlq, e8p.fit_q2), (ldlq.fit_q4_ldlq, e8p.fit_q4)):
        a = fit_ldl(w, signs, h)
        b = fit_plain(w, signs, refine=0)
        assert a.packed.shape == b.packed.shape if hasattr(a, "packed") else True
        la = ldlq.proxy_loss(wr, a.dequantize_rotated(), hn)
        lb = ldlq.proxy_loss(wr, b.dequantize_rotated(), hn)
        assert la < lb, (fit_ldl.__name__, la, lb)


# ------------------------------------------------------------------ beam search
def test_top8_is_exact_and_sorted():
    rng = np.random.default_rng(7)
    x = torch.from_numpy((rng.standard_normal((64, 8)) * 4).astype(np.float32))
    got = search.nearest_top8(x)
    book = search.codebook("cpu")
    d = ((x[:, None, :] - book[None]) ** 2).sum(-1)
    want_d = torch.sort(d, dim=1).values[:, :8]
    got_d = torch.gather(d, 1, got.long())
    assert torch.allclose(got_d, want_d, atol=1e-4)
    # the nearest of the eight is what the single-code encoder finds
    from orinfer_b200.quant.e8p_torch import encode_nearest_t
    one = encode_nearest_t(x)
    assert torch.allclose(torch.gather(d, 1, one.long()[:, None])[:, 0], got_d[:, 0], atol=1e-4)


def test_beam_refinement_never_loses_and_usually_wins():
    rng = np.random.default_rng(8)
    n, k = 12, 256
    signs = e8p.random_signs(k, seed=4)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    start = e8p.fit_q4(w, signs, refine=0)
    better = search.refine_q4(w, start, iterations=2, beam_passes=2)
    wr = e8p.hadamard_rotate(w, signs)
    e0 = ((wr - start.dequantize_rotated()) ** 2).sum(1)
    e1 = ((wr - better.dequantize_rotated()) ** 2).sum(1)
    assert (e1 <= e0 + 1e-12).all()
    assert e1.sum() < 0.97 * e0.sum()
    with pytest.raises(ValueError):
        search.refine_q4(w, start, iterations=9)


# ------------------------------------------------------------------ row Q4
def test_row_q4_roundtrip_and_error():
    rng = np.random.default_rng(9)
    n, k = 200, 256
    signs = e8p.random_signs(k, seed=5)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    q = row_q4.fit(w, signs)
    assert q.packed.shape == (n, k // 2) and q.scales.shape == (n,)
    ints = q.integers()
    assert set(np.unique(np.abs(ints))) <= set(row_q4.LEVELS)
    wr = e8p.hadamard_rotate(w, signs)
    rel = ((q.dequantize_rotated() - wr) ** 2).sum() / (wr ** 2).sum()
    assert rel < 0.02                                   # 8 magnitude levels on Gaussian rows
    codes, scale = row_q4.expand_to_w8(q)
    assert codes.dtype == np.int8 and np.array_equal(codes, ints)
    assert 4.0 < q.bits_per_weight < 4.3
    with pytest.raises(ValueError):
        row_q4.fit(w, signs.astype(np.int32))


def test_row_q4_matches_the_reference():
    ref = _ref("orinfer_build.quantization.row_q4")
    rng = np.random.default_rng(10)
    signs = e8p.random_signs(128, seed=6)
    w = (rng.standard_normal((130, 128)) * 0.03).astype(np.float32)
    want, got = ref.fit(w, signs), row_q4.fit(w, signs)
    assert np.array_equal(got.packed, want.packed)
    assert np.array_equal(got.scales, want.scales)
    assert np.array_equal(got.integers(), want.integers())


# ------------------------------------------------------------------ embedding rows
def test_embedding_packets_roundtrip():
    rng = np.random.default_rng(11)
    k = 160
    signs = e8p.random_signs(k, seed=7)
    rows = (rng.standard_normal((50, k)) * 0.1).astype(np.float32)
    packets = embedding_vq.encode(rows, signs)
    assert packets.dtype == np.uint8 and packets.shape == (50, 2 + k // 4)
    back = embedding_vq.decode(packets, signs)
    rel = ((back - rows) ** 2).sum() / (rows ** 2).sum()
    assert rel < 0.12                                   # 2 bits per weight
    dec = embedding_vq.Decoder()
    assert np.allclose(dec.decode(packets, signs), back, atol=1e-6)
    assert np.allclose(dec.decode(packets[:3], signs), back[:3], atol=1e-6)   # cached state
    with pytest.raises(ValueError):
        dec.decode(packets[:, :-1], signs)
    with pytest.raises(ValueError):
        embedding_vq.decode(packets, np.zeros(k, np.int8))


def test_embedding_decoder_matches_the_reference():
    ref = _ref("orinfer_build.quantization.embedding_vq")
    k = 160
    signs = e8p.random_signs(k, seed=8)
    rows = (np.random.default_rng(12).standard_normal((9, k)) * 0.1).astype(np.float32)
    packets = embedding_vq.encode(rows, signs)
    table = np.array(e8p.basis())
    want = ref.decode(packets, table, signs)
    assert np.allclose(embedding_vq.decode(packets, signs), want, atol=1e-6)
    assert np.allclose(ref.EmbeddingDecoder().decode(packets, table, signs),
                       embedding_vq.Decoder().decode(packets, signs), atol=1e-6)


# ------------------------------------------------------------------ promotion
def _tiny_source(tmp_path):
    from safetensors.torch import save_file

    hf = dict(architectures=["Qwen3ForCausalLM"], hidden_size=128, num_hidden_layers=3,
              num_attention_heads=2, num_key_value_heads=1, head_dim=64, intermediate_size=256,
              vocab_size=64, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True)
    src = tmp_path / "src"
    src.mkdir()
    (src / "config.json").write_text(json.dumps(hf))
    g = torch.Generator().manual_seed(0)
    rnd = lambda *s: (torch.randn(*s, generator=g) * 0.05).to(torch.bfloat16)
    t = {"model.embed_tokens.weight": rnd(64, 128), "model.norm.weight": torch.ones(128).bfloat16()}
    for i in range(3):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"] = torch.ones(128).bfloat16()
        t[p + "post_attention_layernorm.weight"] = torch.ones(128).bfloat16()
        t[p + "self_attn.q_proj.weight"] = rnd(128, 128)
        t[p + "self_attn.k_proj.weight"] = rnd(64, 128)
        t[p + "self_attn.v_proj.weight"] = rnd(64, 128)
        t[p + "self_attn.o_proj.weight"] = rnd(128, 128)
        t[p + "self_attn.q_norm.weight"] = torch.ones(64).bfloat16()
        t[p + "self_attn.k_norm.weight"] = torch.ones(64).bfloat16()
        t[p + "mlp.gate_proj.weight"] = rnd(256, 128)
        t[p + "mlp.up_proj.weight"] = rnd(256, 128)
        t[p + "mlp.down_proj.weight"] = rnd(128, 256)
    save_file(t, str(src / "model.safetensors"))
    return src


def test_promotion_rewrites_only_the_chosen_layers(tmp_path):
    from orinfer_b200.engine.checkpoint import load_model
    from orinfer_b200.quant import convert, promotion
    src = _tiny_source(tmp_path)
    model = convert.convert(src, tmp_path / "q4")
    rep = promotion.promote(src, model, tmp_path / "promoted", [2])
    assert rep["layers"] == [2] and rep["bytes_after"] > rep["bytes_before"]
    assert set(rep["matrices"]) == {"layers.2.qkv", "layers.2.gate_up", "layers.2.down"}
    assert all(err < 1e-3 for err in rep["matrices"].values())      # W8 is near lossless
    old, new = load_model(model, "cpu"), load_model(tmp_path / "promoted", "cpu")
    assert new.layers[2].qkv.fmt == "w8" and new.layers[2].down.fmt == "w8"
    assert new.layers[2].o.fmt == old.layers[2].o.fmt != "w8"
    for i in (0, 1):
        assert new.layers[i].qkv.fmt == old.layers[i].qkv.fmt
        assert torch.equal(new.layers[i].qkv.codes, old.layers[i].qkv.codes)
    from orinfer_b200.ref.cpu_forward import generate_greedy
    ids = torch.arange(1, 20, dtype=torch.int32)
    assert len(generate_greedy(new, ids, 3)[0]) == 3          # the promoted model still runs
    with pytest.raises(convert.ConvertError):
        promotion.promote(src, model, tmp_path / "bad", [7])


def test_converter_beam_search_lowers_the_weight_error(tmp_path):
    from safetensors import safe_open

    from orinfer_b200.engine.checkpoint import load_model
    from orinfer_b200.quant import convert
    from orinfer_b200.ref.ops_ref import hadamard_rotate
    src = _tiny_source(tmp_path)
    plain = load_model(convert.convert(src, tmp_path / "plain"), "cpu")
    beam = load_model(convert.convert(src, tmp_path / "beam", search="beam8"), "cpu")
    with safe_open(str(src / "model.safetensors"), "pt") as f:
        down = f.get_tensor("model.layers.1.mlp.down_proj.weight").float()

    def err(model):
        lin = model.layers[1].down
        from orinfer_b200.quant.e8p_torch import decode_t
        codes = lin.codes.permute(1, 0, 2).reshape(lin.n, lin.k // 8).to(torch.int64) & 0xFFFFFFFF
        q = (4 * decode_t((codes & 0xFFFF).to(torch.int32)).float()
             + decode_t((codes >> 16).to(torch.int32)).float()).reshape(lin.n, lin.k)
        ref = hadamard_rotate(down, lin.signs)
        return float((ref - q * lin.scale.float()[:, None]).square().sum())
    assert err(beam) < 0.98 * err(plain)
    with pytest.raises(convert.ConvertError):
        convert.convert(src, tmp_path / "x", search="widest")


def test_row_q4_projections_are_stored_as_nibbles_and_run_as_w8(tmp_path):
    from safetensors import safe_open

    from orinfer_b200.engine.checkpoint import load_model
    from orinfer_b200.quant import convert
    from orinfer_b200.ref.cpu_forward import generate_greedy
    src = _tiny_source(tmp_path)
    out = convert.convert(src, tmp_path / "rq4", formats={"proj_format": "rq4"})
    with safe_open(str(out / "model.safetensors"), "pt") as f:
        names = set(f.keys())
        packed = f.get_tensor("layers.0.down.rowq4")
    assert "layers.0.down.rowq4" in names and "layers.0.down.int8" not in names
    assert "layers.0.qkv.packed" in names                      # attention keeps the lattice codes
    assert packed.dtype == torch.uint8 and packed.shape == (128, 128)
    model = load_model(out, "cpu", verify=True)
    down = model.layers[0].down
    assert down.fmt == "w8" and down.codes.dtype == torch.int8 and down.rowq4 is not None
    assert set(down.codes.abs().unique().tolist()) <= set(row_q4.LEVELS)
    assert model.config.proj_format == "w8"
    assert len(generate_greedy(model, torch.arange(1, 20, dtype=torch.int32), 3)[0]) == 3
    with pytest.raises(convert.ConvertError):
        convert.convert(src, tmp_path / "bad", formats={"expert_format": "rq4"})


# ------------------------------------------------------------------ draft calibration
def _rounds(rng, n, width, true_t):
    from orinfer_b200.quant import draft_calibration as dc
    conf = rng.uniform(0.3, 0.99, size=(n, width))
    step = dc.survival(conf, np.asarray(true_t))
    cond = np.concatenate([step[:, :1], step[:, 1:] / step[:, :-1]], axis=1)
    ok = rng.uniform(size=(n, width)) < cond
    accepted = np.where(ok.all(1), width, (~ok).argmax(1)).astype(np.int64)
    return conf, accepted


def test_draft_calibration_recovers_position_temperatures():
    from orinfer_b200.quant import draft_calibration as dc
    rng = np.random.default_rng(13)
    true_t = [0.5, 1.0, 2.0]
    conf, accepted = _rounds(rng, 6000, 3, true_t)
    temps = dc.fit(conf, accepted)
    assert np.all(np.abs(np.log(temps / np.asarray(true_t))) < 0.35), temps
    held_c, held_a = _rounds(rng, 3000, 3, true_t)
    raw = dc.metrics(held_c, held_a, np.ones(3))
    cal = dc.metrics(held_c, held_a, temps)
    assert cal["cumulative_brier"] < raw["cumulative_brier"]
    assert abs(cal["predicted_committed_per_round"] - cal["actual_committed_per_round"]) < 0.05
    assert max(cal["prefix_ece"]) < 0.05
    lab = dc.labels(np.array([0, 2, 3]), 3)
    assert lab.tolist() == [[False] * 3, [True, True, False], [True] * 3]
    with pytest.raises(ValueError):
        dc.survival(np.array([[1.2]]), np.array([1.0]))
    with pytest.raises(ValueError):
        dc.labels(np.array([4]), 3)


def test_draft_calibration_matches_the_reference():
    ref = _ref("orinfer_build.quantization.speculative")
    from orinfer_b200.quant import draft_calibration as dc
    rng = np.random.default_rng(14)
    conf, accepted = _rounds(rng, 400, 4, [0.7, 1.0, 1.5, 1.0])
    temps = dc.fit(conf, accepted)
    assert np.allclose(temps, ref.fit_temperatures(conf, accepted))
    assert np.allclose(dc.survival(conf, temps), ref.calibrated_survival(conf, temps))
    mine, theirs = dc.metrics(conf, accepted, temps), ref.calibration_metrics(conf, accepted, temps)
    assert np.isclose(mine["cumulative_brier"], theirs["cumulative_brier"])
    assert np.allclose(mine["prefix_ece"], theirs["prefix_ece"])


# ------------------------------------------------------------------ precision screening
def test_screening_separates_weight_and_activation_error():
    from orinfer_b200.quant import screening as sc
    rng = np.random.default_rng(15)
    w = rng.standard_normal((48, 64)).astype(np.float32) * 0.05
    mix = rng.standard_normal((64, 64)).astype(np.float32) * 0.3 + np.eye(64, dtype=np.float32)
    train = rng.standard_normal((300, 64)).astype(np.float32) @ mix
    hold = rng.standard_normal((200, 64)).astype(np.float32) @ mix
    r8 = sc.screen_linear(w, train, hold, bits=8)
    r4 = sc.screen_linear(w, train, hold, bits=4)
    assert r8["holdout_nmse"] < 1e-3 < r4["holdout_nmse"] < 0.1
    assert r8["activation_only_nmse"] == 0.0 and r8["weight_only_nmse"] == r8["holdout_nmse"]
    joint = sc.screen_linear(w, train, hold, bits=8, quantize_activation=True)
    assert joint["activation_only_nmse"] > 0 and joint["holdout_nmse"] >= joint["weight_only_nmse"]
    assert r4["clip"] in (0.8, 0.9, 0.95, 1.0)
    st = sc.statistics(train)
    assert st["rows"] == 300 and 0 < st["max_channel_energy_fraction"] < 0.2
    with pytest.raises(ValueError):
        sc.quantize_rows(w, bits=5)


def test_integer_refinement_and_scale_fit_lower_the_output_error():
    from orinfer_b200.quant import screening as sc
    rng = np.random.default_rng(16)
    x = rng.standard_normal((256, 32)).astype(np.float32)
    w = rng.standard_normal((12, 32)).astype(np.float32)
    scales = (np.abs(w).max(1) / 7).astype(np.float32)
    codes = np.clip(np.rint(w / scales[:, None]), -8, 7).astype(np.int8)
    want = x @ w.T
    weights = np.ones_like(want)
    err = lambda q, s: float(np.square(want - (x @ q.astype(np.float32).T) * s).sum())
    better = sc.refine_integer_codes(x, want, codes, scales, weights, steps=8)
    assert better.min() >= -8 and better.max() <= 7
    assert err(better, scales) <= err(codes, scales)
    fitted = sc.fit_output_scales(x @ better.astype(np.float32).T, want, scales)
    assert np.all(np.abs(fitted / scales - 1) <= 0.05 + 1e-6)
    assert err(better, fitted) <= err(better, scales) + 1e-6
    with pytest.raises(ValueError):
        sc.refine_integer_codes(x, want, codes.astype(np.int32) * 3, scales, weights)


def test_screening_matches_the_reference():
    ref = _ref("orinfer_build.quantization.activation")
    from orinfer_b200.quant import screening as sc
    rng = np.random.default_rng(17)
    x = rng.standard_normal((128, 32)).astype(np.float32)
    w = rng.standard_normal((10, 32)).astype(np.float32)
    assert np.array_equal(sc.quantize_rows(w, 4, 0.9), ref.quantize_rows(w, 4, 0.9))
    a, b = sc.screen_linear(w, x[:64], x[64:], bits=4), ref.screen_linear(w, x[:64], x[64:], bits=4)
    assert a == b
    scales = (np.abs(w).max(1) / 7).astype(np.float32)
    codes = np.clip(np.rint(w / scales[:, None]), -8, 7).astype(np.int8)
    want = x @ w.T
    weights = rng.uniform(0.5, 1.5, size=want.shape).astype(np.float32)
    assert np.array_equal(sc.refine_integer_codes(x, want, codes, scales, weights),
                          ref.refine_integer_codes(x, want, codes, scales, weights))
    prod = x @ codes.astype(np.float32).T
    assert np.allclose(sc.fit_output_scales(prod, want, scales, weights),
                       ref.fit_output_scales(prod, want, scales, weights))
