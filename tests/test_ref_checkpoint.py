"""A tiny checkpoint written in the reference's published layout with the reference's own
CPU codec (the installed offline toolchain) loads here: every fused projection decodes to
the same integers and scales, and the model generates."""
import json
import os
import sys

import numpy as np
import pytest
import torch

REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


@pytest.fixture(scope="module")
def ref():
    if not os.path.isdir(os.path.join(REF, "orinfer_build")):
        pytest.skip("the reference's offline toolchain is not installed under baseline/_ref")
    sys.path.insert(0, REF)
    try:
        from orinfer_build.quantization import e8p, e8p_q4
    except Exception as e:                                   # noqa: BLE001
        pytest.skip(f"reference codec not importable: {e}")
    finally:
        sys.path.remove(REF)
    return e8p, e8p_q4


def _write(tmp_path, ref):
    from safetensors.numpy import save_file
    e8p, e8p_q4 = ref
    rng = np.random.default_rng(0)
    H, QH, KVH, D, F, V, LAYERS = 128, 2, 1, 64, 256, 256, 2
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": H,
           "num_hidden_layers": LAYERS, "num_attention_heads": QH, "num_key_value_heads": KVH,
           "head_dim": D, "intermediate_size": F, "vocab_size": V, "rms_norm_eps": 1e-6,
           "rope_theta": 1e6, "tie_word_embeddings": False, "max_position_embeddings": 2048,
           "quantization_config": {"quant_method": "orinfer_e8p_q4_int8", "version": 1,
                                   "coefficients": [4, 1], "rotation": "signed-block128",
                                   "scale": "fp16-output-row",
                                   "layout": "u32-low-coarse-high-residual"}}
    signs = {k: np.random.default_rng(20261002 + k).choice(np.array([-1, 1], np.int8), k)
             for k in (H, F, QH * D)}
    shards = {"model-00001-of-00002.safetensors": {}, "model-00002-of-00002.safetensors": {}}
    layouts = {k: {} for k in shards}
    fitted = {}

    def put(shard, name, weight, kind):
        t, lay = shards[shard], layouts[shard]
        if kind == "q4":
            fit = e8p_q4.fit(weight.astype(np.float32), signs[weight.shape[1]], iterations=1)
            fitted[name] = fit
            t[name + ".packed"] = fit.packed
            t[name + ".scale"] = fit.scales
            lay["orin.layout." + name + ".packed"] = "e8p-q4-row-u32"
        elif kind == "w8":
            amax = np.abs(weight).max(1)
            scale = np.maximum(amax / 127.0, 2.0 ** -24).astype(np.float16)
            q = np.clip(np.rint(weight / scale.astype(np.float32)[:, None]), -127, 127)
            fitted[name] = (q.astype(np.int8), scale)
            t[name + ".int8"] = q.astype(np.int8)
            t[name + ".scale"] = scale
            lay["orin.layout." + name + ".int8"] = "native_contiguous"
        else:
            t[name] = weight.astype(np.float16)

    w = lambda n, k: (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    for i in range(LAYERS):
        shard = list(shards)[i % 2]
        p = f"model.layers.{i}."
        put(shard, p + "input_layernorm.weight", np.ones(H, np.float32), "raw")
        put(shard, p + "post_attention_layernorm.weight", np.ones(H, np.float32), "raw")
        put(shard, p + "self_attn.q_proj.weight", w(QH * D, H), "q4")
        put(shard, p + "self_attn.k_proj.weight", w(KVH * D, H), "q4")
        put(shard, p + "self_attn.v_proj.weight", w(KVH * D, H), "q4")
        put(shard, p + "self_attn.q_norm.weight", np.ones(D, np.float32), "raw")
        put(shard, p + "self_attn.k_norm.weight", np.ones(D, np.float32), "raw")
        put(shard, p + "self_attn.o_proj.weight", w(H, QH * D), "w8")
        put(shard, p + "mlp.gate_proj.weight", w(F, H), "q4")
        put(shard, p + "mlp.up_proj.weight", w(F, H), "q4")
        put(shard, p + "mlp.down_proj.weight", w(H, F), "q4")
    first = list(shards)[0]
    put(first, "model.embed_tokens.weight", w(V, H), "q4")
    put(first, "model.norm.weight", np.ones(H, np.float32), "raw")
    put(first, "lm_head.weight", w(V, H), "q4")
    weight_map = {}
    for name, tensors in shards.items():
        save_file(tensors, str(tmp_path / name), metadata=layouts[name])
        weight_map.update({k: name for k in tensors})
    common = {f"orinfer.rotation.k{k}.signs": s for k, s in signs.items()}
    common["orinfer.e8p_q4.basis"] = np.array(e8p.basis())
    save_file(common, str(tmp_path / "quantization.safetensors"))
    weight_map.update({k: "quantization.safetensors" for k in common})
    (tmp_path / "model.safetensors.index.json").write_text(
        json.dumps({"metadata": {}, "weight_map": weight_map}))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    return fitted, signs


def test_reference_layout_loads_bit_for_bit(tmp_path, ref):
    from orinfer_b200.engine.checkpoint import load_model
    from orinfer_b200.engine.ref_checkpoint import is_reference_layout
    fitted, signs = _write(tmp_path, ref)
    assert is_reference_layout(tmp_path)
    m = load_model(tmp_path, "cpu")
    cfg = m.config
    assert (cfg.layers, cfg.hidden, cfg.q_heads, cfg.kv_heads, cfg.ffn) == (2, 128, 2, 1, 256)
    for i, lw in enumerate(m.layers):
        p = f"model.layers.{i}."
        want = np.concatenate([fitted[p + f"self_attn.{x}_proj.weight"].integers()
                               for x in "qkv"])
        assert lw.qkv.fmt == "q4" and np.array_equal(lw.qkv.integers().numpy(), want)
        want_s = np.concatenate([fitted[p + f"self_attn.{x}_proj.weight"].scales for x in "qkv"])
        assert np.array_equal(lw.qkv.scale.numpy(), want_s)
        assert torch.equal(lw.qkv.signs, torch.from_numpy(signs[128]))
        gu = np.concatenate([fitted[p + "mlp.gate_proj.weight"].integers(),
                             fitted[p + "mlp.up_proj.weight"].integers()])
        assert np.array_equal(lw.gate_up.integers().numpy(), gu)
        assert np.array_equal(lw.down.integers().numpy(),
                              fitted[p + "mlp.down_proj.weight"].integers())
        q8, s8 = fitted[p + "self_attn.o_proj.weight"]
        assert lw.o.fmt == "w8" and lw.o.signs is None
        assert np.array_equal(lw.o.codes.numpy(), q8) and np.array_equal(lw.o.scale.numpy(), s8)
    assert m.head.fmt == "q4"
    assert np.array_equal(m.head.integers().numpy(), fitted["lm_head.weight"].integers())
    # the lattice-coded embedding comes back as W8 rows close to the dequantised table
    emb = fitted["model.embed_tokens.weight"]
    from orinfer_b200.ref.ops_ref import hadamard_rotate
    dense = hadamard_rotate(torch.from_numpy(emb.dequantize()), torch.from_numpy(signs[128]))
    back = m.embed_q.float() * m.embed_s.float()[:, None]
    assert float((back - dense).abs().max()) <= float(dense.abs().max()) / 100


def test_reference_layout_model_generates(tmp_path, ref):
    from orinfer_b200.engine.checkpoint import load_model
    from orinfer_b200.engine.engine import Engine
    _write(tmp_path, ref)
    eng = Engine(load_model(tmp_path, "cpu"), kv_pages=16, max_context=256)
    out = eng.generate([[3, 5, 7, 11, 13]], max_new=4)
    assert len(out[0]) == 4 and all(0 <= t < 256 for t in out[0])
