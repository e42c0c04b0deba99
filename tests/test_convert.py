"""Hugging Face Qwen3-style checkpoint -> quantised model directory (resumable)."""
import json

import pytest
import torch
from safetensors.torch import save_file

from orinfer_b200.quant import convert as C
from orinfer_b200.ref.ops_ref import hadamard_rotate

H, HEADS, KV, D, FFN, V, LAYERS = 128, 2, 1, 64, 256, 300, 2


def hf_checkpoint(path, moe=False, tied=True):
    g = torch.Generator().manual_seed(0)
    rnd = lambda *s: (torch.randn(*s, generator=g) * 0.05).to(torch.bfloat16)
    cfg = {"architectures": ["Qwen3MoeForCausalLM" if moe else "Qwen3ForCausalLM"],
           "hidden_size": H, "num_hidden_layers": LAYERS, "num_attention_heads": HEADS,
           "num_key_value_heads": KV, "head_dim": D, "intermediate_size": FFN, "vocab_size": V,
           "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": tied,
           "max_position_embeddings": 4096}
    if moe:
        cfg.update(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128,
                   norm_topk_prob=True)
    t = {"model.embed_tokens.weight": rnd(V, H), "model.norm.weight": torch.ones(H) * 1.5}
    if not tied:
        t["lm_head.weight"] = rnd(V, H)
    for i in range(LAYERS):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"] = torch.ones(H) + 0.1 * i
        t[p + "post_attention_layernorm.weight"] = torch.ones(H)
        t[p + "self_attn.q_proj.weight"] = rnd(HEADS * D, H)
        t[p + "self_attn.k_proj.weight"] = rnd(KV * D, H)
        t[p + "self_attn.v_proj.weight"] = rnd(KV * D, H)
        t[p + "self_attn.o_proj.weight"] = rnd(H, HEADS * D)
        t[p + "self_attn.q_norm.weight"] = torch.ones(D)
        t[p + "self_attn.k_norm.weight"] = torch.ones(D) * 0.5
        if moe:
            t[p + "mlp.gate.weight"] = rnd(4, H)
            for e in range(4):
                t[p + f"mlp.experts.{e}.gate_proj.weight"] = rnd(128, H)
                t[p + f"mlp.experts.{e}.up_proj.weight"] = rnd(128, H)
                t[p + f"mlp.experts.{e}.down_proj.weight"] = rnd(H, 128)
        else:
            t[p + "mlp.gate_proj.weight"] = rnd(FFN, H)
            t[p + "mlp.up_proj.weight"] = rnd(FFN, H)
            t[p + "mlp.down_proj.weight"] = rnd(H, FFN)
    path.mkdir(parents=True, exist_ok=True)
    names = sorted(t)
    save_file({k: t[k].contiguous() for k in names[::2]}, str(path / "model-00001-of-00002.safetensors"))
    save_file({k: t[k].contiguous() for k in names[1::2]}, str(path / "model-00002-of-00002.safetensors"))
    (path / "config.json").write_text(json.dumps(cfg))
    (path / "generation_config.json").write_text(json.dumps({"eos_token_id": [7]}))
    return {k: v.float() for k, v in t.items()}


def rel_error(lin, weight):
    want = hadamard_rotate(weight, lin.signs)
    got = lin.integers().float() * lin.scale.float()[:, None]
    return float((got - want).norm() / want.norm())


def test_dense_conversion_is_faithful_and_resumable(tmp_path):
    from orinfer_b200.config import SchedulerOptions
    from orinfer_b200.engine.checkpoint import load_model, validate_model
    from orinfer_b200.engine.engine import Engine
    src = hf_checkpoint(tmp_path / "hf", tied=False)
    seen = []

    class Stop(Exception):
        pass

    def crash_after_first(i, resumed):
        seen.append((i, resumed))
        if i == 0:
            raise Stop                                    # the job dies after layer 0 is on disk

    with pytest.raises(Stop):
        C.convert(tmp_path / "hf", tmp_path / "out", on_layer=crash_after_first)
    progress = json.loads((tmp_path / "out/.convert/progress.json").read_text())
    assert list(progress["done"]) == ["layer.0"]
    seen.clear()
    out = C.convert(tmp_path / "hf", tmp_path / "out", on_layer=lambda i, r: seen.append((i, r)))
    assert seen == [(0, True), (1, False)]                # layer 0 was kept, not recomputed
    assert not (out / ".convert").exists() and validate_model(out)["ok"]
    assert json.loads((out / "generation_config.json").read_text())["eos_token_id"] == [7]
    w = load_model(out, verify=True)
    cfg = w.config
    assert (cfg.arch, cfg.layers, cfg.hidden, cfg.q_heads, cfg.kv_heads, cfg.head_dim, cfg.ffn,
            cfg.vocab, cfg.tied_embeddings) == ("dense", LAYERS, H, HEADS, KV, D, FFN, V, False)
    l1 = w.layers[1]
    qkv = torch.cat([src[f"model.layers.1.self_attn.{x}_proj.weight"] for x in "qkv"])
    assert l1.qkv.n == (HEADS + 2 * KV) * D and rel_error(l1.qkv, qkv) < 0.12
    gu = torch.cat([src["model.layers.1.mlp.gate_proj.weight"],
                    src["model.layers.1.mlp.up_proj.weight"]])
    assert rel_error(l1.gate_up, gu) < 0.12
    assert rel_error(l1.down, src["model.layers.1.mlp.down_proj.weight"]) < 0.12
    assert torch.allclose(l1.in_norm.float(), torch.full((H,), 1.1), atol=1e-3)
    assert torch.allclose(l1.k_norm.float(), torch.full((D,), 0.5))
    assert torch.allclose(w.final_norm.float(), torch.full((H,), 1.5))
    emb = w.embed_q.float() * w.embed_s.float()[:, None]
    assert float((emb - src["model.embed_tokens.weight"]).norm()
                 / src["model.embed_tokens.weight"].norm()) < 0.02
    assert w.head.n == V and w.head.codes.data_ptr() != w.embed_q.data_ptr()
    eng = Engine(w, sched=SchedulerOptions(max_active=2, prefill_chunk=64), kv_pages=8,
                 max_context=256)
    assert len(eng.generate([[1, 2, 3, 4]], max_new=4)[0]) == 4


def test_moe_conversion_and_refusals(tmp_path):
    from orinfer_b200.engine.checkpoint import load_model
    src = hf_checkpoint(tmp_path / "hf", moe=True)
    w = load_model(C.convert(tmp_path / "hf", tmp_path / "out"))
    cfg = w.config
    assert (cfg.arch, cfg.experts, cfg.top_k, cfg.expert_ffn, cfg.tied_embeddings) == \
        ("moe", 4, 2, 128, True)
    bank = w.layers[0].expert_gate_up
    assert bank.experts == 4 and bank.n == 256 and bank.k == H
    gu2 = torch.cat([src["model.layers.0.mlp.experts.2.gate_proj.weight"],
                     src["model.layers.0.mlp.experts.2.up_proj.weight"]])
    assert rel_error(bank.expert(2), gu2) < 0.12
    assert torch.allclose(w.layers[0].router.float(), src["model.layers.0.mlp.gate.weight"],
                          atol=1e-3)
    bad = json.loads((tmp_path / "hf/config.json").read_text())
    for patch, why in (({"architectures": ["GPT2LMHeadModel"]}, "unsupported architecture"),
                       ({"attention_bias": True}, "bias"),
                       ({"mlp_only_layers": [0]}, "mixed")):
        with pytest.raises(C.ConvertError, match=why):
            C.config_from_hf(dict(bad, **patch))
    (tmp_path / "hf/model-00002-of-00002.safetensors").unlink()
    with pytest.raises(C.ConvertError, match="missing"):
        C.convert(tmp_path / "hf", tmp_path / "out2")


@pytest.mark.parametrize("moe", [False, True], ids=["dense", "moe"])
def test_converted_model_reproduces_the_transformers_implementation(tmp_path, moe):
    """Independent check of the whole decoder semantics (norm convention, q/k head norms,
    rotary pairing, grouped-query attention, SwiGLU, expert routing, head): a random-init
    Qwen3 model of the `transformers` library is saved, converted with 8-bit weights (so that
    quantisation noise stays small) and run through this repository's forward; the logits must
    match the library's."""
    transformers = pytest.importorskip("transformers")
    from orinfer_b200.engine.checkpoint import load_model
    from orinfer_b200.ref.cpu_forward import RefKV, forward_request
    torch.manual_seed(0)
    common = dict(hidden_size=H, num_hidden_layers=2, num_attention_heads=HEADS,
                  num_key_value_heads=KV, head_dim=D, vocab_size=V, rms_norm_eps=1e-6,
                  rope_theta=10000.0, tie_word_embeddings=False, max_position_embeddings=512,
                  attention_bias=False)
    if moe:
        cfg = transformers.Qwen3MoeConfig(intermediate_size=FFN, moe_intermediate_size=128,
                                          num_experts=4, num_experts_per_tok=2, norm_topk_prob=True,
                                          decoder_sparse_step=1, mlp_only_layers=[], **common)
        model = transformers.Qwen3MoeForCausalLM(cfg)
    else:
        cfg = transformers.Qwen3Config(intermediate_size=FFN, **common)
        model = transformers.Qwen3ForCausalLM(cfg)
    model = model.float().eval()
    with torch.no_grad():                         # norms away from 1 so their convention matters
        for name, p in model.named_parameters():
            if name.endswith("norm.weight") or "layernorm" in name:
                p.copy_(1.0 + 0.3 * torch.randn_like(p))
    model.save_pretrained(tmp_path / "hf", safe_serialization=True)
    fmts = {"attn_format": "w8", "proj_format": "w8", "expert_format": "w8"}
    w = load_model(C.convert(tmp_path / "hf", tmp_path / "out", formats=fmts))
    ids = torch.randint(0, V, (24,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = model(ids[None]).logits[0].float()
    got = forward_request(w, ids.int(), 0, RefKV(w.config.layers), quantized=True)
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert float(cos.min()) > 0.99, cos
    agree = (got.argmax(-1) == want.argmax(-1)).float().mean()
    assert float(agree) >= 0.8
    with pytest.raises(C.ConvertError, match="formats"):
        C.convert(tmp_path / "hf", tmp_path / "bad", formats={"attn_format": "fp8"})


def test_hybrid_family_reproduces_the_transformers_implementation(tmp_path):
    """Gated-delta-rule layers (grouped q|k|v|z rows, b|a gates, depthwise convolution, gated
    norm), gated attention with zero-centred head norms and a partially rotated head, routed
    experts with a gated shared expert: converted from a random-init `transformers` model and
    compared with it."""
    transformers = pytest.importorskip("transformers")
    if not hasattr(transformers, "Qwen3NextForCausalLM"):
        pytest.skip("this transformers has no Qwen3-Next")
    from orinfer_b200.engine.checkpoint import load_model
    from orinfer_b200.ref.cpu_forward import RefKV, forward_request
    torch.manual_seed(0)
    cfg = transformers.Qwen3NextConfig(
        hidden_size=H, num_hidden_layers=4, num_attention_heads=HEADS, num_key_value_heads=KV,
        head_dim=D, vocab_size=V, intermediate_size=FFN, moe_intermediate_size=128,
        shared_expert_intermediate_size=128, num_experts=4, num_experts_per_tok=2,
        linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=64,
        linear_value_head_dim=64, partial_rotary_factor=0.25, rope_theta=10000.0,
        tie_word_embeddings=False, max_position_embeddings=512)
    model = transformers.Qwen3NextForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith("norm.weight") or "layernorm" in name:
                p.copy_((0.0 if "linear_attn.norm" not in name else 1.0) + 0.3 * torch.randn_like(p))
            if name.endswith("A_log") or name.endswith("dt_bias"):
                p.copy_(0.5 * torch.randn_like(p))
    model.save_pretrained(tmp_path / "hf", safe_serialization=True)
    fmts = {"attn_format": "w8", "proj_format": "w8", "expert_format": "w8"}
    w = load_model(C.convert(tmp_path / "hf", tmp_path / "out", formats=fmts))
    c = w.config
    assert (c.arch, c.gdn_period, c.rotary_dim, c.zero_centered_norm, c.gated_attention,
            c.shared_expert_ffn) == ("hybrid", 4, 16, True, True, 128)
    assert [lw.kind for lw in w.layers] == ["gdn", "gdn", "gdn", "attn"]
    ids = torch.randint(0, V, (24,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = model(ids[None]).logits[0].float()
    got = forward_request(w, ids.int(), 0, RefKV(c.layers), quantized=True)
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert float(cos.min()) > 0.99, cos
    # the serving engine (paged KV, chunked prefill) walks the same arithmetic as the
    # single-request forward, partial rotary included
    from orinfer_b200.config import SchedulerOptions
    from orinfer_b200.engine.engine import Engine
    from orinfer_b200.ref.cpu_forward import generate_greedy
    eng = Engine(w, sched=SchedulerOptions(max_active=2, prefill_chunk=16), kv_pages=8,
                 max_context=256)
    assert eng.generate([ids.tolist()], max_new=5)[0] == generate_greedy(w, ids.int(), 5)[0]
    perm = C.rotary_permutation(8, 4)
    assert perm.tolist() == [0, 1, 4, 5, 2, 3, 6, 7] and C.rotary_permutation(8, 0).tolist() == list(range(8))


def test_draft_head_of_a_hybrid_checkpoint_is_converted(tmp_path, monkeypatch):
    """``mtp.*`` tensors become the draft head: a full-attention layer shaped like the model's
    own (gated attention, routed experts, shared expert), the [H, 2H] projection and the three
    norms.  The draft layer here is a copy of the model's last layer, so its converted form
    must equal that layer's; the engine then speculates with the head and keeps the text."""
    transformers = pytest.importorskip("transformers")
    if not hasattr(transformers, "Qwen3NextForCausalLM"):
        pytest.skip("this transformers has no Qwen3-Next")
    from safetensors.torch import load_file
    from orinfer_b200.config import LoadOptions, SchedulerOptions
    from orinfer_b200.engine.checkpoint import load_model
    from orinfer_b200.engine.engine import Engine
    torch.manual_seed(0)
    cfg = transformers.Qwen3NextConfig(
        hidden_size=H, num_hidden_layers=4, num_attention_heads=HEADS, num_key_value_heads=KV,
        head_dim=D, vocab_size=V, intermediate_size=FFN, moe_intermediate_size=128,
        shared_expert_intermediate_size=128, num_experts=4, num_experts_per_tok=2,
        linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=64,
        linear_value_head_dim=64, partial_rotary_factor=0.25, rope_theta=10000.0,
        tie_word_embeddings=False, max_position_embeddings=512)
    transformers.Qwen3NextForCausalLM(cfg).float().eval().save_pretrained(
        tmp_path / "hf", safe_serialization=True)
    have = {}
    for f in (tmp_path / "hf").glob("*.safetensors"):
        have.update(load_file(str(f)))
    g = torch.Generator().manual_seed(3)
    extra = {k.replace("model.layers.3.", "mtp.layers.0."): v.clone()
             for k, v in have.items() if k.startswith("model.layers.3.")}
    extra["mtp.fc.weight"] = torch.randn(H, 2 * H, generator=g) * 0.05
    extra["mtp.pre_fc_norm_embedding.weight"] = 0.2 * torch.randn(H, generator=g)
    extra["mtp.pre_fc_norm_hidden.weight"] = 0.2 * torch.randn(H, generator=g)
    extra["mtp.norm.weight"] = 0.2 * torch.randn(H, generator=g)
    save_file({k: v.contiguous() for k, v in extra.items()}, str(tmp_path / "hf/mtp.safetensors"))
    fmts = {"attn_format": "w8", "proj_format": "w8", "expert_format": "w8"}
    w = load_model(C.convert(tmp_path / "hf", tmp_path / "out", formats=fmts))
    c, m = w.config, w.mtp
    assert c.mtp_layers == 1 and c.draft_layer == "model" and m is not None
    last = w.layers[3]
    assert torch.equal(m.layer.qkv.codes, last.qkv.codes) and m.layer.qkv.n == last.qkv.n
    assert torch.equal(m.layer.expert_down.codes, last.expert_down.codes)
    assert torch.equal(m.layer.router, last.router)
    assert torch.equal(m.layer.shared_gate_up.codes, last.shared_gate_up.codes)
    assert m.fc.signs is None and m.fc.n == H and m.fc.k == 2 * H
    got = m.fc.integers().float() * m.fc.scale.float()[:, None]
    assert float((got - extra["mtp.fc.weight"]).norm() / extra["mtp.fc.weight"].norm()) < 0.02
    assert torch.allclose(m.norm_e.float(), extra["mtp.pre_fc_norm_embedding.weight"], atol=1e-3)
    assert torch.allclose(m.final_norm.float(), extra["mtp.norm.weight"], atol=1e-3)
    # speculation with the converted head never changes the text
    monkeypatch.setenv("ORINFER_SINGLE_MTP_POLICY", "fixed2")
    ids = torch.randint(0, V, (20,), generator=torch.Generator().manual_seed(1)).tolist()
    mk = lambda drafts: Engine(w, load=LoadOptions(mtp_drafts=drafts, prefix_cache_bytes=0),
                               sched=SchedulerOptions(max_active=2, prefill_chunk=16),
                               kv_pages=8, max_context=256)
    plain = mk(0).generate([ids], max_new=8)[0]
    eng = mk(2)
    assert eng.runner_has_mtp() and eng.spec.enabled
    assert eng.generate([ids], max_new=8)[0] == plain
    assert eng.spec.statistics()["proposed_tokens"] > 0


def test_llama_style_checkpoints_convert_too(tmp_path):
    """The same decoder without per-head q / k norms (Llama, Mistral)."""
    transformers = pytest.importorskip("transformers")
    from orinfer_b200.engine.checkpoint import load_model
    from orinfer_b200.ref.cpu_forward import RefKV, forward_request
    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(hidden_size=H, num_hidden_layers=2, num_attention_heads=HEADS,
                                   num_key_value_heads=KV, head_dim=D, vocab_size=V,
                                   intermediate_size=FFN, rms_norm_eps=1e-6, rope_theta=10000.0,
                                   tie_word_embeddings=True, max_position_embeddings=512,
                                   attention_bias=False, mlp_bias=False)
    model = transformers.LlamaForCausalLM(cfg).float().eval()
    model.save_pretrained(tmp_path / "hf", safe_serialization=True)
    w = load_model(C.convert(tmp_path / "hf", tmp_path / "out",
                             formats={"attn_format": "w8", "proj_format": "w8"}))
    assert not w.config.qk_norm and w.config.tied_embeddings and w.layers[0].q_norm is None
    ids = torch.randint(0, V, (24,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = model(ids[None]).logits[0].float()
    got = forward_request(w, ids.int(), 0, RefKV(2), quantized=True)
    assert float(torch.nn.functional.cosine_similarity(got, want, dim=-1).min()) > 0.99
    with pytest.raises(C.ConvertError, match="sliding-window"):
        C.config_from_hf({"architectures": ["MistralForCausalLM"], "sliding_window": 4096,
                          "num_attention_heads": 2})


def test_quality_probes_pair_the_library_with_the_converted_model(tmp_path, capsys):
    """The whole comparison as a user runs it: baseline probes from transformers, candidate
    probes from the converted model through the CLI, paired analysis."""
    transformers = pytest.importorskip("transformers")
    from orinfer_b200 import cli
    torch.manual_seed(0)
    cfg = transformers.Qwen3Config(hidden_size=H, num_hidden_layers=2, num_attention_heads=HEADS,
                                   num_key_value_heads=KV, head_dim=D, vocab_size=V,
                                   intermediate_size=FFN, tie_word_embeddings=False,
                                   max_position_embeddings=512)
    transformers.Qwen3ForCausalLM(cfg).save_pretrained(tmp_path / "hf", safe_serialization=True)
    C.convert(tmp_path / "hf", tmp_path / "out", formats={"attn_format": "w8", "proj_format": "w8"})
    toks = ",".join(str((7 * i + 3) % V) for i in range(20))
    base, cand = str(tmp_path / "b.jsonl"), str(tmp_path / "c.jsonl")
    assert cli.main(["bench", "hf-reference", str(tmp_path / "hf"), "--tokens", toks,
                     "--jsonl", base]) == 0
    assert cli.main(["score-model", str(tmp_path / "out"), "--device", "cpu", "--tokens", toks,
                     "--jsonl", cand, "--query-from", base]) == 0
    capsys.readouterr()
    assert cli.main(["bench", "quality", "--baseline", base, "--candidate", cand]) == 0
    rep = json.loads(capsys.readouterr().out)["aggregate"]
    assert rep["positions"] == 19 and rep["mean_abs_probability_error"] < 0.002
    assert rep["top3_overlap"] > 0.6 and abs(rep["delta_target_nll"]) < 0.05
