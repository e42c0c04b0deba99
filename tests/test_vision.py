"""Image inputs: geometry, packing order, span binding, MRoPE, feature overlay in the engine."""
import io

import numpy as np
import pytest
import torch

from orinfer_b200.config import PRESETS, LoadOptions, SchedulerOptions
from orinfer_b200.engine.engine import Engine
from orinfer_b200.engine.request import MediaSpan
from orinfer_b200.models import vision as V
from orinfer_b200.models.weights import random_model
from orinfer_b200.ref import ops_ref as R

SPEC = V.VisionSpec(hidden=256, image_token_id=900, vision_start_token_id=901,
                    vision_end_token_id=902, width=64, depth=1, heads=2, min_pixels=32 * 32)


def image(gh, gw, seed=0):
    rng = np.random.default_rng(seed)
    return V.ImageInput(gh, gw, rng.integers(0, 256, (gh * 16, gw * 16, 3), dtype=np.uint8))


def test_grid_features_and_span_binding():
    assert SPEC.grid_features(4, 6) == 6
    with pytest.raises(V.VisionError, match="merger"):
        SPEC.grid_features(3, 4)
    with pytest.raises(V.VisionError, match="capacity"):
        SPEC.grid_features(256, 256)
    a, b = image(2, 2), image(2, 4, 1)
    toks = [1, 901, 900, 902, 5, 901, 900, 900, 902, 7]
    assert V.image_spans(SPEC, toks, [a, b]) == [(2, 3), (6, 8)]
    for bad, why in (([1, 2], "missing"), ([900, 900], "unbound"), ([1, 900, 5, 900, 900], "unbound")):
        with pytest.raises(V.VisionError, match=why):
            V.image_spans(SPEC, bad, [a])
    with pytest.raises(V.VisionError, match="invalid image token span|outside"):
        V.image_spans(SPEC, [900, 3], [b])
    with pytest.raises(V.VisionError, match="pixel data"):
        V.feature_count(SPEC, V.ImageInput(2, 2, np.zeros((16, 32, 3), np.uint8)))


def test_patch_packing_order_matches_the_loop_statement():
    img = image(4, 2, 3)
    got = V.pack_pixels(SPEC, img)
    p, m, t = 16, 2, 2
    want = []
    for br in range(img.grid_height // m):
        for bc in range(img.grid_width // m):
            for inner in range(m * m):
                for ch in range(3):
                    for _ in range(t):
                        for xy in range(p * p):
                            y = (br * m + inner // m) * p + xy // p
                            x = (bc * m + inner % m) * p + xy % p
                            want.append(img.rgb[y, x, ch] / 127.5 - 1.0)
    assert got.shape == (8, SPEC.patch_values)
    assert torch.allclose(got.reshape(-1), torch.tensor(want, dtype=torch.float32), atol=1e-6)
    coords = V.patch_coordinates(SPEC, 4, 2)
    assert coords[:5].tolist() == [[0, 0], [0, 1], [1, 0], [1, 1], [2, 0]]


def test_resize_geometry_and_decoding():
    assert V.smart_resize(100, 200, 32, 32 * 32, 1 << 20) == (96, 192)
    h, w = V.smart_resize(4000, 3000, 32, 32 * 32, 1 << 20)
    assert h % 32 == 0 and w % 32 == 0 and h * w <= 1 << 20 and abs(h / w - 4 / 3) < 0.05
    h, w = V.smart_resize(10, 20, 32, 256 * 256, 1 << 20)
    assert h * w >= 256 * 256
    with pytest.raises(V.VisionError):
        V.smart_resize(1, 1000, 32, 1, 1 << 20)
    from PIL import Image
    buf = io.BytesIO()
    Image.new("RGBA", (70, 50), (255, 0, 0, 0)).save(buf, format="PNG")
    img = V.load_image(buf.getvalue(), SPEC)
    assert img.rgb.shape == (img.grid_height * 16, img.grid_width * 16, 3)
    assert img.grid_height % 2 == 0 and img.rgb.min() == 255      # transparent over white
    with pytest.raises(V.VisionError, match="decode"):
        V.load_image(b"not an image", SPEC)


def test_mrope_positions_and_tables():
    toks = [1, 2, 901] + [900] * 6 + [902, 3, 4]
    pos, delta = V.mrope_positions(SPEC, toks, [(3, 9)], [(4, 6)])       # merged grid 2 x 3
    assert pos[0].tolist() == [0, 1, 2, 3, 3, 3, 3, 3, 3, 6, 7, 8]
    assert pos[1].tolist() == [0, 1, 2, 3, 3, 3, 4, 4, 4, 6, 7, 8]
    assert pos[2].tolist() == [0, 1, 2, 3, 4, 5, 3, 4, 5, 6, 7, 8]
    assert delta == 9 - 12
    plain, d0 = V.mrope_positions(SPEC, [5, 6, 7], [], [])
    assert plain.tolist() == [[0, 1, 2]] * 3 and d0 == 0
    assert V.mrope_sections(32) == (11, 11, 10)
    p = torch.tensor([0, 5, 17], dtype=torch.int32)
    cos, sin = V.mrope_tables(torch.stack([p, p, p]), 64, 1e6)
    c0, s0 = R.rope_tables(p, 64, 1e6)
    assert torch.equal(cos, c0) and torch.equal(sin, s0)
    cos, _ = V.mrope_tables(torch.tensor([[7], [1], [2]], dtype=torch.int32), 64, 1e6)
    ct, _ = R.rope_tables(torch.tensor([7, 1, 2]), 64, 1e6)
    assert cos[0, 0] == ct[0, 0] and cos[0, 1] == ct[1, 1] and cos[0, 2] == ct[2, 2]
    assert cos[0, 31] == ct[0, 31]                                      # beyond the w section


def test_encoder_and_feature_cache():
    enc = V.VisionEncoder(SPEC, seed=1)
    a, b = image(2, 4), image(2, 4, 9)
    fa = enc.encode(a)
    assert fa.shape == (2, 256) and torch.isfinite(fa).all()
    assert torch.equal(fa, V.VisionEncoder(SPEC, seed=1).encode(a))
    assert not torch.allclose(fa, enc.encode(b))
    cache = V.FeatureCache(budget_bytes=fa.numel() * 4 + 8)
    assert cache.get(a, enc) is cache.get(a, enc) and (cache.hits, cache.misses) == (1, 1)
    cache.get(b, enc)                                                   # evicts a
    cache.get(a, enc)
    assert cache.misses == 3 and cache.bytes <= cache.budget


@pytest.fixture(scope="module")
def weights():
    return random_model(PRESETS["tiny"], seed=0)


def engine(weights, chunk=16):
    return Engine(weights, sched=SchedulerOptions(max_active=4, prefill_chunk=chunk), kv_pages=24,
                  max_context=512, load=LoadOptions(prefix_cache_bytes=4 << 20))


def test_overlay_of_token_embeddings_equals_those_tokens(weights):
    """Placeholders overlaid with the embeddings of other tokens, at ordinary positions, must
    generate exactly what the prompt with those tokens generates, across chunk boundaries."""
    real = [3, 7, 11] + list(range(40, 60)) + [5, 9, 2]
    masked = real[:3] + [900] * 20 + real[23:]
    feats = R.embed_w8(torch.tensor(real[3:23]), weights.embed_q, weights.embed_s)
    want = engine(weights).generate([real], max_new=6)[0]
    eng = engine(weights, chunk=8)
    pos = np.tile(np.arange(len(masked), dtype=np.int32), (3, 1))
    req = eng.submit(masked, max_new=6, media=[MediaSpan(3, 23, feats, 77)], rope_positions=pos)
    while eng.has_work():
        eng.step()
    assert req.generated == want
    other = engine(weights).generate([masked], max_new=6)[0]
    assert other != want                                   # the overlay is what made them equal


def test_rope_delta_shifts_decode_positions(weights):
    prompt = [3, 7, 11, 900, 900, 900, 900, 5]
    feats = R.embed_w8(torch.tensor([40, 41, 42, 43]), weights.embed_q, weights.embed_s)
    pos, delta = V.mrope_positions(SPEC, prompt, [(3, 7)], [(4, 4)])
    assert delta == -2
    eng = engine(weights)
    seen = []
    inner = eng.runner.forward_hidden

    def spy(p):
        seen.append((p.row_pos[:p.rows].tolist(), p.mrope[:, :p.rows].tolist()))
        return inner(p)

    eng.runner.forward_hidden = spy
    req = eng.submit(prompt, max_new=3, media=[MediaSpan(3, 7, feats, 1)],
                     rope_positions=pos, rope_delta=delta)
    while eng.has_work():
        eng.step()
    assert len(req.generated) == 3
    assert seen[0] == (list(range(8)), pos.tolist())              # prefill: KV index vs rotary
    assert seen[1] == ([8], [[6], [6], [6]]) and seen[2] == ([9], [[7], [7], [7]])
    with pytest.raises(ValueError, match="media span"):
        engine(weights).submit(prompt, media=[MediaSpan(3, 7, feats[:2], 1)])


def test_prefix_cache_separates_images(weights):
    eng = engine(weights, chunk=128)
    prompt = [900] * 200 + [4, 5, 6]
    fa = torch.randn(200, 256, generator=torch.Generator().manual_seed(1)).half()
    fb = torch.randn(200, 256, generator=torch.Generator().manual_seed(2)).half()

    def run(feats, digest):
        req = eng.submit(prompt, max_new=3, media=[MediaSpan(0, 200, feats, digest)])
        while eng.has_work():
            eng.step()
        return req

    first = run(fa, 11)
    again = run(fa, 11)
    other = run(fb, 22)
    assert first.cached_tokens == 0 and again.cached_tokens == 128 and other.cached_tokens == 0
    assert again.generated == first.generated


# ------------------------------------------------------------------ HTTP surface
def _png(color, size=(64, 64)):
    import base64
    from PIL import Image
    buf = io.BytesIO()
    Image.new("RGB", size, color).save(buf, format="PNG")
    return "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()


@pytest.fixture(scope="module")
def client(weights):
    from fastapi.testclient import TestClient
    from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec
    from orinfer_b200.api.images import frontend_for
    from orinfer_b200.api.server import Service, create_app
    codec = ChatCodec(ByteTokenizer(1024), context=512, model_name="tiny")
    codec.images = frontend_for(codec.tokenizer, 256, cache_mib=1, min_pixels=32 * 32,
                                width=64, depth=1, heads=2)
    svc = Service(lambda: engine(weights, chunk=64), codec, "tiny")
    svc.start()
    with TestClient(create_app(svc)) as c:
        yield c
    svc.stop(1000)


def _ask(client, parts, **extra):
    body = dict({"messages": [{"role": "user", "content": parts}], "max_tokens": 4,
                 "temperature": 0, "ignore_eos": True}, **extra)
    return client.post("/v1/chat/completions", json=body)


def test_chat_with_images_over_http(client):
    red = {"type": "image_url", "image_url": {"url": _png((255, 0, 0))}, "uuid": "red-1"}
    blue = {"type": "image_url", "image_url": {"url": _png((0, 0, 255), (128, 64)),
                                               "detail": "low"}}
    text = {"type": "text", "text": "compare"}
    r = _ask(client, [text, red, blue])
    assert r.status_code == 200, r.text
    n_text = _ask(client, [text]).json()["usage"]["prompt_tokens"]
    # 64x64 -> 4x4 patches -> 4 features; 128x64 -> 8 features; +2 delimiters each
    assert r.json()["usage"]["prompt_tokens"] == n_text + (4 + 2) + (8 + 2)
    again = _ask(client, [text, {"type": "image_url", "image_url": None, "uuid": "red-1"}, blue])
    assert again.status_code == 200
    assert again.json()["choices"][0]["message"] == r.json()["choices"][0]["message"]
    miss = _ask(client, [text, {"type": "image_url", "image_url": None, "uuid": "nope"}])
    assert miss.status_code == 400 and miss.json()["error"]["code"] == "image_not_cached"
    bad = _ask(client, [{"type": "image_url", "image_url": {"url": "data:image/png;base64,AAAA"}}])
    assert bad.status_code == 400 and "decode" in bad.json()["error"]["message"]
    many = _ask(client, [red, red], image_processing={"max_images": 1})
    assert many.status_code == 400
    big = _ask(client, [red], image_processing={"max_tokens": 2})
    assert big.status_code == 400 and "max_tokens" in big.json()["error"]["message"]
    # a placeholder spelled out in user text is ordinary characters, not a control token
    forged = _ask(client, [{"type": "text", "text": "<|image_pad|>"}])
    assert forged.status_code == 200
    assert forged.json()["usage"]["prompt_tokens"] == n_text - len("compare") + len("<|image_pad|>")
    assert "orinfer_image_inputs_total" in client.get("/metrics").text


def test_model_without_vision_refuses_images(weights):
    from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec, RequestError
    codec = ChatCodec(ByteTokenizer(1024), context=512)
    with pytest.raises(RequestError, match="no image"):
        codec.prepare({"messages": [{"role": "user", "content": [
            {"type": "image_url", "image_url": {"url": _png((1, 2, 3))}}]}]})


def test_ollama_images_become_image_parts(client):
    import base64
    from PIL import Image
    from orinfer_b200.api.chat_codec import RequestError
    from orinfer_b200.api.ollama import translate
    buf = io.BytesIO()
    Image.new("RGB", (64, 64), (0, 255, 0)).save(buf, format="JPEG")
    b64 = base64.b64encode(buf.getvalue()).decode()
    out = translate({"model": "m", "messages": [{"role": "user", "content": "what?",
                                                 "images": [b64]}]}, generate=False)
    parts = out["messages"][0]["content"]
    assert parts[0] == {"type": "text", "text": "what?"}
    assert parts[1]["image_url"]["url"].startswith("data:image/jpeg;base64,")
    assert "images" not in out["messages"][0]
    gen = translate({"model": "m", "prompt": "see", "images": [_png((1, 2, 3)).split(",")[1]]},
                    generate=True)
    assert gen["messages"][-1]["content"][1]["image_url"]["url"].startswith("data:image/png")
    for bad in (["!!!"], [base64.b64encode(b"GIF89a" + b"\0" * 20).decode()], "x"):
        with pytest.raises(RequestError):
            translate({"model": "m", "prompt": "p", "images": bad}, generate=True)
    r = client.post("/api/chat", json={"model": "tiny", "stream": False, "options": {"num_predict": 3},
                                       "messages": [{"role": "user", "content": "what?",
                                                     "images": [b64]}]})
    assert r.status_code == 200 and r.json()["prompt_eval_count"] > 6


def test_max_pixels_refuses_or_resizes(client):
    big = {"type": "image_url", "image_url": {"url": _png((9, 9, 9), (256, 128))}}
    refused = _ask(client, [big], image_processing={"max_pixels": 64 * 64})
    assert refused.status_code == 400 and "auto_resize" in refused.json()["error"]["message"]
    resized = _ask(client, [big], image_processing={"max_pixels": 64 * 64, "auto_resize": True})
    assert resized.status_code == 200
    n_text = _ask(client, [{"type": "text", "text": ""}]).json()["usage"]["prompt_tokens"]
    assert resized.json()["usage"]["prompt_tokens"] - n_text <= 4 + 2      # at most 64x64 -> 4 features
    per_image = _ask(client, [big], image_processing={"max_tokens_per_image": 2})
    assert per_image.status_code == 200
    assert per_image.json()["usage"]["prompt_tokens"] - n_text <= 2 + 2
