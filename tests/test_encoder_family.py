"""Bidirectional encoder family (embedding models) on the CPU runner and over HTTP."""
import pytest
import torch

from orinfer_b200.config import PRESETS, ModelConfig, SchedulerOptions
from orinfer_b200.engine.engine import Engine
from orinfer_b200.models.weights import random_model


_WEIGHTS = {}


def engine(cfg):
    # attention direction, pooling and RoPE base do not change the weights: build them once
    # per depth and swap the configuration
    import dataclasses
    if cfg.layers not in _WEIGHTS:
        _WEIGHTS[cfg.layers] = random_model(ModelConfig(layers=cfg.layers), seed=3)
    weights = dataclasses.replace(_WEIGHTS[cfg.layers], config=cfg)
    return Engine(weights, sched=SchedulerOptions(max_active=2, prefill_chunk=64),
                  kv_pages=16, max_context=256)


def test_every_row_sees_the_whole_input():
    first = dict(bidirectional=True, pooling="first")
    a = [5, 9, 14, 3, 8, 21, 2]
    b = a[:-1] + [77]                                       # only the last token differs
    enc = engine(ModelConfig(name="e", **first))
    ea, _ = enc.encode(a)
    eb, _ = enc.encode(b)
    assert not torch.allclose(ea, eb, atol=1e-4)            # row 0 saw the change at the end
    causal = engine(ModelConfig(name="c", pooling="first"))
    ca, _ = causal.encode(a)
    cb, _ = causal.encode(b)
    assert torch.allclose(ca, cb, atol=1e-6)                # a causal row 0 cannot
    mean = engine(PRESETS["tiny-embed"]).encode(a)[0]
    assert mean.shape == (256,) and abs(float(mean.norm()) - 1.0) < 1e-5
    assert torch.equal(mean, engine(PRESETS["tiny-embed"]).encode(a)[0])    # deterministic
    # slots and pages are returned: many passes on a small pool
    for _ in range(20):
        enc.encode(a)
    with pytest.raises(ValueError, match="does not generate"):
        enc.submit(a, 4)
    with pytest.raises(ValueError, match="bidirectionally"):
        ModelConfig(arch="hybrid", bidirectional=True, gdn_period=4, gdn_k_heads=2, gdn_v_heads=4)
    with pytest.raises(ValueError, match="pooling"):
        ModelConfig(pooling="max")


def test_single_layer_matches_full_attention_statement():
    """One layer, one token pair: with bidirectional attention both rows attend to both keys,
    so swapping the two tokens changes the mean-pooled output only through RoPE (with a huge
    theta just the first frequency pair still turns); causally the first row sees one key in
    one order and two in the other, a much larger change."""
    cfg = ModelConfig(name="sym", layers=1, bidirectional=True, rope_theta=1e30)
    enc = engine(cfg)
    xy, _ = enc.encode([11, 42])
    yx, _ = enc.encode([42, 11])
    causal = engine(ModelConfig(name="asym", layers=1, rope_theta=1e30))
    cxy, _ = causal.encode([11, 42])
    cyx, _ = causal.encode([42, 11])
    assert float((xy - yx).norm()) < 0.5 * float((cxy - cyx).norm())


def test_embeddings_route_of_an_encoder_model():
    from fastapi.testclient import TestClient
    from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec
    from orinfer_b200.api.server import Service, create_app
    svc = Service(lambda: engine(PRESETS["tiny-embed"]),
                  ChatCodec(ByteTokenizer(1024), context=256, model_name="tiny-embed"), "tiny-embed")
    svc.start()
    with TestClient(create_app(svc)) as c:
        assert c.get("/health").json()["status"] == "ready"
        r = c.post("/v1/embeddings", json={"input": ["alpha beta", "gamma"], "dimensions": 64})
        assert r.status_code == 200 and len(r.json()["data"][1]["embedding"]) == 64
        chat = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}]})
        assert chat.status_code == 400 and "does not generate" in chat.json()["error"]["message"]
    svc.stop(1000)
