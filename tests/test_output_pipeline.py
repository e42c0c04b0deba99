"""Output pipeline on its own thread: ordering, isolation between streams, late stop strings."""
import json
import threading

import pytest
from fastapi.testclient import TestClient

from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec
from orinfer_b200.api.server import Service, create_app
from orinfer_b200.config import PRESETS, SchedulerOptions
from orinfer_b200.engine.engine import Engine
from orinfer_b200.models.weights import random_model


@pytest.fixture(scope="module", params=["1", "0"], ids=["async", "inline"])
def client(request):
    import os
    old = os.environ.get("ORINFER_ASYNC_OUTPUT")
    os.environ["ORINFER_ASYNC_OUTPUT"] = request.param
    weights = random_model(PRESETS["tiny"], seed=0)
    svc = Service(lambda: Engine(weights, sched=SchedulerOptions(max_active=8, prefill_chunk=64),
                                 kv_pages=40, max_context=512),
                  ChatCodec(ByteTokenizer(1024), context=512, model_name="tiny"), "tiny")
    svc.start()
    assert (svc.worker.pipeline is not None) == (request.param == "1")
    with TestClient(create_app(svc)) as c:
        yield c
    svc.stop(1000)
    if old is None:
        os.environ.pop("ORINFER_ASYNC_OUTPUT", None)
    else:
        os.environ["ORINFER_ASYNC_OUTPUT"] = old


def forced(char, **extra):
    return dict({"messages": [{"role": "user", "content": "go"}], "temperature": 0,
                 "logit_bias": {str(ord(char)): 100}, "ignore_eos": True}, **extra)


def test_streams_do_not_mix_and_keep_their_order(client):
    results = {}

    def one(ch):
        body = forced(ch, max_tokens=24, stream=True, stream_options={"include_usage": True})
        with client.stream("POST", "/v1/chat/completions", json=body) as r:
            lines = [json.loads(l[6:]) for l in r.iter_lines()
                     if l.startswith("data: ") and l != "data: [DONE]"]
        results[ch] = lines

    threads = [threading.Thread(target=one, args=(ch,)) for ch in "abcdefgh"]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for ch, lines in results.items():
        text = "".join(c["choices"][0]["delta"].get("content", "") for c in lines if c["choices"])
        assert text == ch * 24, ch
        assert lines[0]["choices"][0]["delta"] == {"role": "assistant", "content": ""}
        assert lines[-1]["usage"]["completion_tokens"] == 24 and lines[-1]["choices"] == []
        assert lines[-2]["choices"][0]["finish_reason"] == "length"


def test_stop_string_ends_generation_early(client):
    r = client.post("/v1/chat/completions", json=forced("z", max_tokens=200, stop=["zzzz"])).json()
    assert r["choices"][0]["finish_reason"] == "stop"
    assert r["choices"][0]["message"]["content"] == ""          # the match itself is withheld
    # the engine stops within a few steps of the match, not at the token limit
    assert 4 <= r["usage"]["completion_tokens"] <= 60
    again = client.post("/v1/chat/completions", json=forced("y", max_tokens=6)).json()
    assert again["choices"][0]["message"]["content"] == "yyyyyy"
    assert again["choices"][0]["finish_reason"] == "length"
    lp = client.post("/v1/chat/completions",
                     json=forced("q", max_tokens=5, logprobs=True, top_logprobs=2)).json()
    entries = lp["choices"][0]["logprobs"]["content"]
    assert [e["token"] for e in entries] == ["q"] * 5 and len(entries[0]["top_logprobs"]) == 2


def test_health_reports_the_pipeline_and_caches(client):
    h = client.get("/health").json()
    assert h["output_pipeline"] in ("thread", "inline")
    assert set(h["tokenization_cache"]) == {"entries", "bytes", "hits", "misses"}
    assert h["tokenization_cache"]["misses"] >= 1


def test_every_request_histogram_is_fed(client):
    import re
    client.post("/v1/chat/completions", json=forced("m", max_tokens=3))
    text = client.get("/metrics").text
    for name in ("queue", "prefill", "decode", "finalize", "time_to_first_token", "latency"):
        m = re.search(rf"orinfer_request_{name}_seconds_count (\d+)", text)
        assert m and int(m.group(1)) >= 1, name
    assert "orinfer_request_prefix_store_seconds_count" in text
    assert "orinfer_admission_seconds_total" in text
    for gauge in ("kv_pages_free", "speculation_acceptance_rate", "graph_replays_total"):
        assert re.search(rf"orinfer_{gauge} [0-9.]+", text), gauge
