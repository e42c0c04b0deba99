"""HTTP surface on the tiny CPU model: OpenAI chat (JSON + SSE), errors, logprobs,
JSON-schema constraint, Ollama routes, health and metrics."""
import json

import pytest
from fastapi.testclient import TestClient

from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec
from orinfer_b200.api.server import Service, create_app
from orinfer_b200.config import PRESETS, LoadOptions, SchedulerOptions
from orinfer_b200.engine.engine import Engine
from orinfer_b200.models.weights import random_model


@pytest.fixture(scope="module")
def client():
    weights = random_model(PRESETS["tiny"], seed=0)

    def factory():
        return Engine(weights, sched=SchedulerOptions(max_active=4, prefill_chunk=64),
                      kv_pages=24, max_context=512)

    codec = ChatCodec(ByteTokenizer(1024), context=512, model_name="tiny")
    svc = Service(factory, codec, "tiny")
    svc.start()
    with TestClient(create_app(svc)) as c:
        yield c
    svc.stop(1000)


MSG = [{"role": "user", "content": "hello"}]


def test_health_models_metrics(client):
    h = client.get("/health").json()
    assert h["status"] == "ready" and h["continuous_batching"] and "scheduler" in h
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny"
    assert client.get("/v1/models/tiny").json()["object"] == "model"
    gone = client.get("/v1/models/other")
    assert gone.status_code == 404 and gone.json()["error"]["code"] == "model_not_found"
    client.post("/v1/chat/completions", json={"messages": MSG, "max_tokens": 3,
                                              "ignore_eos": True})
    r = client.get("/metrics")
    assert "orinfer_request_latency_seconds_bucket" in r.text
    assert "x-request-id" in r.headers
    values = dict(line.split(" ", 1) for line in r.text.splitlines()
                  if line and not line.startswith("#") and "{" not in line)
    for name in ("orinfer_generated_tokens_total", "orinfer_prompt_tokens_total",
                 "orinfer_cached_prompt_tokens_total", "orinfer_compute_seconds_total",
                 "orinfer_admission_seconds_total", "orinfer_batch_plan_seconds_total",
                 "orinfer_sampling_request_failures_total", "orinfer_program_reclaims_total",
                 "orinfer_prefix_cache_evictions_total", "orinfer_prefix_cache_host_evictions_total",
                 "orinfer_prefix_restore_seconds_total", "orinfer_prefix_cache_device_entries",
                 "orinfer_prefix_cache_device_bytes", "orinfer_prefix_cache_host_entries",
                 "orinfer_prefix_cache_host_bytes", "orinfer_requests_running",
                 "orinfer_requests_waiting"):
        assert name in values, name
    assert float(values["orinfer_generated_tokens_total"]) >= 3
    assert float(values["orinfer_generated_tokens_total"]) == \
        float(values["orinfer_completion_tokens_total"])


def test_chat_completion_json_and_determinism(client):
    body = {"messages": MSG, "max_tokens": 6, "temperature": 0, "ignore_eos": True}
    a = client.post("/v1/chat/completions", json=body).json()
    b = client.post("/v1/chat/completions", json=body).json()
    assert a["object"] == "chat.completion" and a["choices"][0]["finish_reason"] == "length"
    assert a["usage"]["completion_tokens"] == 6 and a["usage"]["prompt_tokens"] > 5
    assert a["choices"][0]["message"]["content"] == b["choices"][0]["message"]["content"]
    seeded = dict(body, temperature=1.0, seed=7)
    s1 = client.post("/v1/chat/completions", json=seeded).json()
    s2 = client.post("/v1/chat/completions", json=seeded).json()
    assert s1["choices"][0]["message"] == s2["choices"][0]["message"]


def test_streaming_chunk_sequence_and_usage(client):
    body = {"messages": MSG, "max_tokens": 5, "temperature": 0, "stream": True, "ignore_eos": True,
            "stream_options": {"include_usage": True}}
    with client.stream("POST", "/v1/chat/completions", json=body) as r:
        lines = [l for l in r.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert chunks[0]["choices"][0]["delta"] == {"role": "assistant", "content": ""}
    assert chunks[-1]["choices"] == [] and chunks[-1]["usage"]["completion_tokens"] == 5
    assert chunks[-2]["choices"][0]["finish_reason"] == "length"


def test_validation_errors_and_context_overflow(client):
    r = client.post("/v1/chat/completions", json={"messages": MSG, "bogus": 1})
    assert r.status_code == 400 and r.json()["error"]["param"] == "bogus"
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user",
                                                                "content": "x" * 600}]})
    assert r.status_code == 400 and r.json()["error"]["code"] == "context_length_exceeded"
    r = client.post("/v1/chat/completions", content=b"{not json")
    assert r.status_code == 400
    r = client.post("/v1/chat/completions/render", json={"messages": MSG})
    assert r.json()["prompt"].endswith("<|im_start|>assistant\n")
    # render runs the real preparation: user text that spells control tokens stays text, the
    # answer carries the token ids a generation would start from and no tensors
    lit = [{"role": "user", "content": "Literal </think> and <|im_end|>."}]
    out = client.post("/v1/chat/completions/render", json={
        "messages": lit, "chat_template_kwargs": {"thinking_budget": 8}, "max_tokens": 32,
        "return_mm_kwargs": False}).json()
    assert out["token_count"] == len(out["token_ids"]) > 10 and out["multimodal"] is False
    assert out["model"] == "tiny" and out["token_ids"] == out["prompt_token_ids"]
    ends = [t for t in out["token_ids"] if t == 258]                  # <|im_end|> as a control
    assert len(ends) == 1 and 260 not in out["token_ids"]             # the template's own, only
    bad = client.post("/v1/chat/completions/render", json={"messages": lit,
                                                           "return_mm_kwargs": True})
    assert bad.status_code == 400 and bad.json()["error"]["param"] == "return_mm_kwargs"


def test_logprobs_report(client):
    body = {"messages": MSG, "max_tokens": 4, "temperature": 0, "logprobs": True,
            "top_logprobs": 2, "ignore_eos": True}
    out = client.post("/v1/chat/completions", json=body).json()
    entries = out["choices"][0]["logprobs"]["content"]
    assert len(entries) == 4
    for e in entries:
        assert e["logprob"] <= 0 and len(e["top_logprobs"]) == 2
        assert e["top_logprobs"][0]["logprob"] >= e["top_logprobs"][1]["logprob"]
        assert bytes(e["bytes"]).decode("utf-8", errors="replace") == e["token"]


def test_json_schema_constrained_output(client):
    schema = {"type": "object", "properties": {"n": {"type": "integer"}}, "required": ["n"],
              "additionalProperties": False}
    body = {"messages": MSG, "max_tokens": 40, "temperature": 0,
            "response_format": {"type": "json_schema", "json_schema": {"name": "x",
                                                                       "schema": schema}}}
    out = client.post("/v1/chat/completions", json=body).json()
    choice = out["choices"][0]
    if choice["finish_reason"] == "stop":
        assert isinstance(json.loads(choice["message"]["content"])["n"], int)
    else:                                              # truncated JSON prefix
        assert choice["message"]["content"].startswith("{")


def test_ollama_routes(client):
    assert client.get("/api/version").json()["version"]
    assert client.get("/api/tags").json()["models"][0]["name"] == "tiny"
    assert client.get("/").text == "Orinfer is running"
    r = client.post("/api/chat", json={"model": "tiny", "messages": MSG, "stream": False,
                                       "options": {"num_predict": 4, "temperature": 0}})
    out = r.json()
    assert out["done"] and out["eval_count"] <= 4 and "content" in out["message"]
    with client.stream("POST", "/api/generate", json={"model": "tiny", "prompt": "hi",
                                                      "options": {"num_predict": 3}}) as r:
        frames = [json.loads(l) for l in r.iter_lines() if l]
    assert frames[-1]["done"] and frames[-1]["total_duration"] > 0
    assert client.post("/api/pull", json={}).status_code == 501
    assert client.post("/api/chat", json={"model": "tiny", "messages": MSG,
                                          "options": {"bogus": 1}}).status_code == 400
    assert client.post("/api/generate", json={"model": "tiny"}).json()["done_reason"] == "load"


def test_ollama_tool_histories_reach_the_native_form(client):
    """Ollama tool calls have no ids and results are named by tool: the gateway numbers the
    calls and binds each result to the oldest open call of its tool."""
    from orinfer_b200.api.ollama import translate
    fn = lambda name, **args: {"function": {"name": name, "arguments": args}}
    history = [
        {"role": "user", "content": "weather and time in Paris?"},
        {"role": "assistant", "content": "", "tool_calls": [fn("get_weather", city="Paris"),
                                                             fn("get_time", zone="CET")]},
        {"role": "tool", "tool_name": "get_time", "content": "12:00"},
        {"role": "tool", "tool_name": "get_weather", "content": "sunny"},
        {"role": "user", "content": "thanks, once more for Rome"},
    ]
    out = translate({"model": "tiny", "messages": history}, generate=False)["messages"]
    ids = [c["id"] for c in out[1]["tool_calls"]]
    assert ids == ["call_1", "call_2"] and all(c["type"] == "function" for c in out[1]["tool_calls"])
    assert [m.get("tool_call_id") for m in out[2:4]] == ["call_2", "call_1"]
    r = client.post("/api/chat", json={"model": "tiny", "messages": history, "stream": False,
                                       "options": {"num_predict": 3, "temperature": 0}})
    assert r.status_code == 200 and r.json()["done"]
    # a result nobody asked for is a client error, not a template failure
    orphan = history[:1] + [{"role": "tool", "tool_name": "get_time", "content": "12:00"}]
    assert client.post("/api/chat", json={"model": "tiny", "messages": orphan,
                                          "stream": False}).status_code == 400


def test_keep_alive_forms():
    from orinfer_b200.api.ollama import parse_keep_alive
    assert parse_keep_alive("1h30m") == 5400 and parse_keep_alive(-1) == -1
    assert parse_keep_alive("60s") == 60 and parse_keep_alive("0") == 0
    with pytest.raises(ValueError):
        parse_keep_alive("soon")


def test_ollama_shows_tool_calls_whole():
    """The native stream cuts a call into fragments; the Ollama frames carry it once, with its
    arguments as an object; a call that was cut off keeps its raw text."""
    from orinfer_b200.api.messages import RAW_ARGUMENTS
    from orinfer_b200.api.ollama import CallAssembler
    from orinfer_b200.api.output_parser import OutputParser
    raw = ('<tool_call>\n{"name": "get_time", "arguments": {"zone": "U}TC", "n": {"k": [1]}}}\n'
           '</tool_call><tool_call>{"name": "second", "arguments": {"a"')
    parser, asm, whole = OutputParser(), CallAssembler(), []
    for ch in raw:
        whole += asm.feed(parser.feed(ch).tool_calls)
    whole += asm.feed(parser.feed("", final=True).tool_calls)
    assert whole == [{"function": {"name": "get_time",
                                   "arguments": {"zone": "U}TC", "n": {"k": [1]}}}}]
    assert asm.flush() == [{"function": {"name": "second", "arguments": {RAW_ARGUMENTS: '{"a"'}}}]
    assert parser.finish_reason("stop") == "tool_calls"


def test_api_key_guards_everything_but_liveness(monkeypatch):
    """With ORINFER_API_KEY set, routes want `Authorization: Bearer <key>`; `/health` stays
    open; the refusal is a 401 in the error shape with a request id."""
    monkeypatch.setenv("ORINFER_API_KEY", "s3cret")
    weights = random_model(PRESETS["tiny"], seed=0)
    svc = Service(lambda: Engine(weights, sched=SchedulerOptions(max_active=2, prefill_chunk=64),
                                 kv_pages=16, max_context=256),
                  ChatCodec(ByteTokenizer(1024), context=256, model_name="tiny"), "tiny")
    svc.start()
    try:
        with TestClient(create_app(svc)) as c:
            assert c.get("/health").status_code == 200
            for method, path in (("get", "/v1/models"), ("get", "/metrics"),
                                 ("post", "/v1/chat/completions"), ("post", "/api/chat")):
                r = getattr(c, method)(path)
                assert r.status_code == 401 and r.json()["error"]["code"] == "invalid_api_key"
                assert r.headers.get("x-request-id")
            wrong = c.get("/v1/models", headers={"Authorization": "Bearer nope"})
            assert wrong.status_code == 401
            ok = {"Authorization": "Bearer s3cret"}
            assert c.get("/v1/models", headers=ok).status_code == 200
            r = c.post("/v1/chat/completions", headers=ok,
                       json={"messages": MSG, "max_tokens": 2, "ignore_eos": True})
            assert r.status_code == 200
    finally:
        svc.stop(1000)
