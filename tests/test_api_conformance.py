"""API conformance checks in the spirit of the reference's compatibility suite
(tools/api/compatibility.py): seeds, cache hints, logit bias, JSON modes over SSE, request
state isolation, token bytes in logprobs."""
import json

import pytest
from fastapi.testclient import TestClient

from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec
from orinfer_b200.api.server import Service, create_app
from orinfer_b200.config import PRESETS, SchedulerOptions
from orinfer_b200.engine.engine import Engine
from orinfer_b200.models.weights import random_model

MSG = [{"role": "user", "content": "hello"}]


@pytest.fixture(scope="module")
def client():
    weights = random_model(PRESETS["tiny"], seed=0)
    svc = Service(lambda: Engine(weights, sched=SchedulerOptions(max_active=4, prefill_chunk=64),
                                 kv_pages=32, max_context=512),
                  ChatCodec(ByteTokenizer(1024), context=512, model_name="tiny"), "tiny")
    svc.start()
    with TestClient(create_app(svc)) as c:
        yield c
    svc.stop(1000)


def _chat(client, **kw):
    body = dict(dict(messages=MSG, max_tokens=6, ignore_eos=True), **kw)
    r = client.post("/v1/chat/completions", json=body)
    assert r.status_code == 200, r.text
    return r.json()


def test_nullable_and_signed_seed(client):
    a = _chat(client, temperature=1.0, seed=None)
    assert a["choices"][0]["finish_reason"] == "length"
    neg1 = _chat(client, temperature=1.0, seed=-5)
    neg2 = _chat(client, temperature=1.0, seed=-5)
    assert neg1["choices"][0]["message"] == neg2["choices"][0]["message"]
    bad = client.post("/v1/chat/completions", json=dict(messages=MSG, seed="x"))
    assert bad.status_code == 400 and bad.json()["error"]["param"] == "seed"


def test_cache_hints_preserve_output(client):
    plain = _chat(client, temperature=0)
    hinted = _chat(client, temperature=0, prompt_cache_key="tenant-1", prompt_cache_retention="24h")
    again = _chat(client, temperature=0, prompt_cache_key="tenant-1")
    assert plain["choices"][0]["message"] == hinted["choices"][0]["message"] \
        == again["choices"][0]["message"]


def test_logit_bias_forces_and_bans_tokens(client):
    forced = _chat(client, temperature=0, logit_bias={"65": 100})
    assert forced["choices"][0]["message"]["content"] == "A" * 6
    base = _chat(client, temperature=0, logprobs=True, top_logprobs=1)
    first = base["choices"][0]["logprobs"]["content"][0]
    tok_id = first["bytes"][0] if first.get("bytes") else None
    if tok_id is not None and tok_id < 256:
        banned = _chat(client, temperature=0, logit_bias={str(tok_id): -100}, logprobs=True)
        assert banned["choices"][0]["logprobs"]["content"][0]["bytes"] != first["bytes"]
    assert client.post("/v1/chat/completions",
                       json=dict(messages=MSG, logit_bias={"65": 101})).status_code == 400


def test_json_object_and_schema_over_sse(client):
    obj = _chat(client, temperature=0, max_tokens=48, ignore_eos=False,
                response_format={"type": "json_object"})
    text = obj["choices"][0]["message"]["content"]
    if obj["choices"][0]["finish_reason"] == "stop":
        assert isinstance(json.loads(text), dict)
    else:
        assert text.lstrip().startswith("{")
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}}, "required": ["ok"],
              "additionalProperties": False}
    body = dict(messages=MSG, max_tokens=48, temperature=0, stream=True,
                response_format={"type": "json_schema",
                                 "json_schema": {"name": "r", "schema": schema, "strict": True}})
    with client.stream("POST", "/v1/chat/completions", json=body) as r:
        chunks = [json.loads(l[6:]) for l in r.iter_lines()
                  if l.startswith("data: ") and l != "data: [DONE]"]
    text = "".join(c["choices"][0]["delta"].get("content") or "" for c in chunks if c["choices"])
    assert json.loads(text)["ok"] in (True, False)
    assert chunks[-1]["choices"][0]["finish_reason"] == "stop"


def test_request_state_isolation(client):
    """A request's output does not depend on what ran before it or beside it."""
    import concurrent.futures as cf
    solo = _chat(client, temperature=0.9, seed=11)["choices"][0]["message"]
    others = [dict(messages=[{"role": "user", "content": f"noise {i}"}], max_tokens=9,
                   temperature=1.0, seed=i, ignore_eos=True) for i in range(3)]
    with cf.ThreadPoolExecutor(4) as pool:
        futs = [pool.submit(client.post, "/v1/chat/completions", json=b) for b in others]
        mixed = _chat(client, temperature=0.9, seed=11)["choices"][0]["message"]
        assert all(f.result().status_code == 200 for f in futs)
    assert mixed == solo


def test_unicode_token_bytes_in_logprobs(client):
    body = dict(messages=[{"role": "user", "content": "héllo ✓"}], max_tokens=5, temperature=0,
                logprobs=True, top_logprobs=2, ignore_eos=True)
    r = client.post("/v1/chat/completions", json=body).json()
    entries = r["choices"][0]["logprobs"]["content"]
    assert len(entries) == 5
    for e in entries:
        assert isinstance(e["bytes"], list) and all(0 <= b < 256 for b in e["bytes"])
        assert e["logprob"] <= 0 and len(e["top_logprobs"]) == 2
    raw = bytes(b for e in entries for b in e["bytes"])
    assert raw.decode("utf-8", errors="replace") is not None


def test_validation_errors_name_their_parameter(client):
    """Each malformed field is refused with 400, a request id and ``error.param`` naming it."""
    base = dict(messages=MSG, temperature=0, seed=-20261002, max_completion_tokens=16)
    schema_ref = {"type": "json_schema", "json_schema": {
        "name": "remote", "schema": {"$ref": "https://example.com/schema"}}}
    table = [
        ({"stream": "yes"}, "stream"),
        ({"top_logprobs": 3}, "top_logprobs"),
        ({"logprobs": True, "top_logprobs": 21}, "top_logprobs"),
        ({"store": True}, "store"),
        ({"temperature": -1}, "temperature"),
        ({"reasoning_effort": "invalid"}, "reasoning_effort"),
        ({"reasoning_effort": "none", "enable_thinking": True}, "enable_thinking"),
        ({"thinking_token_budget": -1}, "thinking_token_budget"),
        ({"prompt_cache_key": "x" * 65}, "prompt_cache_key"),
        ({"prompt_cache_key": ""}, "prompt_cache_key"),
        ({"prompt_cache_retention": "forever"}, "prompt_cache_retention"),
        ({"enable_thinking": True, "thinking_token_budget": 0, "max_completion_tokens": 1},
         "max_completion_tokens"),
        ({"max_tokens": 4}, "max_completion_tokens"),                 # two limits at once
        ({"logit_bias": {"999999999": 1}}, "logit_bias.999999999"),
        ({"response_format": schema_ref}, "response_format.json_schema.schema"),
        ({"response_format": {"type": "json_schema", "json_schema": {
            "name": "x", "schema": {"properties": {"a": {"x-guidance": {}}}}}}},
         "response_format.json_schema.schema"),
    ]
    for fields, param in table:
        r = client.post("/v1/chat/completions", json=dict(base, **fields))
        assert r.status_code == 400, (fields, r.text)
        assert r.headers.get("x-request-id")
        assert r.json()["error"]["param"] == param, (fields, r.json())
    # the accepted spellings of the same fields
    ok = dict(base, stream=None, tools=None, store=False, metadata={"t": "c"}, service_tier="auto",
              prompt_cache_key="pi-session-probe", prompt_cache_retention="24h",
              reasoning_effort="xhigh", logit_bias={"42": -100})
    assert client.post("/v1/chat/completions", json=ok).status_code == 200


def test_recognizable_context_overflow(client):
    """An output limit the client named is kept or refused, never silently shortened; the
    refusal carries the code clients look for."""
    limit = client.get("/health").json()["max_context"]
    r = client.post("/v1/chat/completions", json=dict(messages=MSG, max_completion_tokens=limit))
    err = r.json()["error"]
    assert r.status_code == 400 and err["code"] == "context_length_exceeded"
    assert "exceeds the context window" in err["message"] and err["param"] == "max_completion_tokens"
    # without a limit of its own a request gets what fits
    assert client.post("/v1/chat/completions", json=dict(messages=MSG)).status_code == 200


def test_unknown_routes_answer_in_the_error_shape(client):
    for path, code in (("/v1/missing", 404), ("/v1/chat/completions", 405)):
        r = client.get(path)
        assert r.status_code == code and r.json()["error"]["message"]


@pytest.fixture(scope="module")
def roomy():
    """A server with room for tool prompts (2048-token context)."""
    weights = random_model(PRESETS["tiny"], seed=0)
    svc = Service(lambda: Engine(weights, sched=SchedulerOptions(max_active=4, prefill_chunk=64),
                                 kv_pages=64, max_context=2048),
                  ChatCodec(ByteTokenizer(1024), context=2048, model_name="tiny"), "tiny")
    svc.start()
    with TestClient(create_app(svc)) as c:
        yield c
    svc.stop(1000)


def _sse(client, body):
    out = []
    with client.stream("POST", "/v1/chat/completions",
                       json=dict(body, stream=True, stream_options={"include_usage": True})) as r:
        for line in r.iter_lines():
            if line.startswith("data: ") and line != "data: [DONE]":
                out.append(json.loads(line[6:]))
    return out


def _check_scores(content, scores, count):
    import math
    assert b"".join(bytes(s["bytes"]) for s in scores).decode() == content
    for s in scores:
        assert math.isfinite(s["logprob"]) and s["logprob"] <= 0
        tops = [t["logprob"] for t in s["top_logprobs"]]
        assert len(tops) <= count and tops == sorted(tops, reverse=True)
        assert all(math.isfinite(t) and t <= 0 for t in tops)


COMMON = dict(temperature=0, seed=-20261002, max_completion_tokens=200,
              messages=[{"role": "user", "content": "2+3?"}])
LITERAL = "<think>中文</think><tool_call>literal</tool_call>"
LITERAL_FORMAT = {"type": "json_schema", "json_schema": {"name": "literal", "strict": True, "schema": {
    "type": "object", "properties": {"text": {"type": "string", "const": LITERAL}},
    "required": ["text"], "additionalProperties": False}}}


def test_json_literal_protocol_tags_and_probabilities_over_sse(roomy):
    """A schema constant that spells the protocol's own tags is content, character for
    character: it is neither parsed as reasoning or a tool call nor emitted as control tokens;
    streamed text and probabilities equal the non-streamed ones; usage rides only the last
    chunk; one token of budget ends with `length`."""
    body = dict(COMMON, logprobs=True, top_logprobs=3, response_format=LITERAL_FORMAT)
    full = roomy.post("/v1/chat/completions", json=body).json()
    choice = full["choices"][0]
    assert choice["finish_reason"] == "stop"
    assert json.loads(choice["message"]["content"]) == {"text": LITERAL}
    assert not choice["message"].get("tool_calls") and not choice["message"].get("reasoning_content")
    _check_scores(choice["message"]["content"], choice["logprobs"]["content"], 3)
    chunks = _sse(roomy, body)
    text = "".join(c["choices"][0]["delta"].get("content") or "" for c in chunks if c["choices"])
    scores = [s for c in chunks if c["choices"]
              for s in (c["choices"][0].get("logprobs") or {}).get("content", [])]
    assert text == choice["message"]["content"] and scores == choice["logprobs"]["content"]
    assert all(c.get("usage") is None for c in chunks[:-1]) and chunks[-1]["usage"]
    assert chunks[-2]["choices"][0]["finish_reason"] == "stop"
    cut = roomy.post("/v1/chat/completions", json=dict(body, max_completion_tokens=1)).json()
    assert cut["choices"][0]["finish_reason"] == "length"
    # sampling under the constraint is reproducible for a seed
    sampled = dict(body, temperature=0.7, top_p=0.9)
    a = roomy.post("/v1/chat/completions", json=sampled).json()
    b = roomy.post("/v1/chat/completions", json=sampled).json()
    assert a["choices"] == b["choices"]


def test_strict_tools_local_references_histories_and_thinking_budgets(roomy):
    tools = [{"type": "function", "function": {
        "name": "read_verification", "strict": True, "description": "Read a local code.",
        "parameters": {"type": "object",
                       "$defs": {"filename": {"type": "string", "enum": ["input.txt"]}},
                       "properties": {"filename": {"$ref": "#/$defs/filename"},
                                      "count": {"type": "integer", "const": 2}},
                       "required": ["filename", "count"], "additionalProperties": False}}}]
    ask = dict(COMMON, tools=tools, parallel_tool_calls=False, tool_choice="required",
               messages=[{"role": "user", "content": "Call read_verification."}])
    want = {"filename": "input.txt", "count": 2}
    first = roomy.post("/v1/chat/completions", json=ask).json()["choices"][0]
    call = first["message"]["tool_calls"][0]
    assert first["finish_reason"] == "tool_calls" and json.loads(call["function"]["arguments"]) == want
    # the call and its result as history (arguments travel as a JSON string), tools switched off
    done = roomy.post("/v1/chat/completions", json=dict(
        ask, tool_choice="none", max_completion_tokens=8, messages=ask["messages"] + [
            {"role": "assistant", "content": None, "tool_calls": [call]},
            {"role": "tool", "tool_call_id": call["id"], "content": '{"code":"CHECK_5824"}'}]))
    assert done.status_code == 200 and not done.json()["choices"][0]["message"].get("tool_calls")
    # a call whose arguments were cut off stays in the history for the model to recover from
    broken = json.loads(json.dumps(call))
    broken["function"]["arguments"] = '{"filename":'
    again = roomy.post("/v1/chat/completions", json=dict(ask, messages=ask["messages"] + [
        {"role": "assistant", "content": None, "tool_calls": [broken]},
        {"role": "tool", "tool_call_id": broken["id"], "content": "Invalid arguments. Retry."}]))
    assert again.status_code == 200, again.text
    retry = again.json()["choices"][0]["message"]["tool_calls"][0]
    assert json.loads(retry["function"]["arguments"]) == want
    # thinking budgets hold beside a forced tool call and beside a schema
    capped = roomy.post("/v1/chat/completions", json=dict(
        ask, enable_thinking=True, thinking_token_budget=8)).json()
    assert capped["choices"][0]["message"]["tool_calls"]
    assert capped["usage"]["completion_tokens_details"]["reasoning_tokens"] <= 8
    capped = roomy.post("/v1/chat/completions", json=dict(
        COMMON, response_format=LITERAL_FORMAT, enable_thinking=True, thinking_token_budget=8)).json()
    assert json.loads(capped["choices"][0]["message"]["content"]) == {"text": LITERAL}
    assert capped["usage"]["completion_tokens_details"]["reasoning_tokens"] <= 8
    # streamed forced call: several argument fragments, finish reason on the chunk before usage
    chunks = _sse(roomy, ask)
    deltas = [d for c in chunks if c["choices"] for d in c["choices"][0]["delta"].get("tool_calls", [])]
    args = "".join(d["function"].get("arguments") or "" for d in deltas)
    assert len(deltas) > 1 and json.loads(args) == want
    assert chunks[-2]["choices"][0]["finish_reason"] == "tool_calls"


def test_a_failing_constraint_fails_one_request_not_the_server(roomy, monkeypatch):
    from orinfer_b200.api import grammar
    real = grammar.GrammarConstraint.consume
    calls = {"n": 0}

    def flaky(self, token):
        calls["n"] += 1
        if calls["n"] == 4:
            raise grammar.GrammarError("parser too complex\nstate dump")
        return real(self, token)

    monkeypatch.setattr(grammar.GrammarConstraint, "consume", flaky)
    body = dict(COMMON, response_format=LITERAL_FORMAT)
    r = roomy.post("/v1/chat/completions", json=body)
    assert r.status_code == 500 and r.json()["error"]["code"] == "generation_failed"
    assert "parser too complex" in r.json()["error"]["message"]
    assert "state dump" not in r.json()["error"]["message"]
    assert roomy.get("/health").status_code == 200                   # still serving
    ok = roomy.post("/v1/chat/completions", json=body)
    assert ok.status_code == 200
    assert json.loads(ok.json()["choices"][0]["message"]["content"]) == {"text": LITERAL}


def test_stream_chunks_keep_one_identity_and_one_field_per_delta(roomy):
    """Every chunk of a stream carries the same id / created / model / object; the role comes
    once; the finish reason rides an empty delta; usage only the last chunk; a delta carries
    content, reasoning or tool-call fragments, never two of them; text parts and a plain
    string give the same result."""
    tools = [{"type": "function", "function": {"name": "get_weather", "strict": True, "parameters": {
        "type": "object", "properties": {"location": {"type": "string", "enum": ["Boston"]}},
        "required": ["location"], "additionalProperties": False}}}]
    body = dict(messages=[{"role": "user", "content": "Call it"}], tools=tools, tool_choice="required",
                parallel_tool_calls=False, max_completion_tokens=80, temperature=0, seed=1)
    chunks = _sse(roomy, body)
    assert len(chunks) > 5
    for name in ("id", "created", "model", "object"):
        assert all(c[name] == chunks[0][name] for c in chunks), name
    deltas = [c["choices"][0]["delta"] for c in chunks if c["choices"]]
    assert [d["role"] for d in deltas if "role" in d] == ["assistant"] and deltas[-1] == {}
    assert all(c["choices"][0]["finish_reason"] is None for c in chunks[:-2])
    assert chunks[-2]["choices"][0]["finish_reason"] == "tool_calls" and chunks[-1]["choices"] == []
    for d in deltas:
        assert sum(bool(d.get(f)) for f in ("content", "reasoning_content", "tool_calls")) <= 1
    usage = chunks[-1]["usage"]
    assert usage["total_tokens"] == usage["prompt_tokens"] + usage["completion_tokens"]
    parts = dict(COMMON, max_completion_tokens=8, messages=[{"role": "user", "content": [
        {"type": "text", "text": "Say"}, {"type": "text", "text": " hi"}]}])
    text = dict(parts, messages=[{"role": "user", "content": "Say hi"}])
    a = roomy.post("/v1/chat/completions", json=parts).json()
    b = roomy.post("/v1/chat/completions", json=text).json()
    assert a["choices"] == b["choices"] and a["usage"] == b["usage"]
