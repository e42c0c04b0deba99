"""Tool-call grammar recipes (JSON form inside <tool_call> markers)."""
import json

import pytest

from orinfer_b200.api import tool_grammar as T
from orinfer_b200.api.chat_codec import ByteTokenizer

llguidance = pytest.importorskip("llguidance")

TOOLS = [{"type": "function", "function": {"name": "edit", "parameters": {
    "type": "object", "properties": {"text": {"type": "string"}, "count": {"type": "integer"}},
    "required": ["text"], "additionalProperties": False}}},
    {"type": "function", "function": {"name": "noop", "parameters": {
        "type": "object", "properties": {}, "additionalProperties": False}}}]
TOK = ByteTokenizer(1024)


def call(name, args):
    # fixed spelling of the envelope, compact arguments (the grammar admits no padding)
    return ('<tool_call>\n{"name": ' + json.dumps(name) + ', "arguments": '
            + json.dumps(args, separators=(",", ":")) + "}\n</tool_call>")


def accepts(text, **kw):
    from orinfer_b200.api.grammar import GrammarConstraint
    c = GrammarConstraint.from_lark(TOK, 1024, T.recipe(TOK, TOOLS, **kw), TOK.eos_ids)
    for t in TOK.encode(text):
        mask = c.mask(1024)
        if not (mask[t // 32] >> (t % 32)) & 1:
            return False
        c.consume(t)
    return bool(c.m.is_accepting())


def test_when_a_recipe_applies():
    assert not T.applies([], "required", True) and not T.applies(TOOLS, "none", True)
    assert T.applies(TOOLS, "required", True)
    assert T.applies(TOOLS, {"type": "function", "function": {"name": "edit"}}, True)
    assert not T.applies(TOOLS, "auto", True) and T.applies(TOOLS, "auto", False)
    strict = [dict(TOOLS[0], function=dict(TOOLS[0]["function"], strict=True))]
    assert T.applies(strict, "auto", True)
    with pytest.raises(ValueError, match="undeclared"):
        T.recipe(TOK, TOOLS, {"type": "function", "function": {"name": "rm"}})


def test_required_calls_follow_names_and_schemas():
    good = call("edit", {"text": "hi", "count": 2})
    assert accepts(good, tool_choice="required")
    assert accepts(good + "\n" + call("noop", {}), tool_choice="required")
    assert not accepts(good + "\n" + call("noop", {}), tool_choice="required", parallel=False)
    assert not accepts("Sure. " + good, tool_choice="required")                 # no free text
    assert not accepts(call("rm", {}), tool_choice="required")                   # undeclared
    assert not accepts(call("edit", {"count": 2}), tool_choice="required")       # missing field
    assert not accepts(call("edit", {"text": 3}), tool_choice="required")        # wrong type
    # markers are control tokens: spelling them out as text is not a call
    spelled = "".join(chr(b) for b in b"<tool_call>")
    assert TOK.encode(spelled) == [TOK.special_ids["<tool_call>"]]
    plain_ids = TOK.encode_plain(spelled)
    from orinfer_b200.api.grammar import GrammarConstraint
    c = GrammarConstraint.from_lark(TOK, 1024, T.recipe(TOK, TOOLS, "required"), TOK.eos_ids)
    mask = c.mask(1024)
    assert not (mask[plain_ids[0] // 32] >> (plain_ids[0] % 32)) & 1


def test_named_choice_and_optional_calls():
    named = {"type": "function", "function": {"name": "noop"}}
    assert accepts(call("noop", {}), tool_choice=named)
    assert not accepts(call("edit", {"text": "x"}), tool_choice=named)
    assert not accepts(call("noop", {}) + "\n" + call("noop", {}), tool_choice=named)
    assert accepts("Just an answer.", tool_choice="auto", parallel=False)
    assert accepts("Let me do it.\n" + call("edit", {"text": "x"}), tool_choice="auto",
                   parallel=False)
    assert not accepts(call("edit", {"text": "x"}) + "\n" + call("noop", {}), tool_choice="auto",
                       parallel=False)


def test_server_constrains_required_tool_calls():
    from fastapi.testclient import TestClient
    from orinfer_b200.api.chat_codec import ChatCodec
    from orinfer_b200.api.server import Service, create_app
    from orinfer_b200.config import PRESETS, SchedulerOptions
    from orinfer_b200.engine.engine import Engine
    from orinfer_b200.models.weights import random_model
    weights = random_model(PRESETS["tiny"], seed=0)
    svc = Service(lambda: Engine(weights, sched=SchedulerOptions(max_active=2, prefill_chunk=64),
                                 kv_pages=24, max_context=1024),
                  ChatCodec(ByteTokenizer(1024), context=1024, model_name="tiny"), "tiny")
    svc.start()
    with TestClient(create_app(svc)) as c:
        body = {"messages": [{"role": "user", "content": "do it"}], "tools": TOOLS[1:],
                "tool_choice": "required", "parallel_tool_calls": False, "max_tokens": 80,
                "temperature": 0}
        r = c.post("/v1/chat/completions", json=body).json()
        # random weights, but the grammar leaves only one way to finish: a noop call
        msg = r["choices"][0]["message"]
        assert r["choices"][0]["finish_reason"] == "tool_calls", r
        assert msg["tool_calls"][0]["function"]["name"] == "noop"
        assert json.loads(msg["tool_calls"][0]["function"]["arguments"]) == {}
        bad = c.post("/v1/chat/completions", json=dict(
            body, tool_choice={"type": "function", "function": {"name": "rm"}}))
        assert bad.status_code == 400 and "undeclared" in bad.json()["error"]["message"]
    svc.stop(1000)
