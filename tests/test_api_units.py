"""Chat codec, output parser, grammar and thinking-budget units (CPU)."""
import json

import numpy as np
import pytest

from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec, RequestError, merge_defaults
from orinfer_b200.api.grammar import GrammarConstraint, ThinkingBudget
from orinfer_b200.api.output_parser import OutputParser, parse_tool_call


def _codec():
    return ChatCodec(ByteTokenizer(1024), context=512, model_name="tiny")


def test_defaults_merge_rules():
    dep = {"temperature": 0.7, "enable_thinking": True, "max_tokens": 64}
    assert merge_defaults({"temperature": None}, dep) == {"enable_thinking": True, "max_tokens": 64}
    got = merge_defaults({"reasoning_effort": "high", "max_completion_tokens": 9}, dep)
    assert got == {"temperature": 0.7, "reasoning_effort": "high", "max_completion_tokens": 9}


def test_prepare_validates_and_tokenises():
    c = _codec()
    p = c.prepare({"messages": [{"role": "user", "content": "hi"}], "seed": -5, "top_k": -1,
                   "max_tokens": 7, "stream": True, "stream_options": {"include_usage": True}})
    assert p.max_new == 7 and p.stream and p.include_usage and p.sampling.top_k == 0
    assert p.sampling.seed == (-5) & (2 ** 64 - 1)
    assert c.tokenizer.decode(p.prompt_ids).endswith("<|im_start|>assistant\n")
    for body, param in [({"messages": []}, "messages"), ({"messages": [{"role": "x"}]}, "messages[0].role"),
                        ({"messages": [{"role": "user", "content": "a"}], "n": 2}, "n"),
                        ({"messages": [{"role": "user", "content": "a"}], "bogus": 1}, "bogus"),
                        ({"messages": [{"role": "user", "content": "a"}], "temperature": 3}, "temperature"),
                        ({"messages": [{"role": "user", "content": "a"}], "stop": ["a"] * 5}, "stop"),
                        ({"messages": [{"role": "user", "content": "a"}], "store": True}, "store")]:
        with pytest.raises(RequestError) as e:
            c.prepare(body)
        assert e.value.param == param
    with pytest.raises(RequestError) as e:
        c.prepare({"messages": [{"role": "user", "content": "x" * 600}]})
    assert e.value.code == "context_length_exceeded" and e.value.status == 400


def test_parser_thinking_tools_and_withholding_every_split():
    text = ("plan</think>Hello <tool_call>\n{\"name\": \"f\", \"arguments\": {\"a\": 1}}\n</tool_call>"
            " bye STOP tail")
    want = None
    for cut in range(1, len(text)):
        p = OutputParser(thinking=True, stops=["STOP"])
        parts = [p.feed(text[:cut]), p.feed(text[cut:], final=True)]
        calls = {}
        for c in (c for d in parts for c in d.tool_calls):       # fragments of a streamed call
            e = calls.setdefault(c["index"], {"name": "", "arguments": ""})
            e["name"] += c["function"].get("name") or ""
            e["arguments"] += c["function"].get("arguments") or ""
        got = ("".join(d.reasoning for d in parts), "".join(d.content for d in parts),
               [calls[i] for i in sorted(calls)], p.stopped)
        want = want or got
        assert got == want, cut
    assert want[0] == "plan" and want[1] == "Hello  bye " and want[3]
    assert want[2] == [{"name": "f", "arguments": "{\"a\": 1}"}]
    assert OutputParser().finish_reason("length") == "length"


def test_parser_xml_tool_call_and_json_mode():
    call = parse_tool_call("<function=get_weather><parameter=city>\nParis\n</parameter>"
                           "<parameter=days>3</parameter></function>")
    assert call["name"] == "get_weather" and json.loads(call["arguments"]) == {"city": "Paris", "days": 3}
    p = OutputParser(json_mode=True)
    d = p.feed('{"a": "<think>x</think><tool_call>"}', final=True)
    assert d.content == '{"a": "<think>x</think><tool_call>"}' and not d.tool_calls


def test_grammar_constraint_masks_and_forks():
    tok = ByteTokenizer(1024)
    schema = {"type": "object", "properties": {"answer": {"type": "integer"}},
              "required": ["answer"], "additionalProperties": False}
    g = GrammarConstraint(tok, 1024, schema, tok.eos_ids)
    allowed = lambda m, t: bool(m[t // 32] >> (t % 32) & 1)
    m = g.mask(1024)
    assert allowed(m, ord("{")) and not allowed(m, ord("x")) and not allowed(m, tok.eos_ids[0])
    fork = g.fork()
    for ch in b'{"answer":42}':
        assert allowed(g.mask(1024), ch), chr(ch)
        g.consume(ch)
    m = g.mask(1024)
    assert allowed(m, tok.eos_ids[0]) and not allowed(m, ord("a"))
    g.consume(tok.eos_ids[0])
    assert g.finished() and not fork.finished()
    assert allowed(fork.mask(1024), ord("{"))


def test_thinking_budget_forces_close():
    tok = ByteTokenizer(1024)
    close = tok.encode("</think>")
    tb = ThinkingBudget(close, budget=3, max_new=20)
    for t in (65, 66, 67):
        assert tb.mask(1024) is None
        tb.consume(t)
    m = tb.mask(1024)
    assert m is not None and int(np.unpackbits(m.view(np.uint8)).sum()) == 1
    tb.consume(close[0])
    assert tb.closed and tb.mask(1024) is None
    # the budget always leaves room for the answer
    assert ThinkingBudget(close, budget=100, max_new=10).budget == 8


def test_codec_loads_templates_kept_in_the_tokenizer_configuration(tmp_path):
    import json
    from orinfer_b200.api.chat_codec import ChatCodec, RequestError
    template = ("{% for m in messages %}{% if m.role == 'tool' %}{{ raise_exception('no tools') }}"
                "{% endif %}{% if loop.index > 2 %}{% break %}{% endif %}"
                "<|im_start|>{{ m.role }}: {{ m.content }}<|im_end|>{% endfor %}")
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"chat_template": template}))
    codec = ChatCodec.load(tmp_path, 1024, 512, "m")
    msgs = [{"role": "user", "content": str(i)} for i in range(4)]
    text = codec.prepare({"messages": msgs}).prompt_text
    assert text == "<|im_start|>user: 0<|im_end|><|im_start|>user: 1<|im_end|>"     # break honoured
    try:
        codec.prepare({"messages": [
            {"role": "user", "content": "q"},
            {"role": "assistant", "content": None, "tool_calls": [
                {"id": "c1", "type": "function", "function": {"name": "f", "arguments": "{}"}}]},
            {"role": "tool", "tool_call_id": "c1", "content": "x"}]})
    except RequestError as e:
        assert "no tools" in e.message
    else:
        raise AssertionError("the template's own refusal must surface as a request error")
    (tmp_path / "chat_template.jinja").write_text("{{ messages[0].content }}!")
    assert ChatCodec.load(tmp_path, 1024, 512, "m").prepare({"messages": msgs}).prompt_text == "0!"


def test_histories_are_normalised_before_the_template_sees_them():
    """Wire shapes of one conversation (text parts, null content, JSON-string arguments,
    developer beside system) reach the template in one form; malformed histories are refused."""
    import json

    import pytest
    from orinfer_b200.api.messages import RAW_ARGUMENTS, MessageError, normalize
    call = lambda cid, args: {"id": cid, "type": "function",
                              "function": {"name": "get_weather", "arguments": args}}
    user = {"role": "user", "content": "What is the weather?"}
    # a tool result sent as text parts is the concatenation of the parts; no parts is ""
    got = normalize([user, {"role": "assistant", "content": None, "tool_calls": [call("c1", "{}")]},
                     {"role": "tool", "tool_call_id": "c1",
                      "content": [{"type": "text", "text": "sunny [img]"},
                                  {"type": "text", "text": ", 72F [img-99]"}]}])
    assert got[1]["content"] == "" and got[1]["tool_calls"][0]["function"]["arguments"] == {}
    assert got[2]["content"] == "sunny [img], 72F [img-99]"
    got = normalize([user, {"role": "assistant", "tool_calls": [call("c1", '{"city":"Paris"}')]},
                     {"role": "tool", "tool_call_id": "c1", "content": []}])
    assert got[2]["content"] == "" and \
        got[1]["tool_calls"][0]["function"]["arguments"] == {"city": "Paris"}
    # system and developer instructions become one system message
    got = normalize([{"role": "system", "content": "Be brief."},
                     {"role": "developer", "content": "Call tools when asked."},
                     {"role": "user", "content": [{"type": "text", "text": "Hi"}]}])
    assert got == [{"role": "system", "content": "Be brief.\n\nCall tools when asked."},
                   {"role": "user", "content": "Hi"}]
    # arguments that are not a JSON object are kept for the model to see, not guessed
    got = normalize([user, {"role": "assistant", "tool_calls": [call("c1", '{"city": "Par')]},
                     {"role": "tool", "tool_call_id": "c1", "content": "error: bad arguments"}])
    assert got[1]["tool_calls"][0]["function"]["arguments"] == {RAW_ARGUMENTS: '{"city": "Par'}
    # an image part keeps the part list for the image front end
    parts = [{"type": "text", "text": "look"}, {"type": "image_url", "image_url": {"url": "x"}}]
    assert normalize([{"role": "user", "content": parts}])[0]["content"] == parts
    # dsml histories: parts joined by a blank line, system messages stay where they are,
    # doubly encoded arguments are unwrapped
    got = normalize([user, {"role": "system", "content": "late"},
                     {"role": "assistant", "tool_calls": [call("c1", json.dumps(json.dumps({"a": 1})))]},
                     {"role": "tool", "tool_call_id": "c1",
                      "content": [{"type": "text", "text": "a"}, {"type": "text", "text": "b"}]}],
                    "dsml")
    assert got[1]["role"] == "system" and got[3]["content"] == "a\n\nb"
    assert got[2]["tool_calls"][0]["function"]["arguments"] == {"a": 1}
    bad = [
        ([], "non-empty"),
        ([{"role": "system", "content": "only instructions"}], "user message"),
        ([user, {"role": "system", "content": "late"}], "precede"),
        ([user, {"role": "narrator", "content": "x"}], "role"),
        ([user, {"role": "tool", "tool_call_id": "nope", "content": "x"}], "tool_call_id"),
        ([user, {"role": "assistant", "tool_calls": [call("c1", "{}")]}, user], "answering"),
        ([user, {"role": "assistant", "tool_calls": [call("c1", "{}")]}], "answering"),
        ([user, {"role": "assistant", "tool_calls": [call("c1", "{}"), call("c1", "{}")]}], "unique"),
        ([user, {"role": "assistant", "tool_calls": [call("", "{}")]}], "unique"),
        ([user, {"role": "user", "tool_calls": [call("c1", "{}")], "content": "x"}], "assistant"),
        ([user, {"role": "assistant", "tool_calls": [
            {"id": "c1", "type": "function", "function": {"name": "bad name!", "arguments": "{}"}}]}],
         "invalid assistant tool call"),
        ([user, {"role": "assistant", "tool_calls": [call("c1", 5)]}], "JSON string"),
        ([{"role": "user", "content": 7}], "content"),
        ([{"role": "user", "content": [{"type": "text"}]}], "text"),
    ]
    for history, word in bad:
        with pytest.raises(MessageError, match=word):
            normalize(history)


def test_parser_and_finish_reason_follow_the_protocol_table():
    """Raw model text -> (reasoning, content, calls) for every way of cutting it into two
    pieces, and the finish reason: running out of tokens wins over a finished tool call."""
    import json
    from orinfer_b200.api.output_parser import OutputParser
    call = '<tool_call>{"name":"get_time","arguments":{"timezone":"UTC"}}</tool_call>'
    cases = [
        ("<think>step-by-step</think>final answer", "step-by-step", "final answer", []),
        ("<think>need a tool</think>" + call, "need a tool", "",
         [("get_time", {"timezone": "UTC"})]),
        ("<think>pondering", "pondering", "", []),
        ("hello", "", "hello", []),
        (call, "", "", [("get_time", {"timezone": "UTC"})]),
        ("", "", "", []),
    ]
    for raw, reasoning, content, calls in cases:
        for cut in range(len(raw) + 1):
            p = OutputParser(thinking=False)
            got_r = got_c = ""
            got_calls = {}
            for piece, final in ((raw[:cut], False), (raw[cut:], True)):
                d = p.feed(piece, final=final)
                got_r, got_c = got_r + d.reasoning, got_c + d.content
                for c in d.tool_calls:
                    e = got_calls.setdefault(c["index"], ["", ""])
                    e[0] += c.get("function", {}).get("name") or ""
                    e[1] += c.get("function", {}).get("arguments") or ""
            assert (got_r.strip(), got_c.strip()) == (reasoning, content), (raw, cut)
            assert [(n, json.loads(a or "{}")) for n, a in
                    (got_calls[i] for i in sorted(got_calls))] == calls, (raw, cut)
    for exhausted, has_tool, want in ((False, False, "stop"), (True, False, "length"),
                                      (False, True, "tool_calls"), (True, True, "length")):
        p = OutputParser()
        if has_tool:
            p.feed(call, final=True)
        assert p.finish_reason("length" if exhausted else "stop") == want


def test_deployment_defaults_are_checked_at_start():
    import pytest
    from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec, validate_defaults
    codec = ChatCodec(ByteTokenizer(1024), context=512, model_name="m")
    validate_defaults(codec, {})
    validate_defaults(codec, {"temperature": 0.3, "max_tokens": 64, "enable_thinking": True})
    for bad, word in (({"model": "x"}, "default_request_params.model"),
                      ({"messages": []}, "default_request_params.messages"),
                      ({"temperature": -1}, "default_request_params.temperature"),
                      ({"bogus": 1}, "default_request_params.bogus"),
                      ({"reasoning_effort": "much"}, "default_request_params.reasoning_effort")):
        with pytest.raises(ValueError, match=word):
            validate_defaults(codec, bad)
    # a default limit is shortened to fit, an explicit one is kept or refused
    p = codec.prepare({"messages": [{"role": "user", "content": "x" * 400}]}, {"max_tokens": 4096})
    assert p.max_new < 4096


def test_defaults_only_fill_what_the_request_left_open():
    """The merge rules of deployment defaults, case by case."""
    import pytest
    from orinfer_b200.api.chat_codec import (ByteTokenizer, ChatCodec, RequestError,
                                             merge_defaults, thinking_budget_of)
    d = {"enable_thinking": True, "temperature": 0.7, "stream": True, "stop": ["END"]}
    assert merge_defaults({}, d) == d
    own = {"enable_thinking": False, "temperature": 0, "stream": False, "stop": []}
    assert merge_defaults(own, d) == own                      # false, 0 and [] are answers
    assert merge_defaults({"enable_thinking": None, "temperature": None, "stream": None}, d) \
        == {"stop": ["END"]}                                  # null: not set, default cleared
    # one group, one spelling
    assert merge_defaults({"max_completion_tokens": 8}, {"max_tokens": 64}) == \
        {"max_completion_tokens": 8}
    assert merge_defaults({"reasoning_effort": "none"}, {"enable_thinking": True}) == \
        {"reasoning_effort": "none"}
    assert merge_defaults({"chat_template_kwargs": {"enable_thinking": False}},
                          {"enable_thinking": True, "reasoning_effort": "high"}) == \
        {"chat_template_kwargs": {"enable_thinking": False}}
    # switching a feature off takes its dependent default with it
    assert merge_defaults({"stream": False}, {"stream_options": {"include_usage": True}}) == \
        {"stream": False}
    assert merge_defaults({"logprobs": False}, {"top_logprobs": 5, "logprobs": True}) == \
        {"logprobs": False}
    # template variables merge key by key; null clears the map
    assert merge_defaults({"chat_template_kwargs": {"a": 1}},
                          {"chat_template_kwargs": {"a": 0, "b": 2}}) == \
        {"chat_template_kwargs": {"a": 1, "b": 2}}
    assert merge_defaults({"chat_template_kwargs": None},
                          {"chat_template_kwargs": {"b": 2}}) == {}
    # every spelling of a default budget yields to either spelling in the request
    for default in ({"thinking_token_budget": 512},
                    {"chat_template_kwargs": {"thinking_token_budget": 512}},
                    {"chat_template_kwargs": {"thinking_budget": 512}}):
        for name in ("thinking_budget", "thinking_token_budget"):
            merged = merge_defaults({"chat_template_kwargs": {name: 0}}, default)
            assert thinking_budget_of(merged) == 0, (default, name)
    both = {"thinking_token_budget": 4,
            "chat_template_kwargs": {"thinking_budget": 16, "thinking_token_budget": 16}}
    assert thinking_budget_of(both) == 4                      # the top-level field wins
    for bad in (-1, True, 1.5, "8"):
        with pytest.raises(RequestError):
            thinking_budget_of({"chat_template_kwargs": {"thinking_budget": bad}})
    with pytest.raises(RequestError, match="disagree"):
        thinking_budget_of({"chat_template_kwargs": {"thinking_budget": 8,
                                                     "thinking_token_budget": 4}})
    codec = ChatCodec(ByteTokenizer(1024), context=512, model_name="m")
    p = codec.prepare({"messages": [{"role": "user", "content": "hi"}], "enable_thinking": True,
                       "chat_template_kwargs": {"thinking_budget": 0}},
                      {"thinking_token_budget": 512})
    assert p.thinking_budget == 0


def test_generation_config_supplies_the_sampling_defaults(tmp_path):
    import json
    from orinfer_b200.api.chat_codec import ChatCodec
    (tmp_path / "generation_config.json").write_text(json.dumps(
        {"eos_token_id": [258, 256], "do_sample": True, "temperature": 0.6, "top_p": 0.95,
         "top_k": 20, "repetition_penalty": 1.05}))
    codec = ChatCodec.load(tmp_path, 1024, 512, "m")
    msgs = [{"role": "user", "content": "hi"}]
    s = codec.prepare({"messages": msgs}).sampling
    assert (s.temperature, s.top_p, s.top_k, s.repetition_penalty) == (0.6, 0.95, 20, 1.05)
    s = codec.prepare({"messages": msgs, "temperature": 0, "top_k": -1}).sampling
    assert s.temperature == 0 and s.top_k == 0 and s.top_p == 0.95       # the request wins
    s = codec.prepare({"messages": msgs}, {"temperature": 0.2}).sampling
    assert s.temperature == 0.2                                          # then the deployment
    (tmp_path / "generation_config.json").write_text(json.dumps(
        {"do_sample": False, "temperature": 0.6, "top_k": 50}))
    s = ChatCodec.load(tmp_path, 1024, 512, "m").prepare({"messages": msgs}).sampling
    assert s.temperature == 0 and s.top_k == 50                          # greedy as shipped
