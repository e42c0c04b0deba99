"""DSML tool-call syntax: streaming parser, renderer, reordering, grammar, parser integration."""
import json

import pytest

from orinfer_b200.api import dsml
from orinfer_b200.api.output_parser import OutputParser, merge_tool_calls

BLOCK = ('\n<｜DSML｜ invoke name="edit">\n'
         '<｜DSML｜ parameter name="text" string="true">say "hi"\nnow</｜DSML｜ parameter>\n'
         '<｜DSML｜ parameter name="count" string="false">3</｜DSML｜ parameter>\n'
         '<｜DSML｜ parameter name="flags" string="false">{"a": [1, 2]}</｜DSML｜ parameter>\n'
         '</｜DSML｜ invoke>\n'
         '<｜DSML｜ invoke name="noop">\n</｜DSML｜ invoke>\n'
         '</｜DSML｜ calls>')


def test_whole_block_and_every_split_give_the_same_calls():
    calls = dsml.parse_calls(BLOCK)
    assert [c["name"] for c in calls] == ["edit", "noop"]
    assert json.loads(calls[0]["arguments"]) == {"text": 'say "hi"\nnow', "count": 3,
                                                 "flags": {"a": [1, 2]}}
    assert calls[1]["arguments"] == "{}"
    for cut in range(1, len(BLOCK)):
        m = dsml.DsmlCalls()
        events = m.feed(BLOCK[:cut]) + m.feed(BLOCK[cut:])
        args = "".join(e[1] for e in events if e[0] == "arguments")
        assert args == calls[0]["arguments"] + "{}" and events[-1] == ("close",), cut
    m = dsml.DsmlCalls()
    stream = [e for ch in BLOCK for e in m.feed(ch)]                # one character at a time
    assert "".join(e[1] for e in stream if e[0] == "arguments") == calls[0]["arguments"] + "{}"


def test_values_stream_before_their_closing_tag():
    m = dsml.DsmlCalls()
    ev = m.feed('<｜DSML｜ invoke name="w">\n<｜DSML｜ parameter name="t" string="true">abc</｜DS')
    assert ev == [("begin", "w"), ("arguments", "{"), ("arguments", '"t":"'), ("arguments", "abc")]
    assert m.feed("ML｜ parameter>") == [("arguments", '"')]


@pytest.mark.parametrize("bad, why", [
    ('<｜DSML｜ invoke name="a">\n<｜DSML｜ parameter name="x">1', "string=true or false"),
    ('<｜DSML｜ invoke name="a">\n<｜DSML｜ parameter name="x" string="false">1</｜DSML｜ parameter>'
     '<｜DSML｜ parameter name="x" string="false">2', "duplicate"),
    ('<｜DSML｜ invoke >', "function name"),
    ('hello', "expected"),
    ('<｜DSML｜ invoke name="a" name="b">', "duplicate DSML attribute"),
])
def test_malformed_blocks_are_errors(bad, why):
    with pytest.raises(dsml.DsmlError, match=why):
        dsml.DsmlCalls().feed(bad)


def test_render_round_trip_and_result_reordering():
    calls = [{"id": "c1", "function": {"name": "edit",
                                       "arguments": json.dumps({"text": "a<b", "n": 2})}},
             {"id": "c2", "function": {"name": "noop", "arguments": ""}}]
    text = dsml.render_calls(calls)
    assert text.startswith(dsml.OPEN) and text.endswith(dsml.CLOSE)
    back = dsml.parse_calls(text[len(dsml.OPEN):])
    assert json.loads(back[0]["arguments"]) == {"text": "a<b", "n": 2} and back[1]["name"] == "noop"
    msgs = [{"role": "user", "content": "go"},
            {"role": "assistant", "tool_calls": calls},
            {"role": "tool", "tool_call_id": "c2", "content": "two"},
            {"role": "tool", "tool_call_id": "zz", "content": "stray"},
            {"role": "tool", "tool_call_id": "c1", "content": "one"},
            {"role": "user", "content": "next"}]
    out = dsml.reorder_tool_results(msgs)
    assert [m.get("content") for m in out[2:5]] == ["one", "two", "stray"]
    assert out[0] is msgs[0] and out[5] is msgs[5] and len(out) == 6


def test_output_parser_streams_dsml_calls():
    text = "Let me edit." + dsml.OPEN + BLOCK + " done"
    for step in (1, 7, len(text)):
        p = OutputParser(tool_format="dsml")
        content, deltas = "", []
        for i in range(0, len(text), step):
            d = p.feed(text[i:i + step], final=i + step >= len(text))
            content += d.content
            deltas += d.tool_calls
        assert content == "Let me edit. done", step
        calls = merge_tool_calls(deltas)
        assert [c["function"]["name"] for c in calls] == ["edit", "noop"]
        assert json.loads(calls[0]["function"]["arguments"])["count"] == 3
        assert calls[0]["id"] == "call_0" and calls[1]["id"] == "call_1"
        assert p.finish_reason("stop") == "tool_calls"
    p = OutputParser(tool_format="dsml")
    d = p.feed("x" + dsml.OPEN + "garbage", final=True)
    assert d.content == "x" and p.stopped and "expected" in p.error
    xml = OutputParser()                                            # other formats untouched
    d = xml.feed('<tool_call>{"name": "f", "arguments": {"a": 1}}</tool_call>', final=True)
    assert merge_tool_calls(d.tool_calls)[0]["function"] == {"name": "f", "arguments": '{"a": 1}'}


TOOLS = [{"type": "function", "function": {"name": "edit", "parameters": {
    "type": "object", "properties": {"text": {"type": "string"}, "count": {"type": "integer"}}}}}]


def test_grammar_accepts_declared_calls_only():
    llguidance = pytest.importorskip("llguidance")
    from orinfer_b200.api.chat_codec import ByteTokenizer
    from orinfer_b200.api.grammar import GrammarConstraint
    tok = ByteTokenizer(1024)

    def accepts(text, **kw):
        c = GrammarConstraint.from_lark(tok, 1024, dsml.grammar(TOOLS, **kw), tok.eos_ids)
        try:
            for t in tok.encode(text):
                mask = c.mask(1024)
                if not (mask[t // 32] >> (t % 32)) & 1:
                    return False
                c.consume(t)
        except Exception:
            return False
        return bool(c.m.is_accepting())

    good = (dsml.OPEN + '\n<｜DSML｜ invoke name="edit">\n'
            '<｜DSML｜ parameter name="count" string="false">3</｜DSML｜ parameter>\n'
            '<｜DSML｜ parameter name="text" string="true">hi</｜DSML｜ parameter>\n'
            '</｜DSML｜ invoke>\n' + dsml.CLOSE)
    assert accepts(good, required=True)
    assert accepts("Just an answer.") and not accepts("Just an answer.", required=True)
    assert not accepts(good.replace('name="edit"', 'name="rm"'), required=True)
    assert not accepts(good.replace(">3<", ">three<"), required=True)
    assert not accepts(good.replace('name="count"', 'name="other"'), required=True)


def test_codec_renders_history_in_wire_syntax():
    from orinfer_b200.api.chat_codec import ByteTokenizer, ChatCodec
    codec = ChatCodec(ByteTokenizer(1024), context=4096)
    codec.tool_format = "dsml"
    p = codec.prepare({"messages": [
        {"role": "user", "content": "go"},
        {"role": "assistant", "content": "ok", "tool_calls": [
            {"id": "a", "type": "function", "function": {"name": "edit",
                                                         "arguments": '{"text": "x"}'}},
            {"id": "b", "type": "function", "function": {"name": "edit",
                                                         "arguments": '{"count": 1}'}}]},
        {"role": "tool", "tool_call_id": "b", "content": "second"},
        {"role": "tool", "tool_call_id": "a", "content": "first"}], "tools": TOOLS})
    text = p.prompt_text
    assert dsml.OPEN in text and "<tool_call>" not in text
    assert text.index("first") < text.index("second")
