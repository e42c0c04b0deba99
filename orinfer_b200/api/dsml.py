"""DSML tool-call wire syntax (DeepSeek-style models): incremental parser to OpenAI tool-call
deltas, renderer for assistant history, tool-result reordering, and the grammar text that
constrains generation to declared tools.

Syntax, as emitted by the model::

    <｜DSML｜ calls>
    <｜DSML｜ invoke name="edit">
    <｜DSML｜ parameter name="text" string="true">hello</｜DSML｜ parameter>
    <｜DSML｜ parameter name="count" string="false">3</｜DSML｜ parameter>
    </｜DSML｜ invoke>
    </｜DSML｜ calls>

The parser turns this into a stream of ``function.arguments`` JSON fragments without waiting
for the end of a value: string values are JSON-escaped piece by piece, and only a suffix that
could still be the start of the closing tag is withheld.  Duplicate parameters, missing
``string`` flags and text where a tag must stand are errors that end the call.  Behaviour
follows the reference's crates/orinfer-api/src/server/output/dsml.rs (events Begin /
Arguments / End), grammar/dsml.rs (recipe) and server/chat/deepseek.rs:4-45 (tool results are
put in the order of the assistant's ``tool_calls``).
"""

from __future__ import annotations

import json
from typing import Dict, List, Optional, Tuple

MARK = "｜DSML｜"
OPEN = "<｜DSML｜ calls>"
CLOSE = "</｜DSML｜ calls>"
INVOKE = "<｜DSML｜ invoke "
INVOKE_END = "</｜DSML｜ invoke>"
PARAMETER = "<｜DSML｜ parameter "
PARAMETER_END = "</｜DSML｜ parameter>"


class DsmlError(ValueError):
    pass


def _held_suffix(text: str, marker: str) -> int:
    """Length of the longest proper prefix of ``marker`` that ends ``text``."""
    for n in range(min(len(marker) - 1, len(text)), 0, -1):
        if text.endswith(marker[:n]):
            return n
    return 0


def _header(text: str) -> Optional[Tuple[int, Dict[str, str]]]:
    """Parse ``key="value" ...>`` at the start of ``text``: (consumed, attributes), or None
    while the closing ``>`` (outside quotes) has not arrived."""
    quoted, end = False, -1
    for i, ch in enumerate(text):
        if ch == '"':
            quoted = not quoted
        elif ch == ">" and not quoted:
            end = i
            break
    if end < 0:
        return None
    attrs: Dict[str, str] = {}
    rest = text[:end].strip()
    while rest:
        key, eq, tail = rest.partition('="')
        key = key.strip()
        if not eq or not key or any(c in key for c in '<>"'):
            raise DsmlError("invalid DSML attribute")
        value, quote, rest = tail.partition('"')
        if not quote:
            raise DsmlError("invalid DSML attributes")
        if key in attrs:
            raise DsmlError("duplicate DSML attribute")
        attrs[key] = value
        rest = rest.strip()
    return end + 1, attrs


class DsmlCalls:
    """State machine over the text after ``OPEN``.  ``feed`` returns events
    ``("begin", name)``, ``("arguments", fragment)``, ``("end",)`` and ``("close",)`` (the
    block ended); unconsumed text stays buffered until more arrives."""

    def __init__(self):
        self.buffer = ""
        self.stage = "invoke"        # invoke | parameter | value | done
        self.string = False
        self.seen: set = set()
        self.done = False

    def feed(self, text: str) -> List[tuple]:
        self.buffer += text
        events: List[tuple] = []
        while not self.done:
            before = (len(self.buffer), self.stage, len(events))
            self._step(events)
            if (len(self.buffer), self.stage, len(events)) == before:
                break
        return events

    def _expect(self, options: List[str]) -> Optional[str]:
        """The option that starts the buffer (after whitespace); None if more text is needed."""
        rest = self.buffer.lstrip()
        for opt in options:
            if rest.startswith(opt):
                self.buffer = rest[len(opt):]
                return opt
        if any(opt.startswith(rest) for opt in options):
            return None
        raise DsmlError("expected " + " or ".join(o.strip() for o in options))

    def _step(self, events: List[tuple]) -> None:
        if self.stage == "invoke":
            hit = self._expect([INVOKE, CLOSE])
            if hit == CLOSE:
                self.done = True
                events.append(("close",))
            elif hit == INVOKE:
                self.stage = "invoke-header"
        elif self.stage == "invoke-header":
            got = _header(self.buffer)
            if got is None:
                return
            n, attrs = got
            name = attrs.get("name")
            if not name:
                raise DsmlError("missing DSML function name")
            self.buffer = self.buffer[n:]
            self.seen = set()
            events.append(("begin", name))
            events.append(("arguments", "{"))
            self.stage = "parameter"
        elif self.stage == "parameter":
            hit = self._expect([PARAMETER, INVOKE_END])
            if hit == INVOKE_END:
                events.append(("arguments", "}"))
                events.append(("end",))
                self.stage = "invoke"
            elif hit == PARAMETER:
                self.stage = "parameter-header"
        elif self.stage == "parameter-header":
            got = _header(self.buffer)
            if got is None:
                return
            n, attrs = got
            key, flag = attrs.get("name"), attrs.get("string")
            if flag not in ("true", "false"):
                raise DsmlError("DSML parameter requires string=true or false")
            if not key or key in self.seen:
                raise DsmlError("empty or duplicate DSML parameter")
            first = not self.seen
            self.seen.add(key)
            self.string = flag == "true"
            self.buffer = self.buffer[n:]
            events.append(("arguments", ("" if first else ",") + json.dumps(key) + ":" +
                           ('"' if self.string else "")))
            self.stage = "value"
        elif self.stage == "value":
            end = self.buffer.find(PARAMETER_END)
            count = end if end >= 0 else len(self.buffer) - _held_suffix(self.buffer,
                                                                         PARAMETER_END)
            piece, self.buffer = self.buffer[:count], self.buffer[count:]
            if piece:
                events.append(("arguments", json.dumps(piece, ensure_ascii=False)[1:-1]
                               if self.string else piece))
            if end >= 0:
                self.buffer = self.buffer[len(PARAMETER_END):]
                if self.string:
                    events.append(("arguments", '"'))
                self.stage = "parameter"


def parse_calls(text: str) -> List[dict]:
    """All calls of a complete DSML block (text after ``OPEN``): [{name, arguments}]."""
    calls: List[dict] = []
    for ev in DsmlCalls().feed(text):
        if ev[0] == "begin":
            calls.append({"name": ev[1], "arguments": ""})
        elif ev[0] == "arguments":
            calls[-1]["arguments"] += ev[1]
    return calls


def render_calls(tool_calls: List[dict], mark: str = MARK) -> str:
    """Assistant history -> wire text.  String arguments are written raw with
    ``string="true"``; everything else as JSON with ``string="false"``.  ``mark`` stands for
    the ``｜DSML｜`` control spelling (a private handle when control tokens are protected)."""
    out = [f"<{mark} calls>"]
    for call in tool_calls:
        fn = call.get("function", call)
        args = fn.get("arguments") or {}
        if isinstance(args, str):
            args = json.loads(args) if args.strip() else {}
        out.append(f'<{mark} invoke name="{fn["name"]}">')
        for key, value in args.items():
            if isinstance(value, str):
                out.append(f'<{mark} parameter name="{key}" string="true">{value}'
                           f'</{mark} parameter>')
            else:
                out.append(f'<{mark} parameter name="{key}" string="false">'
                           f'{json.dumps(value, ensure_ascii=False)}</{mark} parameter>')
        out.append(f"</{mark} invoke>")
    out.append(f"</{mark} calls>")
    return "\n".join(out)


def reorder_tool_results(messages: List[dict]) -> List[dict]:
    """Tool messages that follow an assistant turn are put in the order of that turn's
    ``tool_calls`` (matched by ``tool_call_id``); unmatched results keep their relative order
    after the matched ones.  Other messages are untouched."""
    out: List[dict] = []
    i = 0
    while i < len(messages):
        m = messages[i]
        out.append(m)
        i += 1
        if m.get("role") != "assistant" or not m.get("tool_calls"):
            continue
        j = i
        while j < len(messages) and messages[j].get("role") == "tool":
            j += 1
        results = messages[i:j]
        order = {c.get("id"): k for k, c in enumerate(m["tool_calls"])}
        ranked = sorted(enumerate(results),
                        key=lambda t: (order.get(t[1].get("tool_call_id"), len(order)), t[0]))
        out.extend(r for _, r in ranked)
        i = j
    return out


def grammar(tools: List[dict], required: bool = False, parallel: bool = True) -> str:
    """Lark text (llguidance dialect) for an optional free-text answer followed by one DSML
    block whose invokes name declared tools and whose parameters name declared properties;
    string-typed properties take raw text, the others JSON values."""
    rules = []
    invokes = []
    for t, tool in enumerate(tools):
        fn = tool.get("function", tool)
        props = (fn.get("parameters") or {}).get("properties") or {}
        params = []
        for p, (key, schema) in enumerate(props.items()):
            is_string = schema.get("type") == "string"
            body = "RAW" if is_string else "%json " + json.dumps(schema)
            rules.append(f'p_{t}_{p}: "{PARAMETER}name=\\"{key}\\" string=\\"'
                         f'{"true" if is_string else "false"}\\">" {body} "{PARAMETER_END}" "\\n"')
            params.append(f"p_{t}_{p}")
        inner = ("(" + " | ".join(params) + ")*") if params else ""
        rules.append(f'invoke_{t}: "{INVOKE}name=\\"{fn["name"]}\\">" "\\n" {inner} '
                     f'"{INVOKE_END}" "\\n"')
        invokes.append(f"invoke_{t}")
    one = "(" + " | ".join(invokes) + ")"
    block = f'"{OPEN}" "\\n" {one}{"+" if parallel else ""} "{CLOSE}"'
    start = f"start: {block}" if required else f"start: TEXT ({block})?"
    return "\n".join([start, *rules, 'TEXT: /[^<]*/', 'RAW: /[^<]*/'])
