"""Incremental output parser: token text -> OpenAI deltas.

Splits generated text into ``reasoning_content`` (inside ``<think>...</think>``),
``content`` and ``tool_calls`` (``<tool_call>...</tool_call>`` holding either JSON
``{"name":..., "arguments":...}`` or the XML form
``<function=NAME><parameter=KEY>VALUE</parameter></function>``), applies stop strings,
and withholds the longest suffix that could still become a marker or a stop string so a
client never sees half a tag.  Finish reasons rank ``length`` > ``tool_calls`` > ``stop``.
Behaviour follows crates/orinfer-api/src/server/output.rs:154-343,382-475 of the reference.
"""

from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional

THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
TOOL_OPEN, TOOL_CLOSE = "<tool_call>", "</tool_call>"
DSML_OPEN = "<｜DSML｜ calls>"


def merge_tool_calls(deltas: List[dict]) -> List[dict]:
    """Fold streamed tool-call deltas (same ``index``) into whole calls."""
    calls: Dict[int, dict] = {}
    for d in deltas:
        fn = d.get("function") or {}
        cur = calls.get(d["index"])
        if cur is None:
            cur = calls[d["index"]] = {"id": d.get("id"), "type": d.get("type", "function"),
                                       "function": {"name": fn.get("name", ""), "arguments": ""}}
        elif fn.get("name"):
            cur["function"]["name"] = fn["name"]
        cur["function"]["arguments"] += fn.get("arguments") or ""
    return [calls[i] for i in sorted(calls)]


@dataclass
class Delta:
    content: str = ""
    reasoning: str = ""
    tool_calls: List[dict] = field(default_factory=list)

    def empty(self) -> bool:
        return not (self.content or self.reasoning or self.tool_calls)


def _partial_suffix(text: str, markers: List[str]) -> int:
    """Length of the longest suffix of ``text`` that is a proper prefix of a marker."""
    best = 0
    for m in markers:
        for n in range(min(len(m) - 1, len(text)), 0, -1):
            if text.endswith(m[:n]):
                best = max(best, n)
                break
    return best


def parse_tool_call(body: str) -> Optional[dict]:
    body = body.strip()
    if body.startswith("{"):
        try:
            obj = json.loads(body)
        except json.JSONDecodeError:
            return None
        if not isinstance(obj, dict) or "name" not in obj:
            return None
        args = obj.get("arguments", {})
        return {"name": str(obj["name"]),
                "arguments": args if isinstance(args, str) else json.dumps(args,
                                                                           ensure_ascii=False)}
    m = re.match(r"<function=([^>]+)>(.*)</function>\s*$", body, re.S)
    if not m:
        return None
    args: Dict[str, object] = {}
    for key, val in re.findall(r"<parameter=([^>]+)>\n?(.*?)\n?</parameter>", m.group(2), re.S):
        try:
            args[key] = json.loads(val)
        except json.JSONDecodeError:
            args[key] = val
    return {"name": m.group(1).strip(), "arguments": json.dumps(args, ensure_ascii=False)}


class OutputParser:
    def __init__(self, thinking: bool = False, stops: Optional[List[str]] = None,
                 json_mode: bool = False, tools: bool = True, tool_format: str = "xml"):
        # tool_format "dsml": calls arrive as a DSML block and their arguments are streamed
        # as JSON fragments while the values are still being generated (api/dsml.py)
        self.tool_format = tool_format
        self.dsml = None
        self.error: Optional[str] = None
        self.in_think = thinking            # template already opened <think>
        self.stops = list(stops or [])
        self.json_mode = json_mode          # tags inside a JSON body are data
        self.tools_enabled = tools and not json_mode
        self.buffer = ""
        self.in_tool = False
        self.tool_text = ""
        self.tool_index = 0
        # a JSON call body `{"name": ..., "arguments": {...}}` is streamed: the name as soon
        # as it is complete, the arguments as raw fragments while they are generated
        self.call_stage = 0                 # 0 header, 1 inside the arguments, 2 after them
        self.call_seen = 0                  # characters of tool_text already scanned
        self.call_depth = 0
        self.call_string = self.call_escape = False
        self.stopped = False
        self.saw_tool_call = False
        self.reasoning_chars = 0

    def _markers(self) -> List[str]:
        if self.in_think:
            return [THINK_CLOSE]
        if self.in_tool:
            return [TOOL_CLOSE]
        m = list(self.stops)
        if not self.json_mode:
            m.append(THINK_OPEN)
            if self.tools_enabled:
                m.append(DSML_OPEN if self.tool_format == "dsml" else TOOL_OPEN)
        return m

    def feed(self, text: str, final: bool = False) -> Delta:
        """Consume generated text; returns what may be shown now."""
        delta = Delta()
        if self.stopped:
            return delta
        self.buffer += text
        while True:
            if self.dsml is not None:
                if not self._feed_dsml(delta):
                    break
                continue
            markers = self._markers()
            hit_pos, hit = -1, None
            for m in markers:
                p = self.buffer.find(m)
                if p >= 0 and (hit_pos < 0 or p < hit_pos):
                    hit_pos, hit = p, m
            if hit is None:
                hold = 0 if final else _partial_suffix(self.buffer, markers)
                emit, self.buffer = self.buffer[:len(self.buffer) - hold], \
                    self.buffer[len(self.buffer) - hold:]
                self._emit(delta, emit)
                break
            self._emit(delta, self.buffer[:hit_pos])
            self.buffer = self.buffer[hit_pos + len(hit):]
            if hit == THINK_CLOSE:
                self.in_think = False
            elif hit == THINK_OPEN:
                self.in_think = True
            elif hit == DSML_OPEN and self.tool_format == "dsml":
                from .dsml import DsmlCalls
                self.dsml = DsmlCalls()
            elif hit == TOOL_OPEN:
                self.in_tool, self.tool_text = True, ""
                self.call_stage = self.call_seen = self.call_depth = 0
                self.call_string = self.call_escape = False
            elif hit == TOOL_CLOSE:
                self.in_tool = False
                if self.call_stage:         # streamed: name and arguments are out already
                    self.tool_index += 1
                    continue
                call = parse_tool_call(self.tool_text)
                if call is not None:
                    self.saw_tool_call = True
                    delta.tool_calls.append({
                        "index": self.tool_index, "id": f"call_{self.tool_index}",
                        "type": "function", "function": call})
                    self.tool_index += 1
                else:                       # malformed call is shown as text
                    delta.content += TOOL_OPEN + self.tool_text + TOOL_CLOSE
            else:                           # a stop string
                self.stopped = True
                self.buffer = ""
                break
        if final and self.in_tool:
            # an unfinished call at the end of generation is returned as plain text, unless
            # its name went out already: then it stays a call with truncated arguments
            if self.call_stage:
                self.tool_index += 1
            else:
                delta.content += TOOL_OPEN + self.tool_text
            self.in_tool = False
        return delta

    _CALL_HEAD = re.compile(r'\s*\{\s*"name"\s*:\s*("(?:[^"\\]|\\.)*")\s*,\s*"arguments"\s*:\s*(?=\S)')

    def _stream_call(self, delta: Delta) -> None:
        """Advance the streamed form of the call body collected in ``tool_text``."""
        if self.call_stage == 0:
            m = self._CALL_HEAD.match(self.tool_text)
            if m is None or self.tool_text[m.end()] != "{":
                return                      # not (yet) `{"name": "...", "arguments": {`
            try:
                name = json.loads(m.group(1))
            except json.JSONDecodeError:
                return
            self.saw_tool_call = True
            delta.tool_calls.append({"index": self.tool_index, "id": f"call_{self.tool_index}",
                                     "type": "function",
                                     "function": {"name": str(name), "arguments": ""}})
            self.call_stage, self.call_seen = 1, m.end()
        if self.call_stage != 1:
            return
        start = i = self.call_seen
        text = self.tool_text
        while i < len(text):
            ch = text[i]
            i += 1
            if self.call_string:
                if self.call_escape:
                    self.call_escape = False
                elif ch == "\\":
                    self.call_escape = True
                elif ch == '"':
                    self.call_string = False
            elif ch == '"':
                self.call_string = True
            elif ch == "{":
                self.call_depth += 1
            elif ch == "}":
                self.call_depth -= 1
                if self.call_depth == 0:
                    self.call_stage = 2
                    break
        self.call_seen = i
        if i > start:
            delta.tool_calls.append({"index": self.tool_index,
                                     "function": {"arguments": text[start:i]}})

    def _feed_dsml(self, delta: Delta) -> bool:
        """Run the buffered text through the DSML state machine; True when the block closed
        and ordinary parsing resumes."""
        from .dsml import DsmlError
        text, self.buffer = self.buffer, ""
        try:
            events = self.dsml.feed(text)
        except DsmlError as e:
            self.error = str(e)             # a malformed block ends the visible output
            self.stopped = True
            self.dsml = None
            return False
        for ev in events:
            if ev[0] == "begin":
                self.saw_tool_call = True
                delta.tool_calls.append({"index": self.tool_index, "id": f"call_{self.tool_index}",
                                         "type": "function",
                                         "function": {"name": ev[1], "arguments": ""}})
            elif ev[0] == "arguments":
                delta.tool_calls.append({"index": self.tool_index,
                                         "function": {"arguments": ev[1]}})
            elif ev[0] == "end":
                self.tool_index += 1
            elif ev[0] == "close":
                self.buffer, self.dsml = self.dsml.buffer, None
                return True
        return False

    def _emit(self, delta: Delta, text: str) -> None:
        if not text:
            return
        if self.in_tool:
            self.tool_text += text
            self._stream_call(delta)
        elif self.in_think:
            delta.reasoning += text
            self.reasoning_chars += len(text)
        else:
            delta.content += text

    def finish_reason(self, engine_reason: str) -> str:
        if engine_reason == "length":
            return "length"
        if self.saw_tool_call:
            return "tool_calls"
        return "stop"
