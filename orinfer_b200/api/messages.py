"""Normal form of a chat history before it reaches the template.

Clients send the same conversation in several wire shapes: content as a string, as ``null``
or as a list of text parts; tool-call arguments as the JSON *string* the OpenAI protocol
defines (templates want the mapping); ``developer`` beside ``system``.  ``normalize`` brings
them to one shape and refuses histories a template cannot render meaningfully:

* roles are ``system``, ``developer``, ``user``, ``assistant``, ``tool``; ``developer`` becomes
  ``system``; system messages precede the dialogue and are merged into one, joined by a blank
  line (``dsml`` histories keep them where they are);
* content becomes a string: ``null`` is ``""``, text parts are concatenated (``dsml``: joined
  by a blank line); a message that carries image parts keeps its part list for the image
  front end, with its text parts untouched;
* an assistant message's ``tool_calls`` need unique non-empty ids, type ``function`` and a name
  of at most 64 characters from ``[A-Za-z0-9_-]``; arguments given as a JSON string are parsed;
  what does not parse to an object is kept under ``__orinfer_raw_arguments`` (``dsml``:
  ``arguments``) so that a client can show the model its own malformed call;
* every tool call is answered by ``tool`` messages (by ``tool_call_id``) before the next
  non-tool message; a tool message that answers nothing is refused;
* there is at least one user message.

Behavioural contract: crates/orinfer-api/src/server/chat.rs:894-1040 of the reference; its
protocol vectors (tool results as text parts, empty parts, developer + system) are restated in
``tests/test_api_units.py``.
"""

from __future__ import annotations

import json
import re
from typing import Any, Dict, List

ROLES = ("system", "developer", "user", "assistant", "tool")
RAW_ARGUMENTS = "__orinfer_raw_arguments"
_NAME = re.compile(r"^[A-Za-z0-9_-]{1,64}$")


class MessageError(ValueError):
    """The history is malformed; ``param`` names the offending field."""

    def __init__(self, message: str, param: str = "messages"):
        super().__init__(message)
        self.param = param


def _text(content: Any, separator: str, where: str):
    """-> a string, or the part list unchanged when it carries non-text (media) parts."""
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    if not isinstance(content, list):
        raise MessageError("message content must be a string, null or a list of parts", where)
    texts, media = [], False
    for part in content:
        if not isinstance(part, dict):
            raise MessageError("a content part must be an object", where)
        if part.get("type") == "text":
            if not isinstance(part.get("text"), str):
                raise MessageError("a text part needs `text`", where)
            texts.append(part["text"])
        else:
            media = True
    return content if media else separator.join(texts)


def _arguments(value: Any, dsml: bool) -> Dict[str, Any]:
    if isinstance(value, dict):
        return value
    if not isinstance(value, str):
        raise MessageError("tool call arguments must be a JSON string")
    try:
        parsed = json.loads(value)
        if dsml and isinstance(parsed, str):          # doubly encoded by some clients
            parsed = json.loads(parsed)
    except (ValueError, RecursionError):
        parsed = None
    if isinstance(parsed, dict):
        return parsed
    return {"arguments" if dsml else RAW_ARGUMENTS: value}


def normalize(messages: List[dict], tool_format: str = "xml") -> List[dict]:
    dsml = tool_format == "dsml"
    if not isinstance(messages, list) or not messages:
        raise MessageError("`messages` must be a non-empty array")
    pending, seen = set(), set()
    has_user = dialogue = False
    out: List[dict] = []
    for i, original in enumerate(messages):
        where = f"messages[{i}]"
        if not isinstance(original, dict) or original.get("role") not in ROLES:
            raise MessageError("invalid message role", where + ".role")
        m = dict(original)
        role = m["role"]
        if role in ("system", "developer"):
            if dialogue and not dsml:
                raise MessageError("system and developer messages must precede the dialogue",
                                   where + ".role")
            if not dsml:
                m["role"] = "system"
        else:
            dialogue = True
        has_user = has_user or role == "user"
        if role != "tool" and pending:
            raise MessageError("a tool call has no tool message answering it", where)
        m["content"] = _text(m.get("content"), "\n\n" if dsml else "", where + ".content")
        if dsml and "reasoning_content" not in m and "reasoning" in m:
            m["reasoning_content"] = m["reasoning"]
        if role == "tool":
            answered = m.get("tool_call_id")
            if not isinstance(answered, str):
                raise MessageError("a tool message needs `tool_call_id`", where + ".tool_call_id")
            if answered not in pending:
                raise MessageError("unknown or repeated `tool_call_id`", where + ".tool_call_id")
            pending.discard(answered)
        calls = m.get("tool_calls")
        if calls is not None:
            if role != "assistant":
                raise MessageError("only assistant messages carry `tool_calls`",
                                   where + ".tool_calls")
            if not isinstance(calls, list):
                raise MessageError("`tool_calls` must be an array", where + ".tool_calls")
            fixed = []
            for j, call in enumerate(calls):
                at = f"{where}.tool_calls[{j}]"
                fn = call.get("function") if isinstance(call, dict) else None
                cid = call.get("id") if isinstance(call, dict) else None
                if not isinstance(cid, str) or not cid or cid in seen:
                    raise MessageError("tool call ids must be unique non-empty strings",
                                       at + ".id")
                if call.get("type", "function") != "function" or not isinstance(fn, dict) \
                        or not isinstance(fn.get("name"), str) or not _NAME.match(fn["name"]):
                    raise MessageError("invalid assistant tool call", at)
                seen.add(cid)
                pending.add(cid)
                fixed.append(dict(call, type="function",
                                  function=dict(fn, arguments=_arguments(fn.get("arguments"),
                                                                         dsml))))
            m["tool_calls"] = fixed
        if (not dsml and m["role"] == "system" and out and out[0]["role"] == "system"
                and isinstance(m["content"], str) and isinstance(out[0]["content"], str)):
            out[0] = dict(out[0], content=out[0]["content"] + "\n\n" + m["content"])
        else:
            out.append(m)
    if pending:
        raise MessageError("a tool call has no tool message answering it")
    if not has_user:
        raise MessageError("the history needs at least one user message")
    return out
