"""Grammar recipes that hold generated tool calls to the declared tools (JSON form inside
``<tool_call>...</tool_call>``).

When a recipe applies (the reference's rules, crates/orinfer-api/src/server/grammar.rs:245-340):

* ``tool_choice: "required"``            -> one or more calls, nothing else;
* ``tool_choice: {function: {name}}``    -> exactly that call;
* ``tool_choice: "auto"`` is constrained only when it has to be: a tool marked ``strict`` or
  ``parallel_tool_calls: false`` -> free text, then optionally call(s);
* ``tool_choice: "none"`` or no tools    -> no grammar.

Each call is ``{"name": "<declared name>", "arguments": <object matching the tool's schema>}``;
``parallel_tool_calls: false`` allows a single call.  The markers are written as token
references when the tokenizer has them as control tokens, so text can never spell them.
"""

from __future__ import annotations

import json
from typing import Any, List, Optional


def _marker(tokenizer, text: str) -> str:
    tid = tokenizer.token_id(text) if hasattr(tokenizer, "token_id") else None
    return f"<[{tid}]>" if tid is not None else json.dumps(text)


def _named(tool_choice: Any) -> Optional[str]:
    if isinstance(tool_choice, dict):
        return (tool_choice.get("function") or {}).get("name") or tool_choice.get("name")
    return None


def applies(tools: List[dict], tool_choice: Any, parallel: bool) -> bool:
    if not tools or tool_choice == "none":
        return False
    if tool_choice == "required" or _named(tool_choice):
        return True
    strict = any((t.get("function", t)).get("strict") for t in tools)
    return strict or not parallel


def recipe(tokenizer, tools: List[dict], tool_choice: Any = "auto", parallel: bool = True) -> str:
    """Lark text (llguidance dialect) for the constrained forms above."""
    named = _named(tool_choice)
    known = [t.get("function", t) for t in tools]
    if named is not None:
        known = [f for f in known if f.get("name") == named]
        if not known:
            raise ValueError(f"tool_choice names an undeclared tool `{named}`")
    rules, bodies = [], []
    for i, fn in enumerate(known):
        # compact JSON only: a model cannot pad its arguments with whitespace for ever
        schema = dict(fn.get("parameters") or {"type": "object"})
        schema["x-guidance"] = {"whitespace_flexible": False}
        rules.append(f'body_{i}: "{{\\"name\\": {json.dumps(json.dumps(fn["name"]))[1:-1]}, '
                     f'\\"arguments\\": " %json {json.dumps(schema)} "}}"')
        bodies.append(f"body_{i}")
    open_, close = _marker(tokenizer, "<tool_call>"), _marker(tokenizer, "</tool_call>")
    rules.append(f'call: {open_} "\\n" ({" | ".join(bodies)}) "\\n" {close} "\\n"?')
    calls = "call" if (named is not None or not parallel) else "call+"
    if tool_choice == "required" or named is not None:
        start = f"start: {calls}"
    else:
        start = f"start: TEXT ({calls})?"
        rules.append("TEXT: /(.|\\n)*/")
    return "\n".join([start, *rules])
