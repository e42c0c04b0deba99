"""Control-token provenance: only the chat template and the server itself can place control
tokens in a prompt; the same spelling inside user text is tokenised as plain characters.

How: every control-token spelling in the *template source* is replaced by a private handle
(a per-process random prefix + the token id) before the template is compiled.  Request values
go through the template as data, so after rendering a handle can only come from the template
source or from ``control()`` (server-created delimiters such as media placeholders); a literal
copy of the private prefix inside request data is escaped first.  ``encode`` then splits the
rendered text at the handles: handles become their token ids, the plain regions are encoded by
a tokenizer that knows no control tokens (cached, since system prompts and histories repeat).
This is the scheme of the reference's crates/orinfer-api/src/server/token_boundary.rs:11-180
(private nonce prefix, ``template`` / ``control`` / ``escape_value`` / ``encode``, 64 MiB cache
of plain-region tokenisations, output controls ``<think>`` ``</think>`` ``｜DSML｜``).
"""

from __future__ import annotations

import json
import re
import secrets
from collections import OrderedDict
from typing import Any, Dict, List, Optional

OUTPUT_CONTROLS = ("<think>", "</think>", "｜DSML｜")


class BoundaryError(ValueError):
    pass


def plain_encoder(tokenizer):
    """``text -> ids`` that never yields a control token."""
    if hasattr(tokenizer, "encode_plain"):
        return tokenizer.encode_plain
    if hasattr(tokenizer, "tk"):                      # tokenizers.Tokenizer: drop added vocabulary
        from tokenizers import Tokenizer
        spec = json.loads(tokenizer.tk.to_str())
        spec["added_tokens"] = []
        plain = Tokenizer.from_str(json.dumps(spec))
        return lambda text: plain.encode(text, add_special_tokens=False).ids
    raise BoundaryError("tokenizer offers no plain encoding")


def control_vocabulary(tokenizer) -> Dict[str, int]:
    if hasattr(tokenizer, "special_ids"):
        return dict(tokenizer.special_ids)
    if hasattr(tokenizer, "tk"):
        spec = json.loads(tokenizer.tk.to_str())
        return {t["content"]: t["id"] for t in spec.get("added_tokens", [])}
    return {}


class Boundary:
    def __init__(self, tokenizer, cache_bytes: int = 64 << 20):
        self.tokens = control_vocabulary(tokenizer)
        self._plain = plain_encoder(tokenizer)
        self.prefix = f"__orinfer_control_{secrets.token_hex(16)}_"
        self._split = re.compile(re.escape(self.prefix) + r"(\d+|p);")
        self.output = {i: s for s, i in self.tokens.items() if s in OUTPUT_CONTROLS}
        self._cache: "OrderedDict[str, List[int]]" = OrderedDict()
        self._cache_bytes, self._budget = 0, cache_bytes
        self.hits = self.misses = 0

    # ---- building the prompt ---------------------------------------------------------
    def control(self, spelling: str) -> str:
        """Handle for a control token the server itself inserts."""
        if spelling not in self.tokens:
            raise BoundaryError(f"missing template control token: {spelling}")
        return f"{self.prefix}{self.tokens[spelling]};"

    def controls(self, text: str) -> str:
        """Handles for every control spelling in server-written ``text``."""
        return self.template(text)

    def escape(self, text: str) -> str:
        return text.replace(self.prefix, self.prefix + "p;")

    def template(self, source: str) -> str:
        """Template source with every control spelling replaced by its handle."""
        source = self.escape(source)
        for spelling in sorted(self.tokens, key=len, reverse=True):
            source = source.replace(spelling, f"{self.prefix}{self.tokens[spelling]};")
        return source

    def escape_value(self, value: Any) -> Any:
        """Request data with literal copies of the private prefix defused (object keys too)."""
        if isinstance(value, str):
            return self.escape(value) if self.prefix in value else value
        if isinstance(value, list):
            return [self.escape_value(v) for v in value]
        if isinstance(value, dict):
            return {self.escape_value(k): self.escape_value(v) for k, v in value.items()}
        return value

    # ---- encoding ----------------------------------------------------------------------
    def encode(self, rendered: str) -> List[int]:
        ids: List[int] = []
        pos = 0
        pending = ""
        for m in self._split.finditer(rendered):
            pending += rendered[pos:m.start()]
            pos = m.end()
            if m.group(1) == "p":                     # an escaped literal prefix: still text
                pending += self.prefix
                continue
            ids += self._encode_plain(pending)
            pending = ""
            ids.append(int(m.group(1)))
        ids += self._encode_plain(pending + rendered[pos:])
        return ids

    def _encode_plain(self, text: str) -> List[int]:
        if not text:
            return []
        hit = self._cache.get(text)
        if hit is not None:
            self._cache.move_to_end(text)
            self.hits += 1
            return hit
        self.misses += 1
        ids = list(self._plain(text))
        cost = len(text.encode("utf-8")) + 4 * len(ids) + 64
        if cost <= self._budget:
            self._cache[text] = ids
            self._cache_bytes += cost
            while self._cache_bytes > self._budget:
                old, old_ids = self._cache.popitem(last=False)
                self._cache_bytes -= len(old.encode("utf-8")) + 4 * len(old_ids) + 64
        return ids

    def output_control(self, token_id: int) -> Optional[str]:
        """Spelling of a generated control token that may switch the output parser's state;
        the same characters produced as ordinary text tokens do not."""
        return self.output.get(token_id)

    def cache_statistics(self) -> dict:
        return {"entries": len(self._cache), "bytes": self._cache_bytes, "hits": self.hits,
                "misses": self.misses}
