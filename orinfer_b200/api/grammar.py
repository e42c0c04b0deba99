"""Token-level constraints for decoding: JSON schema / JSON object grammars through
``llguidance`` and the thinking-budget constraint.

A constraint offers ``mask(vocab) -> uint32 bit words or None``, ``consume(token)``,
``finished()`` and ``fork()`` (speculative branches commit only accepted tokens), the
contract of the reference's ``Constraint`` trait
(crates/orinfer-engine/src/sampling/constrained.rs:8-19).  Grammar recipes follow
crates/orinfer-api/src/server/grammar.rs:245-340: an optional free-form thinking prefix
up to ``</think>``, then the JSON body; the end-of-sequence token is the only legal token
once the body is complete.
"""

from __future__ import annotations

import json
from typing import List, Optional, Sequence

import numpy as np


class GrammarError(ValueError):
    pass


class _TokTable:
    """Adapter giving llguidance the byte string of every token id."""

    def __init__(self, tokenizer, vocab: int):
        self.tokens = [tokenizer.token_bytes(i) or b"" for i in range(vocab)]
        eos = list(getattr(tokenizer, "eos_ids", ()) or ())
        self.eos_token_id = eos[0] if eos else vocab - 1
        self.bos_token_id = None
        from .token_boundary import BoundaryError, control_vocabulary, plain_encoder
        specials = [i for i in control_vocabulary(tokenizer).values() if 0 <= i < vocab]
        for i in specials:
            self.tokens[i] = b"\xff" + self.tokens[i]              # never matched as text
        self.special_token_ids = specials
        # text the grammar forces (constants, keys) is tokenised as plain characters: a
        # constant that spells a control token must not come back as that token
        try:
            self._encode = plain_encoder(tokenizer)
        except BoundaryError:
            self._encode = tokenizer.encode

    def __call__(self, s):
        if isinstance(s, bytes):
            s = s.decode("utf-8", errors="replace")
        return self._encode(s)


_TOKENIZERS = {}


def ll_tokenizer(tokenizer, vocab: int):
    import llguidance
    key = (id(tokenizer), vocab)
    if key not in _TOKENIZERS:
        _TOKENIZERS[key] = llguidance.LLTokenizer(llguidance.TokenizerWrapper(
            _TokTable(tokenizer, vocab)))
    return _TOKENIZERS[key]


class GrammarConstraint:
    """JSON-schema (or any-JSON) constrained decoding."""

    def __init__(self, tokenizer, vocab: int, schema: Optional[dict], eos_ids: Sequence[int],
                 _matcher=None):
        import llguidance
        self.vocab = vocab
        self.eos_ids = tuple(eos_ids)
        self._tok = tokenizer
        self._schema = schema
        if _matcher is None:
            body = schema if schema is not None else {"type": "object"}
            grammar = llguidance.LLMatcher.grammar_from_json_schema(
                json.dumps(body), defaults={"whitespace_flexible": False})
            err = llguidance.LLMatcher.validate_grammar(grammar)
            if err:
                raise GrammarError(f"unsupported JSON schema: {err}")
            _matcher = llguidance.LLMatcher(ll_tokenizer(tokenizer, vocab), grammar)
            if _matcher.is_error():
                raise GrammarError(_matcher.get_error())
        self.m = _matcher
        self.words = (vocab + 31) // 32
        self.done = False

    @classmethod
    def from_lark(cls, tokenizer, vocab: int, lark: str, eos_ids: Sequence[int]
                  ) -> "GrammarConstraint":
        """Constraint from grammar text in llguidance's Lark dialect (tool-call syntaxes)."""
        import llguidance
        grammar = llguidance.LLMatcher.grammar_from_lark(lark)
        err = llguidance.LLMatcher.validate_grammar(grammar)
        if err:
            raise GrammarError(f"invalid grammar: {err}")
        m = llguidance.LLMatcher(ll_tokenizer(tokenizer, vocab), grammar)
        if m.is_error():
            raise GrammarError(m.get_error())
        return cls(tokenizer, vocab, None, eos_ids, _matcher=m)

    def needs_mask(self) -> bool:
        return True

    def mask(self, vocab: int) -> np.ndarray:
        buf = np.zeros((1, self.words), dtype=np.int32)
        if self.done or self.m.is_stopped():
            out = buf[0].view(np.uint32)
            for e in self.eos_ids:
                out[e // 32] |= np.uint32(1 << (e % 32))
            return out
        self.m.unsafe_compute_mask_ptr(buf.ctypes.data, buf.size * 4)
        out = buf[0].view(np.uint32).copy()
        if self.m.is_accepting():
            for e in self.eos_ids:
                out[e // 32] |= np.uint32(1 << (e % 32))
        if not out.any():
            raise GrammarError("grammar permits no tokens")
        return out

    def consume(self, token: int) -> None:
        if token in self.eos_ids:
            self.done = True
            return
        if not self.m.consume_token(int(token)):
            raise GrammarError(self.m.get_error() or "token rejected by the grammar")

    def finished(self) -> bool:
        return self.done

    def fork(self) -> "GrammarConstraint":
        c = GrammarConstraint(self._tok, self.vocab, self._schema, self.eos_ids,
                              _matcher=self.m.deep_copy())
        c.done = self.done
        return c


class ThinkingBudget:
    """Forces ``</think>`` once ``budget`` thinking tokens were produced, always leaving
    room for at least one answer token (crates/orinfer-api/src/server/thinking.rs:5-120).
    Wraps an optional inner constraint that starts after the thinking section."""

    def __init__(self, close_ids: Sequence[int], budget: int, max_new: int, inner=None):
        self.close = list(close_ids)                # token ids spelling "</think>"
        self.budget = max(0, min(budget, max_new - len(self.close) - 1))
        self.inner = inner
        self.used = 0
        self.closing = 0                            # how many close tokens were forced
        self.closed = False
        self._seen: List[int] = []

    def needs_mask(self) -> bool:
        return (not self.closed and self.used >= self.budget) or \
            (self.closed and self.inner is not None)

    def mask(self, vocab: int) -> Optional[np.ndarray]:
        if self.closed:
            return self.inner.mask(vocab) if self.inner is not None else None
        if self.used >= self.budget or self.closing:
            out = np.zeros((vocab + 31) // 32, dtype=np.uint32)
            t = self.close[self.closing]
            out[t // 32] |= np.uint32(1 << (t % 32))
            return out
        return None

    def consume(self, token: int) -> None:
        if self.closed:
            if self.inner is not None:
                self.inner.consume(token)
            return
        self._seen.append(token)
        if self._seen[-len(self.close):] == self.close:
            self.closed = True
            return
        if self.used >= self.budget or self.closing:
            self.closing += 1
        else:
            self.used += 1

    def finished(self) -> bool:
        return self.closed and self.inner is not None and self.inner.finished()

    def fork(self) -> "ThinkingBudget":
        c = ThinkingBudget(self.close, self.budget, 10 ** 9,
                           self.inner.fork() if self.inner is not None else None)
        c.budget, c.used, c.closing, c.closed = self.budget, self.used, self.closing, self.closed
        c._seen = list(self._seen)
        return c
