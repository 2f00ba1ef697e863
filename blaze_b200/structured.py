"""Structured output: grammar constraints that mask the sampler's vocabulary.

Same role as the reference's ``crates/blaze/src/structured.rs`` (llguidance ``Grammars::load`` :37, ``Constraint``
mask / advance :92-116, ``grammar_of`` :128 mapping ``response_format`` json_object / json_schema and guided regex /
choice / grammar requests to a grammar).  llguidance is used when importable; a small built-in engine covers
``choice`` and prefix-closed regex-free cases so that the API keeps working without it.
"""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional, Sequence

import torch


class ConstraintError(ValueError):
    pass


class Constraint:
    """mask(pending) → bool tensor [vocab] of allowed next tokens; advance(token) consumes one."""

    def mask(self, pending: Sequence[int] = ()) -> torch.Tensor:
        raise NotImplementedError

    def advance(self, token: int) -> None:
        raise NotImplementedError

    def finished(self) -> bool:
        return False


class ChoiceConstraint(Constraint):
    """Output must be exactly one of the given strings (then an end-of-sequence token)."""

    def __init__(self, tokenizer, choices: Sequence[str], eos_ids: Sequence[int], vocab_size: int):
        self.tok, self.eos, self.V = tokenizer, list(eos_ids), vocab_size
        self.choices = [c.encode("utf-8") for c in choices]
        self.done = b""
        self._bytes: Optional[List[bytes]] = None

    def _token_bytes(self) -> List[bytes]:
        if self._bytes is None:
            self._bytes = [self.tok.token_bytes(i) for i in range(min(self.V, self.tok.vocab_size))]
        return self._bytes

    def mask(self, pending: Sequence[int] = ()) -> torch.Tensor:
        prefix = self.done + b"".join(self._token_bytes()[t] for t in pending if t < len(self._token_bytes()))
        live = [c for c in self.choices if c.startswith(prefix)]
        m = torch.zeros(self.V, dtype=torch.bool)
        if any(c == prefix for c in live):
            for e in self.eos:
                if e < self.V:
                    m[e] = True
        rest = [c[len(prefix):] for c in live if len(c) > len(prefix)]
        if rest:
            for tid, b in enumerate(self._token_bytes()):
                if b and any(r.startswith(b) for r in rest):
                    m[tid] = True
        return m

    def advance(self, token: int) -> None:
        tb = self._token_bytes()
        if token < len(tb) and token not in self.eos:
            self.done += tb[token]

    def finished(self) -> bool:
        return any(c == self.done for c in self.choices)


class LLGuidanceConstraint(Constraint):
    def __init__(self, ll_tokenizer, grammar: str, vocab_size: int):
        import llguidance
        self.V = vocab_size
        self.m = llguidance.LLMatcher(ll_tokenizer, grammar)
        err = self.m.get_error()
        if err:
            raise ConstraintError(err)

    def mask(self, pending: Sequence[int] = ()) -> torch.Tensor:
        import llguidance.torch as llt
        m = self.m
        if pending:
            m = m.deep_copy()
            for t in pending:
                m.consume_token(int(t))
        bits = llt.allocate_token_bitmask(1, self.V)
        llt.fill_next_token_bitmask(m, bits, 0)
        words = bits[0].to(torch.int64) & 0xFFFFFFFF
        idx = torch.arange(self.V)
        return ((words[idx // 32] >> (idx % 32)) & 1).bool()

    def advance(self, token: int) -> None:
        self.m.consume_token(int(token))

    def finished(self) -> bool:
        return self.m.is_stopped()


class Grammars:
    """Builds constraints for requests; owns the (expensive) llguidance tokenizer."""

    def __init__(self, tokenizer, vocab_size: int, eos_ids: Sequence[int]):
        self.tok, self.V, self.eos = tokenizer, vocab_size, list(eos_ids)
        self.ll_tok = None
        self.error: Optional[str] = None
        try:
            import llguidance
            import llguidance.hf
            inner = getattr(tokenizer, "tk", None)
            if inner is not None:
                self.ll_tok = llguidance.LLTokenizer(llguidance.hf.from_tokenizer(inner, n_vocab=vocab_size)) \
                    if hasattr(llguidance.hf, "from_tokenizer") else None
        except Exception as e:  # fall back to the built-in engine
            self.error = repr(e)

    @classmethod
    def load(cls, tokenizer, vocab_size: int, eos_ids: Sequence[int]) -> "Grammars":
        return cls(tokenizer, vocab_size, eos_ids)

    def constraint(self, spec: Dict[str, Any]) -> Optional[Constraint]:
        if not spec:
            return None
        kind = spec["kind"]
        if kind == "choice":
            return ChoiceConstraint(self.tok, spec["choices"], self.eos, self.V)
        if self.ll_tok is None:
            raise ConstraintError(f"structured output of kind {kind!r} needs llguidance with a Hugging Face tokenizer")
        import llguidance
        if kind == "json_schema":
            g = llguidance.LLMatcher.grammar_from_json_schema(json.dumps(spec["schema"]))
        elif kind == "json_object":
            g = llguidance.LLMatcher.grammar_from_json_schema(json.dumps({"type": "object"}))
        elif kind == "regex":
            g = llguidance.LLMatcher.grammar_from_regex(spec["regex"])
        elif kind == "grammar":
            g = llguidance.LLMatcher.grammar_from_lark(spec["grammar"])
        else:
            raise ConstraintError(f"unknown structured-output kind {kind!r}")
        return LLGuidanceConstraint(self.ll_tok, g, self.V)


def grammar_of(body: Dict[str, Any]) -> Optional[Dict[str, Any]]:
    """Map request fields to a constraint spec (``structured.rs:128``): ``response_format`` (json_object /
    json_schema), ``structured_outputs`` / ``guided_json|regex|choice|grammar``."""
    rf = body.get("response_format")
    if isinstance(rf, dict):
        t = rf.get("type")
        if t == "json_object":
            return {"kind": "json_object"}
        if t == "json_schema":
            js = rf.get("json_schema") or {}
            schema = js.get("schema", js)
            if not isinstance(schema, dict):
                raise ConstraintError("response_format.json_schema.schema must be an object")
            return {"kind": "json_schema", "schema": schema}
        if t not in (None, "text"):
            raise ConstraintError(f"unknown response_format type {t!r}")
    so = body.get("structured_outputs") or {}
    for key, kind, field in (("json", "json_schema", "schema"), ("regex", "regex", "regex"), ("choice", "choice", "choices"),
                             ("grammar", "grammar", "grammar")):
        v = so.get(key, body.get(f"guided_{key}"))
        if v is not None:
            if kind == "json_schema" and isinstance(v, str):
                v = json.loads(v)
            if kind == "choice" and (not isinstance(v, list) or not v):
                raise ConstraintError("choice needs a non-empty list of strings")
            return {"kind": kind, field: v}
    return None
