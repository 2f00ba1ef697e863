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
    """``eos_ids``: every token that ends a generation.  The matcher knows one end-of-sequence token (the first); where it
    allows that one, all are allowed (a chat model ends its turn with ``<|im_end|>``, not ``<|endoftext|>``), and any of
    them is consumed as that one."""

    def __init__(self, ll_tokenizer, grammar: str, vocab_size: int, eos_ids: Sequence[int] = ()):
        import llguidance
        self.V = vocab_size
        self.eos = [int(e) for e in eos_ids if int(e) < vocab_size]
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
                m.consume_token(self._as_matcher_token(t))
        bits = llt.allocate_token_bitmask(1, self.V)
        llt.fill_next_token_bitmask(m, bits, 0)
        words = bits[0].to(torch.int64) & 0xFFFFFFFF
        idx = torch.arange(self.V)
        out = ((words[idx // 32] >> (idx % 32)) & 1).bool()
        if self.eos and bool(out[self.eos[0]]):
            out[self.eos] = True
        return out

    def _as_matcher_token(self, token: int) -> int:
        return self.eos[0] if self.eos and int(token) in self.eos else int(token)

    def advance(self, token: int) -> None:
        self.m.consume_token(self._as_matcher_token(token))

    def finished(self) -> bool:
        return self.m.is_stopped()


class _AsGuidanceTokenizer:
    """The view of a tokenizer that ``llguidance.TokenizerWrapper`` asks for: the bytes of every token id, the ids of the
    special tokens (never produced from text), the end-of-sequence id and an encode call."""

    def __init__(self, tokenizer, vocab_size: int, eos_ids: Sequence[int]):
        self._tok = tokenizer
        self.eos_token_id = int(eos_ids[0])
        self.bos_token_id = None
        n = min(vocab_size, getattr(tokenizer, "vocab_size", vocab_size))
        control = set(getattr(tokenizer, "control", ())) | set(int(e) for e in eos_ids)
        self.special_token_ids = sorted(t for t in control if t < vocab_size)
        self.tokens = []
        for i in range(vocab_size):
            b = tokenizer.token_bytes(i) if i < n else b""
            if i in control:
                b = b"\xff" + (b or f"<{i}>".encode())          # the marker llguidance uses for special tokens
            self.tokens.append(b or f"<unused{i}>".encode())

    def __call__(self, text) -> List[int]:
        if isinstance(text, (bytes, bytearray)):
            text = bytes(text).decode("utf-8", errors="replace")
        return self._tok.encode(text)


class Grammars:
    """Builds constraints for requests; owns the (expensive) llguidance tokenizer."""

    def __init__(self, tokenizer, vocab_size: int, eos_ids: Sequence[int]):
        self.tok, self.V, self.eos = tokenizer, vocab_size, list(eos_ids)
        self.ll_tok = None
        self.error: Optional[str] = None
        try:
            import llguidance
            inner = getattr(tokenizer, "tk", None)
            if inner is not None:
                import llguidance.hf
                self.ll_tok = llguidance.LLTokenizer(llguidance.hf.from_tokenizer(inner, n_vocab=vocab_size)) \
                    if hasattr(llguidance.hf, "from_tokenizer") else None
            elif hasattr(tokenizer, "token_bytes") and self.eos:
                # any tokenizer that can name the bytes of its tokens (the byte-level stand-in of synthetic models)
                self.ll_tok = llguidance.LLTokenizer(llguidance.TokenizerWrapper(_AsGuidanceTokenizer(tokenizer, vocab_size, self.eos)),
                                                     n_vocab=vocab_size)
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
        return LLGuidanceConstraint(self.ll_tok, g, self.V, self.eos)


def grammar_of(body: Dict[str, Any], max_ws: int = 64) -> Optional[Dict[str, Any]]:
    """Map request fields to a constraint spec (``structured.rs:118-190``): OpenAI ``response_format`` (json_object /
    json_schema), vLLM ``structured_outputs`` / ``guided_decoding`` {json, regex, choice, grammar, json_object} and the older
    ``guided_json|regex|choice|grammar``, SGLang ``regex`` / ``json_schema``.

    White space between JSON tokens: the grammar engine allows any run of it, and a model that would rather answer in words
    finds white space the likeliest allowed token before ``{`` again and again, to the end of ``max_tokens``.  Runs are bounded
    to ``max_ws`` characters (0: unbounded); a request's ``whitespace_pattern`` / ``guided_whitespace_pattern`` or
    ``disable_any_whitespace`` (compact JSON) win, as does a schema's own ``x-guidance``."""
    so = body.get("structured_outputs") if isinstance(body.get("structured_outputs"), dict) else body.get("guided_decoding")
    so = so if isinstance(so, dict) else {}

    def opt(k):
        v = so.get(k)
        return v if v is not None else body.get(k)

    pattern = opt("whitespace_pattern") if opt("whitespace_pattern") is not None else opt("guided_whitespace_pattern")
    if pattern is not None:
        ws = {"whitespace_pattern": pattern}
    elif opt("disable_any_whitespace") is True:
        ws = {"whitespace_flexible": False}
    elif max_ws > 0:
        ws = {"whitespace_pattern": "[\\x20\\x0A\\x0D\\x09]{1,%d}" % max_ws}
    else:
        ws = None

    def schema_spec(v):
        if isinstance(v, str):
            v = json.loads(v)
        if not isinstance(v, dict):
            raise ConstraintError("a JSON schema must be an object")
        if ws is not None and "x-guidance" not in v:
            v = {**v, "x-guidance": ws}
        return {"kind": "json_schema", "schema": v}

    rf = body.get("response_format")
    if isinstance(rf, dict):
        t = rf.get("type")
        if t == "json_object":
            return schema_spec({"type": "object"})
        if t == "json_schema":
            js = rf.get("json_schema")
            schema = js.get("schema") if isinstance(js, dict) and "schema" in js else (js if isinstance(js, dict) and js and "name" not in js else rf.get("schema"))
            if not isinstance(schema, dict):
                raise ConstraintError("response_format of type json_schema needs json_schema.schema (an object)")
            return schema_spec(schema)
        if t not in (None, "text"):
            raise ConstraintError(f"unknown response_format type {t!r}")

    def field(k, old):
        v = so.get(k)
        return v if v is not None else body.get(old)

    v = field("json", "guided_json")
    if v is None:
        v = body.get("json_schema")
    if v is not None:
        return schema_spec(v)
    if so.get("json_object") is True:
        return schema_spec({"type": "object"})
    v = field("regex", "guided_regex")
    if v is None:
        v = body.get("regex")
    if v is not None:
        if not isinstance(v, str):
            raise ConstraintError("regex must be a string")
        return {"kind": "regex", "regex": v}
    v = field("choice", "guided_choice")
    if v is not None:
        if not isinstance(v, list) or not v or not all(isinstance(c, str) for c in v):
            raise ConstraintError("choice needs a non-empty list of strings")
        return {"kind": "choice", "choices": v}
    v = field("grammar", "guided_grammar")
    if v is not None:
        if not isinstance(v, str):
            raise ConstraintError("grammar must be a string")
        return {"kind": "grammar", "grammar": v}
    return None


#: call syntax per tool-call parser: (opening tag, text before the tool's name, text after it, closing tag)
_CALL_SYNTAX = {
    "qwen3_coder": ("<tool_call>", "<function=", ">", "</tool_call>"),
    "qwen3-coder": ("<tool_call>", "<function=", ">", "</tool_call>"),
    "hermes": ("<tool_call>", '{"name": "', '"', "</tool_call>"),
    "qwen": ("<tool_call>", '{"name": "', '"', "</tool_call>"),
    "qwen25": ("<tool_call>", '{"name": "', '"', "</tool_call>"),
}


def forced_call_grammar(parser: Optional[str], names: Sequence[str], single: bool = False) -> Optional[str]:
    """Lark grammar of an answer that must consist of tool calls (``tool_choice`` "required" or a named function): the
    parser's call syntax around one of ``names``, then whatever the model writes for the arguments up to the closing tag;
    ``single`` allows one call only (``parallel_tool_calls`` false).  None for parsers whose syntax is not listed (the model
    is then only asked).  White space around the calls is bounded: an unbounded ``ws*`` would let a model that prefers to
    answer in words emit white space forever under greedy decoding.  Reference: ``crates/blaze/src/server/chat.rs:81-103``
    (``forced_call_grammar``)."""
    syn = _CALL_SYNTAX.get((parser or "").lower())
    if syn is None or not names:
        return None
    opening, before, after, closing = (json.dumps(t) for t in syn)
    alts = " | ".join(json.dumps(n) for n in names)
    # the arguments are free text that ends with the closing tag (a lexeme with a suffix: the shortest such text)
    return (f"start: ws call{'' if single else ' (ws call)*'} ws\n"
            f"call: {opening} ws {before} name {after} body\n"
            f"name: {alts}\n"
            "ws: /[ \\t\\r\\n]{0,4}/\n"
            f"body[suffix={closing}]: /(?s:.*)/\n")
