"""Tokenizer glue: Hugging Face ``tokenizers`` for real checkpoints, a byte-level stand-in for synthetic models.

Reference: ``crates/blaze/src/text.rs`` — eos ids from generation_config / tokenizer_config (:15), ``frequent_ids`` (:55),
``token_bytes`` (:85, used by the stop-string cutter and the grammar engine).
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence


class ByteTokenizer:
    """ids 0..255 are bytes; a few named specials follow.  Deterministic and dependency-free (tests, synthetic runs)."""

    SPECIALS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>", "<tool_call>", "</tool_call>",
                "<|vision_start|>", "<|vision_end|>", "<|image_pad|>"]

    def __init__(self, vocab_size: int = 1024):
        self.vocab_size = max(vocab_size, 256 + len(self.SPECIALS))
        self.special: Dict[str, int] = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self.inv = {v: k for k, v in self.special.items()}
        self.eos_ids = [self.special["<|endoftext|>"], self.special["<|im_end|>"]]
        # like Qwen tokenizers, the think / tool tags are ordinary added tokens that decoding keeps
        self.control = {self.special[s] for s in self.SPECIALS if s.startswith("<|")}
        self.chat_template: Optional[str] = None

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        out: List[int] = []
        i = 0
        while i < len(text):
            hit = None
            if text[i] == "<":
                for s, tid in self.special.items():
                    if text.startswith(s, i):
                        hit = (s, tid)
                        break
            if hit:
                out.append(hit[1])
                i += len(hit[0])
            else:
                out.extend(text[i].encode("utf-8"))
                i += 1
        return out

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        return self.token_bytes_of(ids, skip_special_tokens).decode("utf-8", errors="replace")

    def token_bytes_of(self, ids: Sequence[int], skip_special_tokens: bool = True) -> bytes:
        buf = bytearray()
        for t in ids:
            if t < 256:
                buf.append(t)
            elif t in self.inv:
                if not skip_special_tokens or t not in self.control:
                    buf.extend(self.inv[t].encode())
            else:
                buf.extend(f"<{t}>".encode())
        return bytes(buf)

    def token_bytes(self, tid: int) -> bytes:
        return self.token_bytes_of([tid], skip_special_tokens=False)

    def token_id(self, token: str) -> Optional[int]:
        return self.special.get(token)


class HFTokenizer:
    def __init__(self, model_dir: str):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(os.path.join(model_dir, "tokenizer.json"))
        self.vocab_size = self.tk.get_vocab_size(with_added_tokens=True)
        self.eos_ids: List[int] = []
        self.chat_template: Optional[str] = None
        cfgp = os.path.join(model_dir, "tokenizer_config.json")
        if os.path.exists(cfgp):
            with open(cfgp) as f:
                tc = json.load(f)
            self.chat_template = tc.get("chat_template")
            eos = tc.get("eos_token")
            if isinstance(eos, dict):
                eos = eos.get("content")
            if isinstance(eos, str):
                tid = self.tk.token_to_id(eos)
                if tid is not None:
                    self.eos_ids.append(tid)
        jin = os.path.join(model_dir, "chat_template.jinja")
        if os.path.exists(jin):
            with open(jin) as f:
                self.chat_template = f.read()
        gp = os.path.join(model_dir, "generation_config.json")
        if os.path.exists(gp):
            with open(gp) as f:
                e = json.load(f).get("eos_token_id")
            for t in (e if isinstance(e, list) else [e]):
                if isinstance(t, int) and t not in self.eos_ids:
                    self.eos_ids.append(t)
        self._bytes_cache: Dict[int, bytes] = {}

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        return self.tk.encode(text, add_special_tokens=add_special_tokens).ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def token_bytes(self, tid: int) -> bytes:
        b = self._bytes_cache.get(tid)
        if b is None:
            b = self.tk.decode([tid], skip_special_tokens=False).encode("utf-8")
            self._bytes_cache[tid] = b
        return b

    def token_id(self, token: str) -> Optional[int]:
        return self.tk.token_to_id(token)


def load_tokenizer(model_dir: Optional[str], vocab_size: int = 1024):
    if model_dir and os.path.exists(os.path.join(model_dir, "tokenizer.json")):
        return HFTokenizer(model_dir)
    return ByteTokenizer(vocab_size)


def frequent_ids(tok, sample_text: str, k: int = 32768) -> List[int]:
    """Ids seen in ``sample_text`` first, then the lowest ids, up to ``k`` (reduced-vocabulary draft heads)."""
    seen: List[int] = []
    have = set()
    for t in tok.encode(sample_text):
        if t not in have:
            have.add(t)
            seen.append(t)
    i = 0
    while len(seen) < min(k, tok.vocab_size):
        if i not in have:
            seen.append(i)
        i += 1
    return seen[:k]


class Detok:
    """Incremental detokeniser that never emits half a UTF-8 character (``server.rs:744``)."""

    def __init__(self, tok, skip_special_tokens: bool = True):
        self.tok, self.skip = tok, skip_special_tokens
        self.ids: List[int] = []
        self.emitted = 0            # characters already returned
        self.window = 0             # ids before this index are final

    def push(self, new_ids: Sequence[int]) -> str:
        self.ids.extend(new_ids)
        text = self.tok.decode(self.ids[self.window:], skip_special_tokens=self.skip)
        if text.endswith("�"):
            return ""
        out = text[self.emitted:]
        self.emitted = len(text)
        if len(self.ids) - self.window > 64:        # keep decode windows short
            self.window = len(self.ids)
            self.emitted = 0
        return out


class StopCutter:
    """Holds back text that could be the start of a stop string; reports the cut when one completes
    (``server.rs:656``; the reference matches with KMP, this keeps the longest possible partial suffix)."""

    def __init__(self, stops: Sequence[str], include: bool = False):
        self.stops = [s for s in stops if s]
        self.include = include
        self.buf = ""
        self.done = False
        self.matched: Optional[str] = None       # the stop string that ended the text

    def push(self, text: str):
        """Returns (text safe to emit, stopped?)."""
        if self.done:
            return "", True
        self.buf += text
        first = None
        for s in self.stops:
            i = self.buf.find(s)
            if i >= 0 and (first is None or i < first[0]):
                first = (i, s)
        if first is not None:
            end = first[0] + (len(first[1]) if self.include else 0)
            out, self.buf, self.done, self.matched = self.buf[:end], "", True, first[1]
            return out, True
        hold = 0
        for s in self.stops:
            for k in range(min(len(s) - 1, len(self.buf)), 0, -1):
                if self.buf.endswith(s[:k]):
                    hold = max(hold, k)
                    break
        out = self.buf[:len(self.buf) - hold]
        self.buf = self.buf[len(self.buf) - hold:]
        return out, False

    def flush(self) -> str:
        out, self.buf = self.buf, ""
        return out
