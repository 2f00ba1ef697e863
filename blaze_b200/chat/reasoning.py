"""Streaming split of model text into reasoning (inside ``<think>…</think>``) and answer text.
Reference: ``crates/blaze-chat/src/think`` (reasoning tag detectors)."""
from __future__ import annotations

from typing import Tuple


class ThinkParser:
    def __init__(self, open_tag: str = "<think>", close_tag: str = "</think>", starts_in_think: bool = False):
        self.open, self.close = open_tag, close_tag
        self.in_think = starts_in_think
        self.buf = ""
        self.seen_any = False

    def _hold(self, tag: str) -> int:
        for k in range(min(len(tag) - 1, len(self.buf)), 0, -1):
            if self.buf.endswith(tag[:k]):
                return k
        return 0

    def push(self, text: str) -> Tuple[str, str]:
        """Returns (reasoning delta, content delta)."""
        self.buf += text
        reasoning, content = "", ""
        while self.buf:
            if self.in_think:
                i = self.buf.find(self.close)
                if i >= 0:
                    reasoning += self.buf[:i]
                    self.buf = self.buf[i + len(self.close):].lstrip("\n")
                    self.in_think = False
                    continue
                h = self._hold(self.close)
                reasoning += self.buf[:len(self.buf) - h]
                self.buf = self.buf[len(self.buf) - h:]
                break
            i = self.buf.find(self.open)
            if i >= 0 and not self.seen_any and not self.buf[:i].strip():
                self.buf = self.buf[i + len(self.open):].lstrip("\n")
                self.in_think = True
                self.seen_any = True
                continue
            h = self._hold(self.open) if not self.seen_any else 0
            out = self.buf[:len(self.buf) - h]
            if out.strip():
                self.seen_any = True
            content += out
            self.buf = self.buf[len(self.buf) - h:]
            break
        return reasoning, content

    def flush(self) -> Tuple[str, str]:
        out, self.buf = self.buf, ""
        return (out, "") if self.in_think else ("", out)


#: reasoning markers per model family (reference: ``crates/blaze-chat/src/think/models`` — qwen3.rs, kimi_k3.rs;
#: ``kimi_k3_format.rs`` for the channel markers)
THINK_TAGS = {
    "qwen3": ("<think>", "</think>"),
    "deepseek": ("<think>", "</think>"),
    "glm": ("<think>", "</think>"),
    "kimi": ("<|open|>think<|sep|>", "<|close|>think<|sep|>"),
}


def get_think_parser(name: str = "qwen3", starts_in_think: bool = False) -> ThinkParser:
    key = (name or "qwen3").lower()
    for family, tags in THINK_TAGS.items():
        if key.startswith(family):
            return ThinkParser(tags[0], tags[1], starts_in_think)
    raise ValueError(f"unknown reasoning parser {name!r}")
