"""Turns generated token ids into API deltas: incremental detokenisation, stop strings, reasoning split, tool calls.
Reference: ``crates/blaze-chat/src/parser`` (``ChatResponseProcessor``) and ``crates/blaze/src/server.rs`` (``Detok`` :744,
``StopCutter`` :656, ``Gen`` :794)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

from ..text import Detok, StopCutter
from .reasoning import ThinkParser
from .tools import ToolCall, ToolParser


class Delta:
    __slots__ = ("content", "reasoning", "tool_calls", "stopped")

    def __init__(self):
        self.content, self.reasoning, self.tool_calls, self.stopped = "", "", [], False

    def empty(self) -> bool:
        return not (self.content or self.reasoning or self.tool_calls)


class ChatResponseProcessor:
    def __init__(self, tokenizer, stop: Sequence[str] = (), include_stop: bool = False, skip_special_tokens: bool = True,
                 reasoning: bool = False, starts_in_think: bool = False, tool_parser: Optional[ToolParser] = None,
                 think_parser: Optional[ThinkParser] = None):
        self.detok = Detok(tokenizer, skip_special_tokens)
        self.cut = StopCutter(stop, include_stop) if stop else None
        self.think = (think_parser or ThinkParser(starts_in_think=starts_in_think)) if reasoning else None
        self.tools = tool_parser
        self.text = ""
        self.reasoning_text = ""
        self.tool_calls: List[ToolCall] = []
        self.stopped = False

    @property
    def stop_matched(self) -> Optional[str]:
        """The stop string that ended the answer (None: it ended otherwise)."""
        return self.cut.matched if self.cut is not None else None

    def _route(self, text: str, d: Delta, final: bool = False) -> None:
        r, c = (self.think.push(text) if self.think else ("", text))
        if final and self.think:
            fr, fc = self.think.flush()
            r, c = r + fr, c + fc
        if self.tools is not None:
            c2, calls = self.tools.push(c)
            if final:
                fc, fcalls = self.tools.flush()
                c2, calls = c2 + fc, calls + fcalls
            c = c2
            d.tool_calls.extend(calls)
            self.tool_calls.extend(calls)
        d.reasoning += r
        d.content += c
        self.reasoning_text += r
        self.text += c

    def push(self, token_ids: Sequence[int]) -> Delta:
        d = Delta()
        if self.stopped:
            d.stopped = True
            return d
        text = self.detok.push(token_ids)
        if self.cut is not None:
            text, hit = self.cut.push(text)
            if hit:
                self.stopped = d.stopped = True
        if text:
            self._route(text, d)
        return d

    def finish(self) -> Delta:
        d = Delta()
        tail = self.cut.flush() if (self.cut is not None and not self.stopped) else ""
        self._route(tail, d, final=True)
        return d
