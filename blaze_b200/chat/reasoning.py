"""Split of model text into reasoning and answer text, whole or streamed.

``ThinkParser`` handles the tag families (``<think>…</think>``): reasoning ends at the close tag, or where the model starts
a tool call without closing its thinking (for Qwen3 and DeepSeek only when the call marker opens a line, so that reasoning
which merely quotes the marker stays reasoning).  ``KimiThinkParser`` handles Kimi-K3's channels (think / response / tools
inside a message).  Both offer ``parse`` (the whole output at once) and ``push`` / ``flush`` (streaming; text that could be
the beginning of a marker is held back until it is decided).  Options: ``starts_in_think`` (the prompt ended inside the
reasoning channel), ``stream_reasoning`` (False: reasoning is delivered in one piece when it ends) and ``nonempty`` (an
output that never left the reasoning channel is delivered as answer text).
Reference: ``crates/blaze-chat/src/think/mod.rs`` (``TagDetector``), ``think/models/*.rs``; expected splits:
``crates/blaze-chat/tests/fixtures/reasoning_parity``."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple


def _partial_suffix(text: str, marker: str) -> int:
    """Length of the longest proper prefix of ``marker`` that ``text`` ends with."""
    for k in range(min(len(marker) - 1, len(text)), 0, -1):
        if text.endswith(marker[:k]):
            return k
    return 0


class ThinkParser:
    def __init__(self, open_tag: str = "<think>", close_tag: str = "</think>", starts_in_think: bool = False,
                 tool_start: Optional[str] = None, tool_at_line_start: bool = False, stream_reasoning: bool = True,
                 nonempty: bool = False):
        self.open, self.close = open_tag, close_tag
        self.tool_start, self.tool_at_line_start = tool_start, tool_at_line_start
        self.in_think = starts_in_think
        self.stream_reasoning, self.nonempty = stream_reasoning, nonempty
        self.buf = ""
        self.open_seen = False          # an open tag was consumed, or the reasoning is over: later ones are text
        self.last_char = ""             # last reasoning character already delivered (line-start test across chunks)
        self.kept: List[str] = []       # reasoning delivered so far, for ``nonempty``

    # ---- tool-call marker that ends unclosed reasoning
    def _tool_at(self, text: str, before: str) -> int:
        if not self.tool_start:
            return -1
        i = text.find(self.tool_start)
        while i >= 0:
            prev = text[i - 1] if i > 0 else before
            if not self.tool_at_line_start or prev in ("", "\n"):
                return i
            i = text.find(self.tool_start, i + 1)
        return -1

    def _drop_partial_tool(self, text: str, before: str) -> str:
        """Without the beginning of a call marker the output was cut in (only where a whole marker would have counted)."""
        if not self.tool_start or not self.tool_at_line_start:
            return text
        n = _partial_suffix(text, self.tool_start)
        if n == 0:
            return text
        cut = len(text) - n
        prev = text[cut - 1] if cut > 0 else before
        return text[:cut] if prev in ("", "\n") else text

    # ---- the whole output at once
    def parse(self, text: str) -> Tuple[str, str]:
        if not (self.in_think or self.open in text):
            return "", text
        while text.startswith(self.open):
            text = text[len(self.open):]
        if self.close in text:
            reasoning, answer = text.split(self.close, 1)
        else:
            i = self._tool_at(text, "")
            reasoning, answer = (text[:i], text[i:]) if i >= 0 else (self._drop_partial_tool(text, ""), "")
        if self.nonempty and not answer:
            return "", reasoning
        return reasoning, answer

    # ---- streaming
    def push(self, text: str) -> Tuple[str, str]:
        """Returns (reasoning delta, answer delta)."""
        r, c = self._push(text)
        if self.nonempty:
            if self.in_think:
                self.kept.append(r)
            else:
                self.kept.clear()
        return r, c

    def _push(self, text: str) -> Tuple[str, str]:
        self.buf += text
        cur = self.buf
        for marker in (self.open, self.close, self.tool_start):
            if marker and marker != cur and marker.startswith(cur):
                return "", ""                    # could still become a marker: wait
        if not self.open_seen:
            i, j = cur.find(self.open), cur.find(self.close)
            if i >= 0 and (j < 0 or i < j):
                cur = cur[:i] + cur[i + len(self.open):]
                self.buf = cur
                self.open_seen = self.in_think = True
        if self.in_think:
            j = cur.find(self.close)
            if j >= 0:
                self.buf, self.in_think, self.open_seen = "", False, True
                return cur[:j], cur[j + len(self.close):]
            t = self._tool_at(cur, self.last_char)
            if t >= 0:
                self.buf, self.in_think, self.open_seen = "", False, True
                return cur[:t], cur[t:]
            if not self.stream_reasoning:
                return "", ""
            hold = max(_partial_suffix(cur, m) for m in
                       (self.close, self.tool_start or "", "" if self.open_seen else self.open))
            out, self.buf = cur[:len(cur) - hold], cur[len(cur) - hold:]
            if out:
                self.last_char = out[-1]
            return out, ""
        self.buf = ""
        return "", cur

    def flush(self) -> Tuple[str, str]:
        out, self.buf = self.buf, ""
        if not self.in_think:
            return "", out
        if out.startswith(self.open):
            out = out[len(self.open):]
        out = self._drop_partial_tool(out, self.last_char)
        if self.nonempty:
            kept, self.kept = "".join(self.kept), []
            return "", kept + out
        return out, ""


# ---- Kimi-K3 channels -----------------------------------------------------------------------------------------------
K_THINK_OPEN, K_THINK_CLOSE = "<|open|>think<|sep|>", "<|close|>think<|sep|>"
K_RESP_OPEN, K_RESP_CLOSE = "<|open|>response<|sep|>", "<|close|>response<|sep|>"
K_TOOLS_OPEN, K_MSG_CLOSE = "<|open|>tools<|sep|>", "<|close|>message<|sep|>"
_K_CUT_MARKERS = ("<|open|>", "<|close|>", "<|close|>think", "<|open|>response", "<|close|>response", "<|open|>tools",
                  "<|close|>tools", "<|close|>message")


def _k_partial(text: str, markers: Sequence[str]) -> int:
    return max((_partial_suffix(text, m) for m in markers), default=0)


def _k_strip_cut(text: str) -> str:
    """Without a marker that the token limit cut before its separator."""
    for m in _K_CUT_MARKERS:
        if text.endswith(m):
            return text[:len(text) - len(m)]
    return text


def _k_unwrap(text: str) -> str:
    """Answer text of a response channel: the first channel's text if one opens, else the text without closes."""
    i = text.find(K_RESP_OPEN)
    if i >= 0:
        inner = text[i + len(K_RESP_OPEN):]
        j = inner.find(K_RESP_CLOSE)
        text = inner if j < 0 else inner[:j]
    else:
        text = text.replace(K_RESP_CLOSE, "")
    return _k_strip_cut(text.replace(K_MSG_CLOSE, ""))


def _k_clean(text: str) -> str:
    """Answer text with a tools channel passed through as it is."""
    t = text.find(K_TOOLS_OPEN)
    return _k_unwrap(text) if t < 0 else _k_unwrap(text[:t]) + text[t:]


def _k_strip_markers(text: str) -> str:
    for m in (K_RESP_OPEN, K_RESP_CLOSE, K_MSG_CLOSE):
        text = text.replace(m, "")
    return text


def _k_next_channel(text: str, start: int) -> int:
    found = [i for i in (text.find(K_RESP_OPEN, start), text.find(K_TOOLS_OPEN, start)) if i >= 0]
    return min(found) if found else -1


def _k_skipped_think(text: str, start: int, close: int, channel: int) -> bool:
    """The model answered without a think channel: a response close comes before any think close or channel opening."""
    rc = text.find(K_RESP_CLOSE, start)
    return rc >= 0 and all(b < 0 or rc < b for b in (close, channel))


def _k_plain_answer(text: str) -> bool:
    return (not any(t in text for t in (K_THINK_OPEN, K_THINK_CLOSE, "<|open|>think", "<|close|>think"))
            and (K_RESP_CLOSE in text or K_MSG_CLOSE in text))


class KimiThinkParser:
    """Kimi-K3: reasoning is the think channel; the answer is the response channel's text with the channel and message
    markers removed; a tools channel is passed on verbatim for the tool-call parser."""

    def __init__(self, starts_in_think: Optional[bool] = True, stream_reasoning: bool = True, nonempty: bool = False):
        self.in_think = True if starts_in_think is None else starts_in_think
        self.stream_reasoning, self.nonempty = stream_reasoning, nonempty
        self.buf = ""
        self.open_seen = False
        self.done = False               # the reasoning is over (or there was none)
        self.tools_raw = False          # inside the tools channel: pass through
        self.all_text = ""              # everything pushed, for ``nonempty``
        self.sent: List[str] = []       # reasoning pieces delivered while it was still undecided whether they are reasoning
        self.drop_late_close = False    # a think close after a skipped think channel is dropped

    def parse(self, text: str) -> Tuple[str, str]:
        if not (self.in_think or K_THINK_OPEN in text) and K_THINK_CLOSE not in text:
            return "", _k_clean(text)
        if self.nonempty and _k_plain_answer(text):
            return "", _k_clean(text)
        o = text.find(K_THINK_OPEN)
        start = 0 if o < 0 else o + len(K_THINK_OPEN)
        close, tools, channel = text.find(K_THINK_CLOSE, start), text.find(K_TOOLS_OPEN, start), _k_next_channel(text, start)
        if _k_skipped_think(text, start, close, channel):
            return "", _k_clean(text[start:].replace(K_THINK_CLOSE, ""))
        if close >= 0 and 0 <= tools < close:
            return _k_strip_cut(text[start:tools]), _k_clean(text[tools:])
        if close < 0:
            if channel >= 0:
                return _k_strip_cut(text[start:channel]), _k_clean(text[channel:])
            return _k_strip_cut(text[start:]), ""
        return text[start:close], _k_clean(text[close + len(K_THINK_CLOSE):])

    def push(self, text: str) -> Tuple[str, str]:
        self.buf += text
        if self.nonempty:
            self.all_text += text
        if not self.in_think and not self.done:
            o = self.buf.find(K_THINK_OPEN)
            if o >= 0:
                self.buf = self.buf[o + len(K_THINK_OPEN):]
                self.in_think = self.open_seen = True
            elif K_THINK_OPEN.startswith(self.buf):
                return "", ""
            else:
                self.done = True
        if not self.in_think:
            return "", self._answer()
        if not self.open_seen:
            o = self.buf.find(K_THINK_OPEN)
            if o >= 0:
                self.buf = self.buf[o + len(K_THINK_OPEN):]
                self.open_seen = True
        buf = self.buf
        close, tools, channel = buf.find(K_THINK_CLOSE), buf.find(K_TOOLS_OPEN), _k_next_channel(buf, 0)
        if _k_skipped_think(buf, 0, close, channel):
            replay, self.sent = "".join(self.sent), []
            self.in_think, self.done, self.drop_late_close = False, True, True
            return "", replay + self._answer()
        if close >= 0 and (tools < 0 or tools >= close):
            self.buf = buf[close + len(K_THINK_CLOSE):]
            self.in_think, self.done, self.sent = False, True, []
            return buf[:close], self._answer()
        if channel >= 0:
            self.buf = buf[channel:]
            self.in_think, self.done, self.sent = False, True, []
            self.tools_raw = self.buf.startswith(K_TOOLS_OPEN)
            return _k_strip_cut(buf[:channel]), self._answer()
        if not self.stream_reasoning:
            return "", ""
        markers = [K_THINK_CLOSE, K_TOOLS_OPEN, K_RESP_OPEN, K_RESP_CLOSE, K_MSG_CLOSE] + ([] if self.open_seen else [K_THINK_OPEN])
        out = _k_strip_cut(buf[:len(buf) - _k_partial(buf, markers)])
        self.buf = buf[len(out):]
        self.sent.append(out)
        return out, ""

    def _answer(self) -> str:
        if not self.buf:
            return ""
        buf, self.buf = self.buf, ""
        late = _k_partial(buf, [K_THINK_CLOSE]) if self.drop_late_close else 0

        def drop(t: str) -> str:
            return t.replace(K_THINK_CLOSE, "") if self.drop_late_close else t

        if self.tools_raw:
            out, self.buf = buf[:len(buf) - late], buf[len(buf) - late:]
            return drop(out)
        t = buf.find(K_TOOLS_OPEN)
        if t >= 0:
            out, self.buf = buf[:len(buf) - late], buf[len(buf) - late:]
            t = min(t, len(out))
            self.tools_raw = True
            return drop(_k_strip_markers(out[:t])) + drop(out[t:])
        markers = [K_RESP_OPEN, K_RESP_CLOSE, K_MSG_CLOSE, K_TOOLS_OPEN] + ([K_THINK_CLOSE] if self.drop_late_close else [])
        hold = _k_partial(buf, markers)
        out, self.buf = buf[:len(buf) - hold], buf[len(buf) - hold:]
        return drop(_k_strip_markers(out))

    def flush(self) -> Tuple[str, str]:
        self.sent = []
        if self.nonempty:
            text, self.all_text = self.all_text, ""
            if self.in_think and _k_plain_answer(text):
                self.buf = ""
                return "", _k_clean(text)
            if self.in_think and not self.stream_reasoning and self.buf:
                out, self.buf = self.buf, ""
                return out, ""
            return "", ""
        out, self.buf = self.buf, ""
        if not self.in_think:
            return "", out
        return (out[len(K_THINK_OPEN):] if out.startswith(K_THINK_OPEN) else out), ""


#: tag families by ``--reasoning-parser`` name: (tool-call marker that ends unclosed reasoning, only at a line start)
_TAG_FAMILIES = {
    "qwen3": ("<tool_call>", True),
    "deepseek-v41": ("<｜DSML｜ calls>", True),
    "deepseek-v4": ("<｜DSML｜tool_calls>", True),
    "deepseek": ("<｜DSML｜tool_calls>", True),
    "glm": ("<tool_call>", False),
}


def get_think_parser(name: str = "qwen3", starts_in_think: Optional[bool] = None, stream_reasoning: bool = True,
                     nonempty: bool = False):
    """Reasoning splitter of a family (names as the reference's ``--reasoning-parser``: qwen3, deepseek-v4, deepseek-v41,
    glm45, kimi_k3; family prefixes are accepted).  ``starts_in_think`` None takes the family's default (Kimi-K3 prompts
    end inside the think channel, the others do not)."""
    key = (name or "qwen3").lower().replace("_", "-")
    if key.startswith("kimi"):
        return KimiThinkParser(starts_in_think, stream_reasoning, nonempty)
    if key in ("deepseek-v4.1", "deepseekv41"):
        key = "deepseek-v41"
    for family, (tool, at_line) in _TAG_FAMILIES.items():
        if key.startswith(family):
            return ThinkParser("<think>", "</think>", bool(starts_in_think), tool, at_line, stream_reasoning, nonempty)
    raise ValueError(f"unknown reasoning parser {name!r}")
