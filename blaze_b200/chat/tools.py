"""Tool-call extraction from generated text, streaming-safe.

Two wire formats (reference: ``crates/blaze-chat/src/tool_call`` — qwen3_coder, deepseek, kimi parsers):
  * ``hermes`` / Qwen3: ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>``
  * ``qwen3_coder``: ``<tool_call><function=NAME><parameter=KEY>VALUE</parameter>…</function></tool_call>``
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class ToolCall:
    name: str
    arguments: str                      # JSON text
    id: str = field(default_factory=lambda: "call_" + uuid.uuid4().hex[:24])

    def to_openai(self, index: int = 0) -> Dict[str, Any]:
        return {"index": index, "id": self.id, "type": "function", "function": {"name": self.name, "arguments": self.arguments}}


class ToolParser:
    OPEN, CLOSE = "<tool_call>", "</tool_call>"

    def __init__(self, tools: Optional[List[Dict[str, Any]]] = None):
        self.tools = tools or []
        self.buf = ""
        self.inside = False
        self.calls: List[ToolCall] = []

    def parse_body(self, body: str) -> Optional[ToolCall]:
        raise NotImplementedError

    def _hold(self, tag: str) -> int:
        for k in range(min(len(tag) - 1, len(self.buf)), 0, -1):
            if self.buf.endswith(tag[:k]):
                return k
        return 0

    def push(self, text: str) -> Tuple[str, List[ToolCall]]:
        """Returns (plain content delta, tool calls completed by this delta)."""
        self.buf += text
        content, done = "", []
        while self.buf:
            if self.inside:
                i = self.buf.find(self.CLOSE)
                if i < 0:
                    break
                call = self.parse_body(self.buf[:i])
                if call is not None:
                    done.append(call)
                    self.calls.append(call)
                self.buf = self.buf[i + len(self.CLOSE):]
                self.inside = False
                continue
            i = self.buf.find(self.OPEN)
            if i >= 0:
                content += self.buf[:i].rstrip("\n") if not self.buf[:i].strip() else self.buf[:i]
                self.buf = self.buf[i + len(self.OPEN):]
                self.inside = True
                continue
            h = self._hold(self.OPEN)
            content += self.buf[:len(self.buf) - h]
            self.buf = self.buf[len(self.buf) - h:]
            break
        return content, done

    def flush(self) -> Tuple[str, List[ToolCall]]:
        if self.inside:      # unterminated call: try to salvage it
            call = self.parse_body(self.buf)
            self.buf = ""
            if call is not None:
                self.calls.append(call)
                return "", [call]
            return "", []
        out, self.buf = self.buf, ""
        return out, []


class HermesToolParser(ToolParser):
    def parse_body(self, body: str) -> Optional[ToolCall]:
        body = body.strip()
        try:
            obj = json.loads(body)
        except ValueError:
            m = re.search(r"\{.*\}", body, re.S)
            if not m:
                return None
            try:
                obj = json.loads(m.group(0))
            except ValueError:
                return None
        name = obj.get("name")
        if not isinstance(name, str):
            return None
        args = obj.get("arguments", obj.get("parameters", {}))
        return ToolCall(name, args if isinstance(args, str) else json.dumps(args, ensure_ascii=False))


class Qwen3CoderToolParser(ToolParser):
    FN = re.compile(r"<function=([^>\s]+)>(.*?)(?:</function>|$)", re.S)
    PARAM = re.compile(r"<parameter=([^>\s]+)>(.*?)(?:</parameter>|(?=<parameter=)|$)", re.S)

    def _schema(self, fn: str) -> Dict[str, Any]:
        for t in self.tools:
            f = t.get("function", t)
            if f.get("name") == fn:
                return (f.get("parameters") or {}).get("properties") or {}
        return {}

    def parse_body(self, body: str) -> Optional[ToolCall]:
        m = self.FN.search(body)
        if not m:
            return None
        name, inner = m.group(1), m.group(2)
        props = self._schema(name)
        args: Dict[str, Any] = {}
        for pm in self.PARAM.finditer(inner):
            key, raw = pm.group(1), pm.group(2)
            raw = raw[1:] if raw.startswith("\n") else raw
            raw = raw[:-1] if raw.endswith("\n") else raw
            typ = (props.get(key) or {}).get("type", "string")
            val: Any = raw
            if typ in ("integer", "number", "boolean", "object", "array", "null") or typ != "string":
                try:
                    val = json.loads(raw)
                except ValueError:
                    low = raw.strip().lower()
                    val = True if low == "true" else False if low == "false" else raw
            args[key] = val
        return ToolCall(name, json.dumps(args, ensure_ascii=False))


def get_tool_parser(name: str, tools=None) -> ToolParser:
    name = (name or "hermes").lower()
    if name in ("hermes", "qwen", "qwen3", "qwen25", "json"):
        return HermesToolParser(tools)
    if name in ("qwen3_coder", "qwen3-coder", "xml"):
        return Qwen3CoderToolParser(tools)
    raise ValueError(f"unknown tool-call parser {name!r}")
