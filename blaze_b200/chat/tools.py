"""Tool-call extraction from generated text, streaming-safe.

Wire formats (reference: ``crates/blaze-chat/src/tool_call/models`` — qwen3_coder.rs, deepseek_v4.rs, kimi_k3.rs):
  * ``hermes`` / Qwen3: ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>``
  * ``qwen3_coder``: ``<tool_call><function=NAME><parameter=KEY>VALUE</parameter>…</function></tool_call>``
  * ``deepseek`` (DSML): ``<｜DSML｜tool_calls><｜DSML｜invoke name="F"><｜DSML｜parameter name="K" string="true|false">V
    </｜DSML｜parameter>…</｜DSML｜invoke>…</｜DSML｜tool_calls>``; ``string="false"`` values are JSON
  * ``kimi``: a tools channel ``<|open|>tools<|sep|> … <|close|>tools<|sep|>`` of
    ``<|open|>call tool="F"<|sep|><|open|>argument key="K" type="T"<|sep|>V<|close|>argument<|sep|>…<|close|>call<|sep|>``
  * ``glm``: ``<tool_call>F\n<arg_key>K</arg_key>\n<arg_value>V</arg_value>…</tool_call>``
One block may carry several calls; ``parse_body`` then returns a list.
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


def _as_list(found) -> List["ToolCall"]:
    return [] if found is None else list(found) if isinstance(found, (list, tuple)) else [found]


def _json_or_text(raw: str) -> Any:
    try:
        return json.loads(raw)
    except ValueError:
        return raw


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
                for call in _as_list(self.parse_body(self.buf[:i])):
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
            calls = _as_list(self.parse_body(self.buf))
            self.buf = ""
            self.calls.extend(calls)
            return "", calls
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


class DsmlToolParser(ToolParser):
    """DeepSeek's DSML block.  ``strip_strings`` trims string values (the first tag set); the second tag set
    (names that start with a space: ``｜DSML｜ calls``) keeps them as written."""
    MARK = "｜DSML｜"

    def __init__(self, tools=None, spaced: bool = False):
        super().__init__(tools)
        block, inv, par = (" calls", " invoke", " parameter") if spaced else ("tool_calls", "invoke", "parameter")
        m = re.escape(self.MARK)
        self.OPEN, self.CLOSE = f"<{self.MARK}{block}>", f"</{self.MARK}{block}>"
        self.strip_strings = not spaced
        self.INVOKE = re.compile(rf'<{m}{re.escape(inv)}\s+name="([^"]+)"\s*(?:/>|>(.*?)(?:</{m}{re.escape(inv)}>|$))', re.S)
        self.PARAM = re.compile(rf'<{m}{re.escape(par)}\s+name="([^"]+)"\s+string="([^"]+)"\s*>(.*?)</{m}{re.escape(par)}>', re.S)

    def parse_body(self, body: str):
        out = []
        for m in self.INVOKE.finditer(body):
            args: Dict[str, Any] = {}
            for pm in self.PARAM.finditer(m.group(2) or ""):
                key, is_str, raw = pm.group(1), pm.group(2) == "true", pm.group(3)
                args[key] = (raw.strip() if self.strip_strings else raw) if is_str else _json_or_text(raw.strip())
            out.append(ToolCall(m.group(1), json.dumps(args, ensure_ascii=False)))
        return out


class KimiToolParser(ToolParser):
    """Kimi's tools channel.  Text outside the channel loses its response wrappers; calls without a tool name are dropped."""
    OPEN, CLOSE = "<|open|>tools<|sep|>", "<|close|>tools<|sep|>"
    SEP = "<|sep|>"
    WRAPPERS = ("<|open|>response<|sep|>", "<|close|>response<|sep|>", "<|close|>message<|sep|>")
    ATTR = re.compile(r'(\w+)="([^"]*)"')

    @classmethod
    def _blocks(cls, text: str, open_: str, close: str):
        pos = 0
        while True:
            i = text.find(open_, pos)
            if i < 0:
                return
            start = i + len(open_)
            rest = text[start:]
            attrs_at = len(rest) - len(rest.lstrip())
            if attrs_at == 0:                       # the marker must be followed by white space
                pos = start
                continue
            sep = rest.find(cls.SEP, attrs_at)
            if sep < 0:
                return
            body = rest[sep + len(cls.SEP):]
            end = body.find(close)
            if end < 0:
                return
            yield rest[attrs_at:sep], body[:end]
            pos = start + sep + len(cls.SEP) + end + len(close)

    @classmethod
    def _attr(cls, attrs: str, name: str) -> Optional[str]:
        vals = [v for k, v in cls.ATTR.findall(attrs) if k == name]
        return vals[-1].replace("&quot;", '"').replace("&amp;", "&") if vals else None

    def parse_body(self, body: str):
        out = []
        for attrs, inner in self._blocks(body, "<|open|>call", "<|close|>call<|sep|>"):
            name = self._attr(attrs, "tool")
            if not name:
                continue
            args: Dict[str, Any] = {}
            for a_attrs, raw in self._blocks(inner, "<|open|>argument", "<|close|>argument<|sep|>"):
                typ = self._attr(a_attrs, "type") or "string"
                args[self._attr(a_attrs, "key") or ""] = raw if typ == "string" else _json_or_text(raw)
            out.append(ToolCall(name, json.dumps(args, ensure_ascii=False)))
        return out

    def _unwrap(self, text: str) -> str:
        for w in self.WRAPPERS:
            text = text.replace(w, "")
        return text

    def push(self, text: str):
        content, calls = super().push(text)
        # a wrapper marker cut by the delta boundary stays in the buffer until it is whole
        content = self._held + content
        keep = 0
        for w in self.WRAPPERS:
            for k in range(min(len(w) - 1, len(content)), keep, -1):
                if content.endswith(w[:k]):
                    keep = k
                    break
        self._held = content[len(content) - keep:] if keep else ""
        return self._unwrap(content[:len(content) - keep] if keep else content), calls

    def flush(self):
        content, calls = super().flush()
        content, self._held = self._held + content, ""
        return self._unwrap(content), calls

    _held = ""


class GlmToolParser(ToolParser):
    """GLM: the function name on the first line, then ``<arg_key>``/``<arg_value>`` pairs; values of parameters whose
    schema type is not ``string`` are JSON."""
    PAIR = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)

    def parse_body(self, body: str):
        head = body.split("<arg_key>", 1)[0].strip()
        if not head:
            return None
        name = head.splitlines()[0].strip()
        props: Dict[str, Any] = {}
        for t in self.tools:
            f = t.get("function", t)
            if f.get("name") == name:
                props = (f.get("parameters") or {}).get("properties") or {}
        args: Dict[str, Any] = {}
        for k, v in self.PAIR.findall(body):
            k = k.strip()
            typ = (props.get(k) or {}).get("type")
            args[k] = v if typ == "string" else _json_or_text(v.strip()) if typ else _json_or_text(v)
        return ToolCall(name, json.dumps(args, ensure_ascii=False))


def get_tool_parser(name: str, tools=None) -> ToolParser:
    name = (name or "hermes").lower()
    if name in ("hermes", "qwen", "qwen3", "qwen25", "json"):
        return HermesToolParser(tools)
    if name in ("qwen3_coder", "qwen3-coder", "xml"):
        return Qwen3CoderToolParser(tools)
    if name in ("deepseek", "deepseek_v4", "deepseekv4", "dsml"):
        return DsmlToolParser(tools)
    if name in ("deepseek_v41", "deepseekv41"):
        return DsmlToolParser(tools, spaced=True)
    if name in ("kimi", "kimi_k3", "kimik3"):
        return KimiToolParser(tools)
    if name in ("glm", "glm45", "glm53"):
        return GlmToolParser(tools)
    raise ValueError(f"unknown tool-call parser {name!r}")
