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
            keep = not (self.DROP_TEXT_AFTER_CALLS and self.calls)
            if i >= 0:
                if keep:
                    content += self.buf[:i].rstrip("\n") if not self.buf[:i].strip() else self.buf[:i]
                self.buf = self.buf[i + len(self.OPEN):]
                self.inside = True
                continue
            h = self._hold(self.OPEN)
            if keep:
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
        return ("" if self.DROP_TEXT_AFTER_CALLS and self.calls else out), []

    DROP_TEXT_AFTER_CALLS = False        # families whose answer text ends where the first call begins


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


def _schema_kind(spec: Any) -> Optional[str]:
    """The JSON type a parameter's schema asks for: its ``type`` (the first one that is not "null" of a list), the first
    typed alternative of ``anyOf`` / ``oneOf``, a non-string member of ``allOf``, "enum" for an enumeration, and object /
    array where only ``properties`` / ``items`` say so."""
    if not isinstance(spec, dict):
        return None
    t = spec.get("type")
    if isinstance(t, list):
        t = next((x for x in t if x != "null"), t[0] if t else None)
    if isinstance(t, str):
        return t.strip().lower()
    for key in ("anyOf", "oneOf"):
        for alt in spec.get(key) or []:
            k = _schema_kind(alt)
            if k and k != "null":
                return k
    kinds = [k for k in (_schema_kind(a) for a in spec.get("allOf") or []) if k]
    if kinds:
        return next((k for k in kinds if k not in ("string", "null")), kinds[0])
    if "enum" in spec:
        return "enum"
    if "properties" in spec:
        return "object"
    if "items" in spec:
        return "array"
    return None


def _typed_value(raw: str, spec: Any) -> Any:
    """A parameter's text as the value its schema asks for (``_schema_kind``); text that does not read as that type stays
    a string.  Integers and numbers read as Python does (underscores, any Unicode digits, inf / nan); a number written
    without a point or exponent becomes an integer; objects, arrays and untyped values read as JSON, then as a Python
    literal (single quotes, tuples, None / True / False)."""
    import ast
    if raw.lower() == "null":
        return None
    kind = _schema_kind(spec)
    if kind is None or kind in ("string", "str", "text", "varchar", "char"):
        return raw
    if kind == "enum":
        try:
            v = json.loads(raw)
        except ValueError:
            return raw
        return v if any(v == e and type(v) is type(e) for e in spec["enum"]) else raw
    if kind.startswith(("int", "uint", "long", "short", "unsigned")):
        try:
            return int(raw)
        except ValueError:
            return raw
    if kind.startswith(("num", "float", "double")):
        try:
            f = float(raw)
        except ValueError:
            return raw
        whole = "." not in raw and "e" not in raw.lower()
        return int(f) if whole and f == f and f not in (float("inf"), float("-inf")) and f.is_integer() else f
    if kind in ("boolean", "bool", "binary"):
        return raw.lower() == "true"
    depth = deepest = 0
    for ch in raw:
        if ch in "[({":
            depth += 1
            deepest = max(deepest, depth)
        elif ch in "])}":
            depth -= 1
    if deepest > 200:                    # nesting beyond what a literal may have
        return raw
    if kind in ("object", "array", "dict", "list", "arr", "map"):
        try:
            return json.loads(raw)
        except (ValueError, RecursionError):
            pass
    try:
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # odd escapes in the text are not this process's concern
            v = ast.literal_eval(raw)
        json.dumps(v)                    # sets, bytes, complex numbers have no JSON form
        return v
    except (ValueError, SyntaxError, TypeError, MemoryError, RecursionError):
        return raw


class Qwen3CoderToolParser(ToolParser):
    """``<tool_call>`` around one or more ``<function=name>`` elements with ``<parameter=key>`` children; values are typed
    by the request's tool schemas (``_typed_value``)."""
    DROP_TEXT_AFTER_CALLS = True
    FN = re.compile(r"<function=([^>\s]+)>(.*?)(?:</function>|(?=<function=)|$)", re.S)
    PARAM = re.compile(r"<parameter=([^>]+)>(.*?)(?:</parameter>|(?=<parameter=)|$)", re.S)

    def _schema(self, fn: str) -> Dict[str, Any]:
        for t in self.tools:
            f = t.get("function", t)
            if f.get("name") == fn:
                params = f.get("parameters")
                if not isinstance(params, dict):
                    return {}
                if isinstance(params.get("properties"), dict):
                    return params["properties"]
                merged: Dict[str, Any] = {}
                for alt in (params.get("anyOf") or []) + (params.get("oneOf") or []):     # first alternative that has the key
                    for k, v in ((alt.get("properties") or {}) if isinstance(alt, dict) else {}).items():
                        merged.setdefault(k, v)
                return merged or params
        return {}

    def parse_body(self, body: str):
        out = []
        for m in self.FN.finditer(body):
            name, inner = m.group(1), m.group(2)
            props = self._schema(name)
            args: Dict[str, Any] = {}
            for pm in self.PARAM.finditer(inner):
                key, raw = pm.group(1), pm.group(2)
                raw = raw[1:] if raw.startswith("\n") else raw
                raw = raw[:-1] if raw.endswith("\n") else raw
                args[key] = _typed_value(raw, props.get(key))
            out.append(ToolCall(name, json.dumps(args, ensure_ascii=False)))
        return out


class DsmlToolParser(ToolParser):
    """DeepSeek's DSML calls: ``<｜DSML｜tool_calls>`` around ``<｜DSML｜invoke name="...">`` elements whose arguments are
    ``<｜DSML｜parameter name="..." string="true|false">`` children (``string="false"`` values are JSON) or one JSON object
    as the element's text.  V4.1 spells the tags with a space (``｜DSML｜ calls``, ``｜DSML｜ invoke``).  Text before the
    first call is the answer (trailing white space dropped once a call follows); text after the calls is dropped; a bare
    invoke without the wrapper counts; an invoke with a malformed parameter is dropped.  ``parse`` (whole output) keeps only
    calls to the request's tools, the stream keeps all (the caller validates names)."""
    MARK = "｜DSML｜"

    def __init__(self, tools=None, spaced: bool = False):
        super().__init__(tools)
        block, inv, par = (" calls", " invoke", " parameter") if spaced else ("tool_calls", "invoke", "parameter")
        m = re.escape(self.MARK)
        self.OPEN, self.CLOSE = f"<{self.MARK}{block}>", f"</{self.MARK}{block}>"
        self.INV_OPEN = f"<{self.MARK}{inv}"
        self.INVOKE = re.compile(rf'<{m}{re.escape(inv)}\s+name="([^"]+)"\s*(?:/>|>(.*?)</{m}{re.escape(inv)}>)', re.S)
        self.PARAM = re.compile(rf'<{m}{re.escape(par)}\s+name="([^"]+)"\s+string="(true|false)"\s*>(.*?)</{m}{re.escape(par)}>', re.S)
        self.ANY_PARAM = f"<{self.MARK}{par}"
        self.names = {(t.get("function") or t).get("name") for t in self.tools if isinstance(t, dict)}
        self.started = False            # a call marker was seen: the answer text is over
        self.space = ""                 # trailing white space of the answer, held until more text or a call follows

    def _call_of(self, m, verbatim: bool) -> Optional[ToolCall]:
        body = m.group(2) or ""
        params = self.PARAM.findall(body)
        if body.count(self.ANY_PARAM) != len(params):
            return None                 # a parameter without the string attribute, or cut
        if not params and body.strip().startswith("{"):
            try:
                obj = json.loads(body.strip())
            except ValueError:
                return None
            if not isinstance(obj, dict):
                return None
            return ToolCall(m.group(1), body.strip() if verbatim else json.dumps(obj, ensure_ascii=False))
        args: Dict[str, Any] = {}
        for key, is_str, raw in params:
            args[key] = raw if is_str == "true" else _json_or_text(raw.strip())
        return ToolCall(m.group(1), json.dumps(args, ensure_ascii=False))

    def _first_marker(self, text: str) -> int:
        found = [i for i in (text.find(self.OPEN), text.find(self.INV_OPEN)) if i >= 0]
        return min(found) if found else -1

    def parse(self, text: str) -> Tuple[str, List[ToolCall]]:
        """The whole output at once."""
        i = self._first_marker(text)
        if i < 0:
            return text, []
        calls = [c for c in (self._call_of(m, False) for m in self.INVOKE.finditer(text, i)) if c is not None]
        return text[:i].strip(), [c for c in calls if not self.names or c.name in self.names]

    def push(self, text: str) -> Tuple[str, List[ToolCall]]:
        self.buf += text
        content, done = "", []
        if not self.started:
            i = self._first_marker(self.buf)
            if i >= 0:
                content, self.buf, self.started, self.space = self.space + self.buf[:i], self.buf[i:], True, ""
                content = content.rstrip()
            else:
                hold = max(_partial_tail(self.buf, self.OPEN), _partial_tail(self.buf, self.INV_OPEN))
                out, self.buf = self.space + self.buf[:len(self.buf) - hold], self.buf[len(self.buf) - hold:]
                kept = out.rstrip()
                content, self.space = kept, out[len(kept):]
                return content, done
        while True:
            m = self.INVOKE.search(self.buf)
            if m is None:
                break
            call = self._call_of(m, True)
            if call is not None:
                done.append(call)
                self.calls.append(call)
            self.buf = self.buf[m.end():]
        return content, done

    def flush(self) -> Tuple[str, List[ToolCall]]:
        out, self.buf = self.buf, ""
        if self.started:
            return "", []               # a cut call, or text after the calls
        out, self.space = self.space + out, ""
        return out, []


def _partial_tail(text: str, marker: str) -> int:
    for k in range(min(len(marker) - 1, len(text)), 0, -1):
        if text.endswith(marker[:k]):
            return k
    return 0


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

    def parse(self, text: str):
        """The whole output at once: without a tools channel the text is returned as it is; with one, the answer is the
        response channel's text before it and the calls are those of the first channel."""
        from .reasoning import _k_unwrap
        i = text.find(self.OPEN)
        if i < 0:
            return text, []
        body = text[i + len(self.OPEN):]
        j = body.find(self.CLOSE)
        return _k_unwrap(text[:i]), _as_list(self.parse_body(body if j < 0 else body[:j]))

    def push(self, text: str):
        self.buf += text
        content, done = "", []
        while self.buf:
            if self.inside:
                i = self.buf.find(self.CLOSE)
                if i < 0:
                    break
                calls = _as_list(self.parse_body(self.buf[:i]))
                done.extend(calls)
                self.calls.extend(calls)
                self.buf, self.inside, self.after = self.buf[i + len(self.CLOSE):], False, True
                continue
            i = self.buf.find(self.OPEN)
            if i >= 0:
                if not self.after:
                    content += self.buf[:i]
                self.buf, self.inside = self.buf[i + len(self.OPEN):], True
                continue
            # a marker cut by the delta boundary stays in the buffer until it is whole
            hold = max(_partial_tail(self.buf, m) for m in (self.OPEN,) + self.WRAPPERS)
            if not self.after:
                content += self.buf[:len(self.buf) - hold]
            self.buf = self.buf[len(self.buf) - hold:]
            break
        return self._unwrap(content), done

    def flush(self):
        from .reasoning import _k_strip_cut
        out, self.buf = self.buf, ""
        if self.inside:                  # the channel was never closed: the calls that are whole still count
            self.inside = False
            calls = _as_list(self.parse_body(out))
            self.calls.extend(calls)
            return "", calls
        return ("" if self.after else _k_strip_cut(self._unwrap(out))), []

    after = False                        # a tools channel has closed: later text is not part of the answer


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
