"""Request fields the prompt renderers share: the reasoning toggle and effort an OpenAI-style request implies, lenient
booleans, which tools a ``tool_choice`` lets the prompt show, and JSON-schema type names as the model families expect them.
Reference: ``crates/blaze-chat/src/render/reasoning.rs``, ``render/models/schema_types.rs``, ``render/models/deepseek_v4.rs``
(``pydantic_bool``, ``renders_tools``)."""
from __future__ import annotations

import copy
from typing import Any, Dict, List, Optional


def truthy(v: Any) -> bool:
    """Template truthiness of a JSON value: empty strings, containers, zero and null are false."""
    return bool(v)


def pydantic_bool(v: Any) -> bool:
    """Lenient boolean of request validation: true/false, 0/1, and the usual words; anything else is an error."""
    if isinstance(v, bool):
        return v
    if isinstance(v, (int, float)) and v in (0, 1):
        return bool(v)
    if isinstance(v, str):
        s = v.lower()
        if s in ("0", "off", "f", "false", "n", "no"):
            return False
        if s in ("1", "on", "t", "true", "y", "yes"):
            return True
    raise ValueError(f"Input should be a valid boolean, got {v!r}")


def wide_int(text: str):
    """``parse_int`` hook for request JSON: integers beyond 64 bits arrive as floats."""
    n = int(text)
    return n if -(1 << 63) <= n < (1 << 64) else float(n)


def effort_of(request: Dict[str, Any]) -> Any:
    """``reasoning.effort``, then ``reasoning.reasoning_effort``, then the top-level ``reasoning_effort``."""
    r = request.get("reasoning")
    r = r if isinstance(r, dict) else {}
    for v in (r.get("effort"), r.get("reasoning_effort"), request.get("reasoning_effort")):
        if v is not None:
            return v
    return None


def thinking_requested(request: Dict[str, Any]) -> Optional[bool]:
    """An effort turns thinking off only when it is "none"; without one a truthy ``reasoning.enabled`` turns it on."""
    e = effort_of(request)
    if e is not None:
        return e != "none"
    r = request.get("reasoning")
    r = r if isinstance(r, dict) else {}
    v = r.get("enabled") if r.get("enabled") is not None else r.get("enable")
    if v is None:
        return None
    on = v.strip().lower() in ("1", "true", "yes", "y", "on") if isinstance(v, str) else truthy(v)
    return True if on else None


def renders_tools(request: Dict[str, Any], tools: List[Any]) -> bool:
    """``tool_choice`` "none" hides the tools; a named choice shows all of them when it names one of them."""
    choice = request.get("tool_choice")
    if choice is None:
        return True
    if isinstance(choice, str):
        return choice != "none"
    name = ((choice.get("function") or {}).get("name") if isinstance(choice, dict) else None)
    return any(isinstance(t, dict) and (t.get("function") or {}).get("name") == name for t in tools)


_STANDARD = ("null", "boolean", "object", "array", "number", "string", "integer")
_ALIASES = {**{k: "string" for k in ("str", "text", "varchar", "char", "enum", "uuid", "date", "datetime", "time", "timestamp",
                                      "binary", "blob", "bytea", "bytes", "varbinary")},
            "bool": "boolean", "bigint": "integer", "smallint": "integer", "tinyint": "integer",
            "double": "number", "decimal": "number", "real": "number", "numeric": "number",
            "arr": "array", "tuple": "array", "set": "array", "map": "object"}
_PREFIXES = ((("int", "uint", "long", "short", "unsigned"), "integer"), (("num", "float"), "number"), (("list",), "array"),
             (("dict",), "object"))
_BOUNDARY = "0123456789[<( \t"
_MAPS = ("properties", "patternProperties", "$defs", "definitions", "dependentSchemas")
_LISTS = ("anyOf", "oneOf", "allOf", "prefixItems")
_VALUES = ("items", "additionalProperties", "not", "if", "then", "else", "contains", "propertyNames", "unevaluatedItems",
           "unevaluatedProperties")


def _normalize_type(raw: str) -> Optional[str]:
    if raw in _STANDARD:
        return None
    base = raw.split("(")[0].strip(" \t\n\r\x0b\x0c\x1c\x1d\x1e\x1f").lower()
    if base in _STANDARD:
        return base
    if base in _ALIASES:
        return _ALIASES[base]
    for prefixes, target in _PREFIXES:
        for p in prefixes:
            if base == p or (base.startswith(p) and base[len(p):len(p) + 1] and base[len(p)] in _BOUNDARY):
                return target
    return None


def _walk(s: Any) -> None:
    if isinstance(s, list):
        for x in s:
            _walk(x)
        return
    if not isinstance(s, dict):
        return
    t = s.get("type")
    if isinstance(t, str):
        n = _normalize_type(t)
        if n is not None:
            s["type"] = n
    elif isinstance(t, list):
        out: List[Any] = []
        for x in t:
            n = _normalize_type(x) if isinstance(x, str) else None
            x = n if n is not None else x
            if x not in out:
                out.append(x)
        s["type"] = out
    for k in _MAPS:
        if isinstance(s.get(k), dict):
            for v in s[k].values():
                _walk(v)
    for k in _LISTS:
        if isinstance(s.get(k), list):
            for v in s[k]:
                _walk(v)
    for k in _VALUES:
        if k in s:
            _walk(s[k])


def normalize_schema_types(schema: Any) -> Any:
    """A copy of a JSON schema with database / Python style type names ("varchar(255)", "Int32", "list[str]") rewritten
    to the JSON-schema names."""
    schema = copy.deepcopy(schema)
    _walk(schema)
    return schema


def engine_message(m: Any) -> Dict[str, Any]:
    """The fields the serving layer keeps: lower-case role, no null fields, ``user`` reduced to its content."""
    m = dict(m) if isinstance(m, dict) else {}
    role = str(m.get("role") or "").lower()
    kept = ("content",) if role == "user" else ("content", "tool_call_id", "name", "reasoning_content", "tool_calls", "tools")
    out = {k: v for k, v in m.items() if k in kept and v is not None}
    out["role"] = role
    out.setdefault("content", "")
    if isinstance(out.get("tool_calls"), list):
        calls = []
        for c in out["tool_calls"]:
            c = c if isinstance(c, dict) else {}
            f = c.get("function") if isinstance(c.get("function"), dict) else {}
            calls.append({"id": c.get("id"), "index": c.get("index"), "type": "function",
                          "function": {"name": f.get("name"), "arguments": f.get("arguments")}})
        out["tool_calls"] = calls
    return out


def split_continuation(messages: List[Dict[str, Any]], request: Dict[str, Any]) -> str:
    """A final assistant turn with text content is either the prefix to continue or, without the flag, a user turn."""
    if not messages or messages[-1]["role"] != "assistant" or not isinstance(messages[-1]["content"], str):
        return ""
    content = messages[-1]["content"]
    flag = request.get("continue_final_message")
    if flag is not None and pydantic_bool(flag):
        messages.pop()
        return content
    messages[-1] = {"role": "user", "content": content}
    return ""


def normalize_tools(tools: List[Any]) -> List[Dict[str, Any]]:
    """Request tools as the serving layer dumps them: description, name, parameters (type names normalised), strict,
    and ``defer_loading`` when the function or the tool sets it."""
    out = []
    for t in tools:
        f = t.get("function") if isinstance(t, dict) and isinstance(t.get("function"), dict) else {}
        if not isinstance(f.get("name"), str):
            raise ValueError("tool function requires name")
        fn: Dict[str, Any] = {"description": f.get("description"), "name": f["name"],
                              "parameters": normalize_schema_types(f.get("parameters"))}
        fn["strict"] = pydantic_bool(f["strict"]) if "strict" in f else False
        defer = next((v for v in (f.get("defer_loading"), t.get("defer_loading")) if v is not None), None)
        if defer is not None:
            fn["defer_loading"] = pydantic_bool(defer)
        out.append({"type": "function", "function": fn})
    return out
