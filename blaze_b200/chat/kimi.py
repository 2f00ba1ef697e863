"""Kimi-K3 prompt encoder (XTML markers: ``<|open|>tag attr="..."<|sep|> ... <|close|>tag<|sep|>``).

The prompt is a list of messages, each closed by ``<|close|>message<|sep|><|end_of_msg|>``: a tool declaration, a note with
the thinking effort, the conversation (assistant turns carry think / response / tools channels, tool results name their
call), then notes for a forced tool choice and a JSON response format, then the opened assistant turn.
Request preparation follows ``crates/blaze-chat/src/render/models/kimi_k3.rs``; the markers are those of
``crates/blaze-chat/src/kimi_k3_format.rs``; the layout is pinned by ``crates/blaze-chat/tests/fixtures/parity/kimi-k3.json``."""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional, Tuple

from .request import effort_of, normalize_schema_types, pydantic_bool, thinking_requested, truthy, wide_int

O, C, S = "<|open|>", "<|close|>", "<|sep|>"
MSG_END = f"{C}message{S}<|end_of_msg|>"
IMAGE = "<|kimi_image_placeholder|>"
EFFORTS = ("low", "high", "max")
_MEDIA = ("image_url", "video_url", "audio_url", "input_audio")
_RESERVED_KWARGS = ("conversation", "messages", "tools", "add_generation_prompt")


def _esc(v: Any) -> str:
    return str(v).replace("&", "&amp;").replace('"', "&quot;")


def _neutral(v: Any) -> Any:
    """The image placeholder typed as text must not read as the special token."""
    if isinstance(v, str):
        return v.replace(IMAGE, "<| kimi_image_placeholder |>")
    if isinstance(v, list):
        return [_neutral(x) for x in v]
    if isinstance(v, dict):
        return {k: _neutral(x) for k, x in v.items()}
    return v


def _compact(v: Any) -> str:
    return json.dumps(v, ensure_ascii=False, sort_keys=True, separators=(",", ":"))


def _tool_dump(tool: Any) -> Dict[str, Any]:
    tool = tool if isinstance(tool, dict) else {}
    f = tool.get("function") if isinstance(tool.get("function"), dict) else {}
    if not isinstance(f.get("name"), str):
        raise ValueError("tool function requires name")
    fn: Dict[str, Any] = {k: f[k] for k in ("name", "description", "parameters") if k in f}
    if "parameters" in fn:
        fn["parameters"] = normalize_schema_types(fn["parameters"])
    if "strict" in f:
        fn["strict"] = pydantic_bool(f["strict"])
    defer = next((v for v in (f.get("defer_loading"), tool.get("defer_loading")) if v is not None), None)
    if defer is not None:
        fn["defer_loading"] = pydantic_bool(defer)
    out: Dict[str, Any] = {}
    if "type" in tool:
        out["type"] = tool["type"]
    out["function"] = fn
    if "defer_loading" in tool:
        out["defer_loading"] = None if tool["defer_loading"] is None else pydantic_bool(tool["defer_loading"])
    return out


def _prepare(m: Any, index: int) -> Dict[str, Any]:
    m = dict(m) if isinstance(m, dict) else {}
    role = str(m.get("role") or "").lower()
    kept = ("content",) if role == "user" else ("content", "tool_call_id", "name", "reasoning_content", "tool_calls", "tools")
    out = {k: v for k, v in m.items() if k in kept and v is not None}
    out["role"] = "system" if role == "developer" else role
    if out["role"] not in ("system", "user", "assistant", "tool"):
        raise ValueError(f"Unknown message role {role!r} at index {index}.")
    content = out.get("content", "")
    if isinstance(content, list):
        for p in content:
            t = p.get("type") if isinstance(p, dict) else None
            if t in _MEDIA:
                raise ValueError(f"Model only supports text input; received unsupported content type {t!r}.")
        out["content"] = [p for p in content if isinstance(p, dict) and p.get("type") == "text"]
    else:
        out["content"] = content
    out["content"] = _neutral(out["content"])
    if "reasoning_content" in out:
        out["reasoning_content"] = _neutral(out["reasoning_content"])
    calls = []
    for c in (out.get("tool_calls") or []) if out["role"] == "assistant" else []:
        c = c if isinstance(c, dict) else {}
        f = c.get("function") if isinstance(c.get("function"), dict) else {}
        a = f.get("arguments")
        if isinstance(a, str):
            try:
                parsed = json.loads(a, parse_int=wide_int)
                if isinstance(parsed, dict):
                    a = parsed
            except ValueError:
                pass
        calls.append({"id": c.get("id"), "name": f.get("name"), "arguments": _neutral(a)})
    out["tool_calls"] = calls
    tools = out.pop("tools", None)
    if out["role"] == "system" and isinstance(tools, list) and tools:
        out["tools"] = [_tool_dump(t) for t in tools]
        out["content"] = ""
    return out


def _text(content) -> str:
    if isinstance(content, list):
        return "".join(p.get("text") or "" for p in content)
    return content or ""


def _value_type(v: Any) -> str:
    if isinstance(v, str):
        return "string"
    if isinstance(v, bool):
        return "boolean"
    if isinstance(v, (int, float)):
        return "number"
    if v is None:
        return "null"
    return "array" if isinstance(v, list) else "object"


def _call(c: Dict[str, Any], index: int) -> str:
    out = [f'{O}call tool="{_esc(c["name"])}" index="{index}"{S}']
    a = c["arguments"]
    if isinstance(a, dict):
        for k, v in a.items():
            out.append(f'{O}argument key="{_esc(k)}" type="{_value_type(v)}"{S}'
                       + (v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)) + f"{C}argument{S}")
    elif isinstance(a, str) and a:
        out.append(f'{O}json type="object"{S}{a}{C}json{S}')          # not a JSON object: passed through as text
    out.append(f"{C}call{S}")
    return "".join(out)


def _response_format_dump(fmt: Any) -> Optional[Dict[str, Any]]:
    if not isinstance(fmt, dict) or "type" not in fmt:
        return None
    kind = fmt["type"]
    js = None
    if isinstance(fmt.get("json_schema"), dict) and fmt["json_schema"]:
        js = {k: v for k, v in fmt["json_schema"].items() if k in ("name", "description", "schema", "strict")}
    elif kind == "json_schema" and isinstance(fmt.get("schema"), dict) and fmt["schema"]:
        schema = dict(fmt["schema"])
        if isinstance(schema.get("properties"), dict):
            schema["properties"] = {k: v for k, v in schema["properties"].items() if k != "strict"}
        js = {"schema": schema}
    out = {"type": kind}
    if js is not None:
        out["json_schema"] = js
    return out


def render_request(request: Dict[str, Any], defaults: Optional[Dict[str, Any]] = None) -> Tuple[str, str]:
    """``(prompt, continuation prefix)`` of a chat request."""
    defaults = defaults or {}
    raw = request.get("messages")
    if not isinstance(raw, list):
        raise ValueError("messages must be an array")
    messages = [_prepare(m, i) for i, m in enumerate(raw)]
    prefix = ""
    flag = request.get("continue_final_message")
    if (flag is not None and pydantic_bool(flag) and messages and messages[-1]["role"] == "assistant"
            and isinstance(messages[-1]["content"], str)):
        prefix = messages.pop()["content"]

    kwargs = dict(request.get("chat_template_kwargs") or {})
    kw_effort = kwargs.pop("reasoning_effort", None)
    t = thinking_requested(request)
    if t is not None:
        kwargs.setdefault("thinking", t)
    for k, v in defaults.items():
        kwargs.setdefault(k, v)
    for k in _RESERVED_KWARGS:
        if k in kwargs:
            raise TypeError(f"got multiple values for keyword argument {k!r}")
    thinking = truthy(kwargs["thinking"]) if "thinking" in kwargs else True
    effort = kw_effort if kw_effort is not None else effort_of(request)
    if effort is None:
        effort = defaults.get("reasoning_effort")
    thinking_effort = kwargs["thinking_effort"] if "thinking_effort" in kwargs else (effort if effort in EFFORTS else "max")
    if thinking and thinking_effort is not None and thinking_effort not in EFFORTS:
        raise ValueError(f"Unsupported thinking_effort={thinking_effort!r}; supported values are {sorted(EFFORTS)}.")

    tools = [_tool_dump(t_) for t_ in request["tools"]] if isinstance(request.get("tools"), list) and request["tools"] else None
    has_tools = tools is not None or any("tools" in m for m in messages)
    choice = request.get("tool_choice")
    if not has_tools and isinstance(choice, str) and choice.lower() == "required":
        raise ValueError("Tools cannot be empty if tool choice is set to required.")
    if has_tools and choice in ("required", "none"):
        kwargs.setdefault("tool_choice", choice)
    shown_choice = kwargs.get("tool_choice") if kwargs.get("tool_choice") in ("required", "none") else None

    req_format = _response_format_dump(request.get("response_format"))
    if req_format and req_format["type"] == "json_schema" and (req_format.get("json_schema") or {}).get("schema") is None:
        raise ValueError("schema_ is required for json_schema response format request.")
    rf = kwargs.get("response_format")
    fmt = {"type": rf} if isinstance(rf, str) else dict(rf) if isinstance(rf, dict) else req_format
    if fmt is not None and "response_schema" in kwargs:
        fmt["json_schema"] = {"schema": kwargs["response_schema"]}

    out: List[str] = []
    if tools is not None:
        out.append(f'{O}message role="system" type="tool-declare"{S}# Tools\nHere are the available tools, described in '
                   f"JSONSchema.\n\n```json\n{_compact(tools)}\n```{MSG_END}")
    if thinking and thinking_effort is not None:
        out.append(f'{O}message role="system" type="thinking-effort"{S}`thinking_effort` guides on how much to think in your '
                   "thinking channel (not including the response channel), supported values include `low`, `medium`, `high`, "
                   f"and `max`.\nNow the system is invoked with `thinking_effort={thinking_effort}`.{MSG_END}")
    i, n = 0, len(messages)
    pending: List[Dict[str, Any]] = []
    while i < n:
        m = messages[i]
        role = m["role"]
        name = f' name="{_esc(m["name"])}"' if m.get("name") is not None and role != "tool" else ""
        if role == "system" and "tools" in m:
            out.append(f'{O}message role="system" type="tool-declare"{S}## New Tools Available\nThe system dynamically extends '
                       "the toolset via lazy-loading.\nYou have access to all existing and extended tools.\nHere are the specs "
                       f"for the extended tools.\n\n```json\n{_compact(m['tools'])}\n```{MSG_END}")
        elif role in ("system", "user"):
            out.append(f'{O}message role="{role}"{name}{S}{_text(m["content"])}{MSG_END}')
        elif role == "assistant":
            body = [f'{O}message role="assistant"{name}{S}']
            if thinking:
                body.append(f'{O}think{S}{m.get("reasoning_content") or ""}{C}think{S}')
            body.append(f'{O}response{S}{_text(m["content"])}{C}response{S}')
            pending = [dict(c, index=k + 1) for k, c in enumerate(m["tool_calls"])]
            if pending:
                body.append(f"{O}tools{S}" + "".join(_call(c, c["index"]) for c in pending) + f"{C}tools{S}")
            out.append("".join(body) + MSG_END)
        else:
            # the run of tool results that answers the calls above, in the order of the calls
            run = []
            j = i
            while j < n and messages[j]["role"] == "tool":
                tm = messages[j]
                call = next((c for c in pending if tm.get("tool_call_id") is not None and c["id"] == tm["tool_call_id"]), None)
                if call is None and j - i < len(pending) and tm.get("tool_call_id") is None:
                    call = pending[j - i]
                tool_name = tm["name"] if tm.get("name") is not None else call["name"] if call else None
                if tool_name is None:
                    raise ValueError("Kimi K3 tool messages need a resolvable tool name: carry `tool`/`name`, or match a "
                                     "preceding assistant tool_call by order.")
                idx = call["index"] if call else j - i + 1
                run.append((idx, f'{O}message role="tool" tool="{_esc(tool_name)}" index="{idx}"{S}{_text(tm["content"])}{MSG_END}'))
                j += 1
            run.sort(key=lambda r: r[0])
            out.extend(r[1] for r in run)
            pending = []
            i = j
            continue
        if role != "assistant":
            pending = []
        i += 1
    if shown_choice is not None:
        out.append(f'{O}message role="system" type="tool-choice"{S}The system is invoked with `tool_choice={shown_choice}`.\n'
                   + ("You MUST call tools in the next message." if shown_choice == "required"
                      else "You MUST NOT call any tools in the next message.") + MSG_END)
    if fmt is not None and fmt.get("type") in ("json_object", "json_schema"):
        text = (f"The system is invoked with `response_format={fmt['type']}`.\nYour response must be raw JSON data without "
                "markdown code blocks (```json) or any additional formatting.")
        schema = (fmt.get("json_schema") or {}).get("schema") if isinstance(fmt.get("json_schema"), dict) else None
        if fmt["type"] == "json_schema" and schema is not None:
            text += f"\nThe JSON data must match the following schema:\n```json\n{_compact(schema)}\n```"
        out.append(f'{O}message role="system" type="response-format"{S}{text}{MSG_END}')
    out.append(f'{O}message role="assistant"{S}' + (f"{O}think{S}" if thinking else f"{O}response{S}"))
    return "".join(out), prefix
