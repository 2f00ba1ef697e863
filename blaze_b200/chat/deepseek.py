"""DeepSeek-V4 and DeepSeek-V4.1 prompt encoders.

These families ship no Jinja template: the prompt is built by an encoder that merges user and tool-result turns into one
user block, writes tool calls as DSML elements, keeps or drops earlier reasoning, and prefixes a reasoning-effort note.
``render_request`` takes the OpenAI request body and returns ``(prompt, prefix)``: ``prefix`` is the text of a final
assistant turn that ``continue_final_message`` asked to continue (it is tokenised on its own, after the prompt).
Behaviour follows ``crates/blaze-chat/src/render/models/deepseek_v4.rs`` and ``deepseek_v41.rs`` (request preparation) and
the golden prompts of ``crates/blaze-chat/tests/fixtures/parity/deepseek-v4*.json`` (the encoders' output)."""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional, Tuple

from .request import (effort_of, engine_message, normalize_tools, pydantic_bool, renders_tools, split_continuation,
                      thinking_requested, truthy, wide_int)

BOS, EOS = "<｜begin▁of▁sentence｜>", "<｜end▁of▁sentence｜>"
USER, ASSISTANT, SYSTEM = "<｜User｜>", "<｜Assistant｜>", "<｜System｜>"
IMAGE_TOKEN = "<｜deepseek_image｜>"

_TOOLS_HEAD = (
    "## Tools\n\nYou have access to a set of tools to help answer the user's question. You can invoke tools by writing a "
    "\"<{calls}>\" block like the following:\n\n<{calls}>\n<{invoke} name=\"$TOOL_NAME\">\n<{param} name=\"$PARAMETER_NAME\" "
    "string=\"true|false\">$PARAMETER_VALUE</{param}>\n...\n</{invoke}>\n<{invoke} name=\"$TOOL_NAME2\">\n...\n</{invoke}>\n"
    "</{calls}>\n\nString parameters should be specified as is and set `string=\"true\"`. For all other types (numbers, "
    "booleans, arrays, objects), pass the value in JSON format and set `string=\"false\"`.\n\nIf thinking_mode is enabled "
    "(triggered by <think>), you MUST output your complete reasoning inside <think>...</think> BEFORE any tool calls or final "
    "response.\n\nOtherwise, output directly after </think> with tool calls or final response.\n\n### Available Tool Schemas\n\n"
    "{schemas}\n\nYou MUST strictly follow the above defined tool name and parameter schemas to invoke tool calls.\n")

_EFFORT_HIGH = (
    "Reasoning Effort: Absolute maximum with no shortcuts permitted.\nYou MUST be very thorough in your thinking and "
    "comprehensively decompose the problem to resolve the root cause, rigorously stress-testing your logic against all "
    "potential paths, edge cases, and adversarial scenarios.\nExplicitly write out your entire deliberation process, "
    "documenting every intermediate step, considered alternative, and rejected hypothesis to ensure absolutely no assumption "
    "is left unchecked.\n\n")
_EFFORT_MAX = (
    "Reasoning Effort: Beyond maximum — exhaustive, relentless, and uncompromising.\nYou MUST reason with the utmost depth and "
    "rigor, leaving absolutely nothing to chance: exhaustively decompose the problem into its most fundamental components, "
    "trace every causal chain to its root, and resolve the underlying cause rather than any surface symptom.\nDo not stop "
    "reasoning until you have independently verified the solution from multiple angles and are certain that no assumption "
    "remains unchecked and no error remains undiscovered.\n\n")


class _Dialect:
    """Tag spelling and joins that differ between the two encoders."""

    def __init__(self, v41: bool):
        d = "｜DSML｜"
        self.v41 = v41
        self.calls = f"{d} calls" if v41 else f"{d}tool_calls"
        self.invoke = f"{d} invoke" if v41 else f"{d}invoke"
        self.param = f"{d} parameter" if v41 else f"{d}parameter"
        self.part_join = "\n\n" if v41 else " "


def _flatten(content, join: str) -> str:
    if isinstance(content, list):
        return join.join(p["text"] for p in content
                         if isinstance(p, dict) and p.get("type") in ("text", "input_text") and isinstance(p.get("text"), str))
    return content


def _check_arguments(m: Dict[str, Any]) -> None:
    if m["role"] != "assistant":
        return
    for c in m.get("tool_calls") or []:
        a = c["function"].get("arguments")
        if isinstance(a, str):
            try:
                json.loads(a)
            except ValueError:
                raise ValueError("Assistant tool call function.arguments must be valid JSON.")
            if not a.lstrip().startswith("{"):
                raise ValueError("assistant tool arguments must be a JSON object")


def _tool_payload_v41(t: Any) -> Dict[str, Any]:
    f = t.get("function") if isinstance(t, dict) and isinstance(t.get("function"), dict) else {}
    if not isinstance(f.get("name"), str):
        raise ValueError("tool function requires name")
    fn = {k: f[k] for k in ("name", "description", "parameters") if f.get(k) is not None}
    if "strict" in f:
        fn["strict"] = pydantic_bool(f["strict"])
    defer = next((v for v in (f.get("defer_loading"), t.get("defer_loading")) if v is not None), None)
    if defer is not None:
        fn["defer_loading"] = pydantic_bool(defer)
    return {"type": "function", "function": fn}


def _normalize_messages(messages: List[Dict[str, Any]]) -> None:
    for m in messages:
        if m["role"] == "assistant":
            for c in m.get("tool_calls") or []:
                a = c["function"].get("arguments")
                if isinstance(a, str):
                    a = json.loads(a, parse_int=wide_int)
                if not isinstance(a, dict):
                    raise ValueError("assistant tool arguments must be a JSON object")
                c["function"]["arguments"] = a
        if isinstance(m.get("tools"), list):
            if m["tools"]:
                m["tools"] = normalize_tools(m["tools"])
            else:
                del m["tools"]
        if isinstance(m.get("tool_calls"), list) and not m["tool_calls"]:
            del m["tool_calls"]


def _budget_of(value) -> Optional[int]:
    """V4.1 reasoning budget (1-100) from a tier name, a whole number or a fraction."""
    if isinstance(value, str):
        return {"low": 50, "high": 75, "xhigh": 75, "max": 100}.get(value)
    if isinstance(value, bool):
        return None
    if isinstance(value, int):
        return value if 1 <= value <= 100 else None
    if isinstance(value, float):
        return max(1, int(round(value * 100))) if 0.0 <= value <= 0.99 else None      # round() rounds ties to even
    return None


def _v41_budget(request: Dict[str, Any], defaults: Dict[str, Any]) -> int:
    kw = (request.get("chat_template_kwargs") or {}).get("reasoning_effort")
    req = effort_of(request)
    if req is not None and not isinstance(req, bool):        # the request field is validated as a float where it parses as one
        if isinstance(req, (int, float)):
            req = float(req)
        elif isinstance(req, str):
            try:
                req = float(req.strip())
            except ValueError:
                pass
    chosen = kw if kw is not None else req if req is not None else defaults.get("reasoning_effort")
    b = _budget_of(chosen) if chosen is not None else None
    return b if b is not None else 75


def _v4_effort_text(profile: str, request: Dict[str, Any], defaults: Dict[str, Any]) -> str:
    kw = (request.get("chat_template_kwargs") or {}).get("reasoning_effort")
    chosen = kw if kw is not None else effort_of(request)
    if chosen is None:
        chosen = defaults.get("reasoning_effort")
    if not isinstance(chosen, str):
        return ""
    if (profile, chosen) in (("official", "high"), ("preview", "max")):
        return _EFFORT_HIGH
    if (profile, chosen) == ("official", "max"):
        return _EFFORT_MAX
    return ""


def _thinking(request: Dict[str, Any], defaults: Dict[str, Any]) -> bool:
    kw = request.get("chat_template_kwargs") or {}
    if "thinking" in kw:
        return truthy(kw["thinking"])
    t = thinking_requested(request)
    if t is not None:
        return t
    if "thinking" in defaults:
        return truthy(defaults["thinking"])
    return False


def _tools_block(tools: List[Dict[str, Any]], d: _Dialect) -> str:
    schemas = "\n".join(json.dumps(t["function"], ensure_ascii=False) for t in tools)
    return "\n\n" + _TOOLS_HEAD.format(calls=d.calls, invoke=d.invoke, param=d.param, schemas=schemas)


def _calls_block(calls: List[Dict[str, Any]], d: _Dialect) -> str:
    invokes = []
    for c in calls:
        fn = c["function"]
        params = [f'<{d.param} name="{k}" string="{"true" if isinstance(v, str) else "false"}">'
                  + (v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)) + f"</{d.param}>"
                  for k, v in fn["arguments"].items()]
        invokes.append(f'<{d.invoke} name="{fn["name"]}">\n' + "\n".join(params) + f"\n</{d.invoke}>")
    return f"\n\n<{d.calls}>\n" + "\n".join(invokes) + f"\n</{d.calls}>"


def _encode(messages: List[Dict[str, Any]], thinking: bool, d: _Dialect, lead: str) -> str:
    """The encoder proper.  ``lead`` is the reasoning-effort note: V4 writes it straight after BOS, V4.1 at the head of the
    first system turn."""
    keep_all = any(m.get("tools") for m in messages)       # with tools in the conversation earlier reasoning stays
    last_user = max((i for i, m in enumerate(messages) if m["role"] in ("user", "developer")), default=-1)
    out = [BOS]
    if not d.v41:
        out.append(lead)
    i, n = 0, len(messages)
    tail_task = None
    while i < n:
        m = messages[i]
        role = m["role"]
        content = _flatten(m["content"], d.part_join)
        tail_task = None
        if role == "system":
            body = content + (_tools_block(m["tools"], d) if m.get("tools") else "")
            out.append((SYSTEM + (lead if i == 0 else "") + body) if d.v41 else body)
            tail_task = m.get("task")
            if tail_task is not None and i + 1 < n:
                out.append(f"<｜{tail_task}｜>")
            i += 1
        elif role in ("user", "tool", "developer"):
            # one user block: this turn and the user / tool-result turns that follow it
            parts: List[str] = []
            results: List[Tuple[int, str]] = []
            order = {}
            if i > 0 and messages[i - 1]["role"] == "assistant":
                order = {c.get("id"): k for k, c in enumerate(messages[i - 1].get("tool_calls") or [])}

            def flush_results():
                results.sort(key=lambda r: r[0])
                parts.extend(r[1] for r in results)
                results.clear()

            j = i
            while j < n and (j == i or (messages[j]["role"] in ("user", "tool") and messages[j - 1]["role"] in ("user", "tool"))):
                mj = messages[j]
                text = _flatten(mj["content"], d.part_join)
                if mj["role"] == "tool":
                    results.append((order.get(mj.get("tool_call_id"), len(order) + j), f"<tool_result>{text}</tool_result>"))
                else:
                    flush_results()
                    parts.append(text + (_tools_block(mj["tools"], d) if mj.get("tools") else ""))
                    if mj.get("task") is not None:
                        tail_task = mj["task"]
                j += 1
            flush_results()
            out.append(USER + "\n\n".join(parts))
            if tail_task is not None and j < n:
                out.append(f"<｜{tail_task}｜>")
            i = j
        elif role == "assistant":
            if thinking and (keep_all or i > last_user):
                think = "<think>" + (m.get("reasoning_content") or "") + "</think>"
            else:
                think = "</think>"
            out.append(ASSISTANT + think + content + (_calls_block(m["tool_calls"], d) if m.get("tool_calls") else "") + EOS)
            i += 1
        else:
            raise ValueError(f"unknown message role {role!r}")
    last = messages[-1]["role"]
    if last in ("user", "developer", "tool", "system"):
        if tail_task is not None and tail_task != "action":
            out.append(f"<｜{tail_task}｜>")
        elif last != "system":
            out.append(ASSISTANT + ("<think>" if thinking else "</think>") + ("<｜action｜>" if tail_task == "action" else ""))
    return "".join(out)


def render_request(request: Dict[str, Any], defaults: Optional[Dict[str, Any]] = None, v41: bool = False,
                   profile: str = "official") -> Tuple[str, str]:
    """``(prompt, continuation prefix)`` of a chat request.  ``profile`` is the V4 checkpoint's reasoning-effort profile
    (``dsv4_reasoning_effort_profile`` of its config: "official" or "preview")."""
    defaults = defaults or {}
    d = _Dialect(v41)
    raw = request.get("messages")
    if not isinstance(raw, list):
        raise ValueError("messages must be an array")
    messages = [engine_message(m) for m in raw]
    for m in messages:
        if v41:
            if isinstance(m["content"], list):
                for p in m["content"]:
                    t = p.get("type") if isinstance(p, dict) else None
                    if t != "text":
                        raise ValueError(f"Model only supports text input; received unsupported content type {t!r}.")
            text = _flatten(m["content"], "")
            if isinstance(text, str) and IMAGE_TOKEN in text:
                raise ValueError(f"Message content contains image special token '{IMAGE_TOKEN}'. Images should be provided as "
                                 "image content blocks.")
        else:
            m["content"] = _flatten(m["content"], d.part_join)
        _check_arguments(m)
    prefix = split_continuation(messages, request)
    if not messages:
        raise IndexError("list index out of range")
    req_tools = request.get("tools") if isinstance(request.get("tools"), list) and request.get("tools") else None
    shown = req_tools if req_tools and renders_tools(request, req_tools) else None
    if v41 and shown and messages[0]["role"] != "system":
        messages.insert(0, {"role": "system", "content": ""})
    task = request.get("task")
    if task is not None:
        roles = ("user", "developer")
        target = next((m for k, m in reversed(list(enumerate(messages)))
                       if m["role"] in roles or (v41 and m["role"] == "system" and k > 0)), None)
        if target is None:
            raise ValueError("task requires a user or developer message")
        target["task"] = task
    for k in range(1, len(messages)):                       # a user turn folded into the block before it loses its task
        if messages[k]["role"] == "user" and messages[k - 1]["role"] in ("user", "tool"):
            messages[k].pop("task", None)
    _normalize_messages(messages)
    thinking = _thinking(request, defaults)
    if v41:
        payloads = [_tool_payload_v41(t) for t in req_tools] if req_tools else None
        if shown:
            messages[0]["tools"] = payloads
        lead = ""
        if thinking:
            lead = (f"Reasoning Effort: {_v41_budget(request, defaults)} (range 1-100, the higher the value, the more thorough "
                    "the reasoning)\n\n")
            if messages[0]["role"] != "system":
                messages.insert(0, {"role": "system", "content": ""})
    else:
        if messages[0]["role"] != "system":
            messages.insert(0, {"role": "system", "content": ""})
        if req_tools:
            normalized = normalize_tools(req_tools)
            if shown:
                messages[0]["tools"] = normalized
        lead = _v4_effort_text(profile, request, defaults) if thinking else ""
    return _encode(messages, thinking, d, lead), prefix
