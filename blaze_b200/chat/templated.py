"""GLM-5.3 and Qwen3.8 prompts: the checkpoint's Jinja template, fed the request the way the serving layer prepares it.

Both templates take tool-call arguments as objects, joined text parts, the dumped tool list (filtered by ``tool_choice``),
and the request's thinking toggle and reasoning effort as template variables.  Request preparation follows
``crates/blaze-chat/src/render/models/glm53.rs`` and ``qwen38.rs``; the expected prompts are those of
``crates/blaze-chat/tests/fixtures/parity/glm-5.3*.json`` and ``qwen3.8-*.json``."""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional, Tuple

from .request import (effort_of, engine_message, normalize_tools, pydantic_bool, split_continuation, thinking_requested,
                      wide_int)

_RESERVED = ("add_generation_prompt", "chat_template", "continue_final_message", "conversation", "messages",
             "return_assistant_tokens_mask", "return_dict", "tokenize", "tools")
_MEDIA = ("image_url", "video_url", "audio_url", "input_audio")


def is_glm53(template: str) -> bool:
    return (all(t in template for t in ("[gMASK]<sop>", "Reasoning Effort:", "<tool_call>", "<arg_key>", "<arg_value>"))
            and "enable_thinking" not in template)


def is_qwen38(template: str) -> bool:
    return all(t in template for t in ("<|im_start|>", "<function=", "<parameter=", "preserve_thinking",
                                       "Reasoning effort is set to"))


def takes_content_parts(template: str) -> bool:
    return any(k in template for k in ("image", "audio", "video", "vision"))


def _valid_documents(d: Any) -> bool:
    if d is None:
        return True
    if isinstance(d, list):
        return all(isinstance(x, dict) for x in d)
    if isinstance(d, (str, dict)):
        return not d
    return False


def _template_args(request: Dict[str, Any], defaults: Dict[str, Any]) -> Dict[str, Any]:
    kw = request.get("chat_template_kwargs")
    if kw is not None and not isinstance(kw, dict):
        raise ValueError("chat_template_kwargs must be an object")
    kwargs = dict(kw or {})
    t = thinking_requested(request)
    if t is not None:
        kwargs.setdefault("thinking", t)
        kwargs.setdefault("enable_thinking", t)
    effort = kwargs.pop("reasoning_effort", None)
    if effort is None:
        effort = effort_of(request)
    for k, v in defaults.items():
        kwargs.setdefault(k, v)
    for k in _RESERVED:
        if k in kwargs:
            raise TypeError(f"chat_template_kwargs.{k} collides with an argument of the template call")
    if not _valid_documents(kwargs.get("documents")):
        raise TypeError("chat_template_kwargs.documents must iterate as objects")
    if effort is None:
        effort = kwargs.get("reasoning_effort")
    args = {"reasoning_effort": effort} if effort is not None else {}
    args.update(kwargs)
    return args


def _template_tools(request: Dict[str, Any], qwen: bool) -> Optional[List[Dict[str, Any]]]:
    tools = request.get("tools")
    choice = request.get("tool_choice")
    if not isinstance(tools, list) or not tools or choice == "none":
        return None
    dumped = normalize_tools(tools)
    if qwen:
        for d, t in zip(dumped, tools):
            defer = t.get("defer_loading") if isinstance(t, dict) else None
            d["defer_loading"] = None if defer is None else pydantic_bool(defer)
            if isinstance(t, dict) and isinstance(t.get("type"), str):
                d["type"] = t["type"]
    if isinstance(choice, dict):
        name = (choice.get("function") or {}).get("name")
        dumped = [d for d in dumped if d["function"]["name"] == name]
    return dumped or None


def _arguments_as_objects(m: Dict[str, Any], qwen: bool) -> None:
    for c in m.get("tool_calls") or []:
        f = c["function"]
        a = f.get("arguments")
        if isinstance(a, str):
            try:
                a = json.loads(a, parse_int=wide_int)
            except ValueError:
                a = None
            if not isinstance(a, dict):
                raise ValueError("assistant tool arguments must be a JSON object")
        if qwen:
            c["function"] = {"name": f.get("name"), "arguments": a}
        elif "arguments" in f and f["arguments"] is not None:
            f["arguments"] = a


def _message(m: Any, qwen: bool, content_parts: bool) -> Dict[str, Any]:
    m = engine_message(m)
    m.pop("tools", None)
    if m["role"] == "assistant":
        _arguments_as_objects(m, qwen)
    parts = m["content"]
    if not isinstance(parts, list):
        return m
    kept: List[Dict[str, Any]] = []
    for p in parts:
        t = p.get("type") if isinstance(p, dict) else None
        if qwen:
            if t in _MEDIA:
                raise ValueError(f"Model only supports text input; received unsupported content type {t!r}.")
            if t == "text":
                kept.append({"type": "text", "text": p.get("text")})
            elif t == "tool_reference" and content_parts:
                kept.append({"type": "tool_reference", "name": p.get("name")})
        else:
            if t in ("thinking", "reasoning"):
                continue
            if t == "text":
                kept.append({"type": "text", "text": p.get("text")})
            elif t == "tool_reference":
                kept.append({"type": "tool_reference", "name": p.get("name")})
            else:
                raise ValueError(f"Model only supports text input; received unsupported content type {t!r}.")
    all_text = all(p["type"] == "text" for p in kept)
    if (qwen and not content_parts) or (m["role"] == "tool" and all_text):
        m["content"] = " ".join(p["text"] for p in kept if isinstance(p.get("text"), str))
    else:
        m["content"] = kept
    return m


def _join_text_parts(m: Dict[str, Any]) -> None:
    c = m["content"]
    if isinstance(c, list) and c and all(p["type"] == "text" for p in c):
        m["content"] = "".join(p["text"] for p in c if isinstance(p.get("text"), str))


def render_request(formatter, request: Dict[str, Any], defaults: Optional[Dict[str, Any]] = None,
                   family: str = "glm53") -> Tuple[str, str]:
    """``(prompt, continuation prefix)``.  ``formatter`` is the ``ChatFormatter`` holding the checkpoint's template;
    ``family`` is "glm53" or "qwen38"."""
    defaults = dict(defaults or {})
    qwen = family == "qwen38"
    if isinstance(defaults.get("chat_template"), str) and "chat_template" not in (request.get("chat_template_kwargs") or {}):
        # a server-side default template replaces the checkpoint's
        formatter = type(formatter)(defaults.pop("chat_template"), formatter.bos_token, formatter.eos_token, formatter.family)
    args = _template_args(request, defaults)
    tools = _template_tools(request, qwen)
    raw = request.get("messages")
    if not isinstance(raw, list):
        raise ValueError("messages must be an array")
    content_parts = qwen and takes_content_parts(formatter.template_src or "")
    messages = [_message(m, qwen, content_parts) for m in raw]
    prefix = split_continuation(messages, request)
    if qwen:
        if any(m["role"] == "system" for m in messages[1:]):
            raise ValueError("System message must be at the beginning.")
    elif not messages:
        raise IndexError("list index out of range")
    for m in messages:
        _join_text_parts(m)
    # without a generation prompt the template ends after the last turn (not combined with a continued turn, whose prefix
    # already stands for the opened assistant turn)
    gen = request.get("add_generation_prompt") is not False or bool(prefix)
    return formatter.render_prepared(messages, tools, args, add_generation_prompt=gen), prefix
