"""The Anthropic Messages API as a view of a chat request: content blocks to chat messages, tools and ``tool_choice`` to
their chat forms, the answer to content blocks, and the event sequence of a streamed message.  Nothing here touches the
model; the route in ``server/app.py`` runs the chat request these functions produce.

Behaviour follows the reference's adapter (``crates/blaze/src/server/messages.rs``): user blocks keep their order around
tool results :131-155, an ``is_error`` result is prefixed :142, thinking blocks of earlier assistant turns are replayed as
reasoning :112, server tools (a ``type`` other than ``custom``) are left out :175, ``tool_choice`` auto / any / none / tool
and ``disable_parallel_tool_use`` :184-196, thinking only when asked for with ``budget_tokens`` as the budget :198, a block
per kind of output in the stream with a ``signature_delta`` closing a thinking block :279."""
from __future__ import annotations

import json
import uuid
from typing import Any, Dict, List, Optional, Tuple

from ..service import RequestError

SAMPLING = ("model", "max_tokens", "temperature", "top_p", "top_k", "samplers", "top_nsigma", "top_h", "min_p", "presence_penalty",
            "frequency_penalty", "repetition_penalty", "logit_bias", "seed")


def new_id(prefix: str) -> str:
    return f"{prefix}_{uuid.uuid4().hex[:24]}"


ERROR_KINDS = {400: "invalid_request_error", 413: "invalid_request_error", 422: "invalid_request_error", 401: "authentication_error",
               403: "permission_error", 404: "not_found_error", 429: "rate_limit_error", 529: "overloaded_error"}


def error_body(status: int, message: str) -> Dict[str, Any]:
    return {"type": "error", "error": {"type": ERROR_KINDS.get(status, "api_error"), "message": message}}


def result_text(c: Any) -> str:
    """Text of a tool_result's content: a string or text blocks (images are not carried into a tool message)."""
    if isinstance(c, str):
        return c
    if isinstance(c, list):
        return "\n".join(b["text"] for b in c if isinstance(b, dict) and isinstance(b.get("text"), str))
    return "" if c is None else json.dumps(c)


def image_part(b: Dict[str, Any]) -> Dict[str, Any]:
    src = b.get("source") or {}
    kind = src.get("type")
    if kind == "base64":
        url = f"data:{src.get('media_type') or 'image/png'};base64,{src.get('data') or ''}"
    elif kind == "url":
        url = src.get("url") or ""
    else:
        raise RequestError(f"image source {kind!r} is not supported (base64, url)", "messages")
    return {"type": "image_url", "image_url": {"url": url}}


def chat_request(body: Dict[str, Any]) -> Dict[str, Any]:
    """The chat request of a Messages request."""
    messages: List[Dict[str, Any]] = []
    system = body.get("system")
    if isinstance(system, list):
        system = "\n".join(b["text"] for b in system if isinstance(b, dict) and isinstance(b.get("text"), str))
    if isinstance(system, str) and system:
        messages.append({"role": "system", "content": system})
    if not isinstance(body.get("messages"), list):
        raise RequestError("messages is required", "messages")
    for m in body["messages"]:
        role, content = m.get("role") or "user", m.get("content")
        blocks = [{"type": "text", "text": content}] if isinstance(content, str) else (content if isinstance(content, list) else [])
        if role == "assistant":
            text, thinking, calls = "", "", []
            for b in blocks:
                kind = b.get("type") or ""
                if kind == "text":
                    text += b.get("text") or ""
                elif kind == "thinking":
                    thinking += b.get("thinking") or ""
                elif kind == "redacted_thinking":
                    pass
                elif kind == "tool_use":
                    calls.append({"id": b.get("id"), "type": "function",
                                  "function": {"name": b.get("name"), "arguments": json.dumps(b.get("input") or {})}})
                else:
                    raise RequestError(f"assistant block {kind!r} is not supported", "messages")
            msg: Dict[str, Any] = {"role": "assistant", "content": None if (not text and calls) else text}
            if thinking:
                msg["reasoning_content"] = thinking
            if calls:
                msg["tool_calls"] = calls
            messages.append(msg)
            continue
        parts: List[Dict[str, Any]] = []

        def flush():
            if parts:
                only_text = all(p["type"] == "text" for p in parts)
                messages.append({"role": "user", "content": "".join(p["text"] for p in parts) if only_text and len(parts) == 1 else list(parts)})
                parts.clear()
        for b in blocks:
            kind = b.get("type") or ""
            if kind == "text":
                parts.append({"type": "text", "text": b.get("text") or ""})
            elif kind == "image":
                parts.append(image_part(b))
            elif kind == "tool_result":
                flush()
                text = result_text(b.get("content"))
                if b.get("is_error") is True:
                    text = "Error: " + text
                messages.append({"role": "tool", "tool_call_id": b.get("tool_use_id"), "content": text})
            elif kind in ("document", "search_result"):
                raise RequestError("document blocks are not supported", "messages")
            else:
                raise RequestError(f"user block {kind!r} is not supported", "messages")
        flush()
    chat: Dict[str, Any] = {"messages": messages}
    for k in SAMPLING:
        if body.get(k) is not None:
            chat[k] = body[k]
    if isinstance(body.get("stop_sequences"), list):
        chat["stop"] = body["stop_sequences"]
    tools = [{"type": "function", "function": {"name": t.get("name"), "description": t.get("description"),
                                               "parameters": t.get("input_schema") or {"type": "object"}}}
             for t in (body.get("tools") or []) if t.get("type") in (None, "custom")]
    if tools:
        chat["tools"] = tools
    tc = body.get("tool_choice")
    if tc is not None:
        kind = tc.get("type") if isinstance(tc, dict) else None
        if kind == "auto":
            choice: Any = "auto"
        elif kind == "any":
            choice = "required"
        elif kind == "none":
            choice = "none"
        elif kind == "tool":
            choice = {"type": "function", "function": {"name": tc.get("name")}}
        else:
            raise RequestError(f"tool_choice type {kind!r}", "tool_choice")
        if tools:
            chat["tool_choice"] = choice
        if tc.get("disable_parallel_tool_use") is True:
            chat["parallel_tool_calls"] = False
    # thinking only when asked for (this API's default); budget_tokens is the thinking budget
    th = body.get("thinking") if isinstance(body.get("thinking"), dict) else {}
    on = th.get("type") == "enabled"
    chat["enable_thinking"] = on
    chat["chat_template_kwargs"] = {"enable_thinking": on, "thinking": on}       # the families' templates read one of the two
    if on and isinstance(th.get("budget_tokens"), int):
        chat["thinking_token_budget"] = th["budget_tokens"]
    if body.get("stream") is True:
        chat["stream"] = True
    return chat


def stop_reason(length: bool, has_calls: bool, stop: Optional[str]) -> Tuple[str, Optional[str]]:
    """``(stop_reason, stop_sequence)``; ``stop``: the stop string that ended the answer."""
    if length:
        return "max_tokens", None
    if has_calls:
        return "tool_use", None
    if stop is not None:
        return "stop_sequence", stop
    return "end_turn", None


def usage(prompt: int, output: int, cached: int = 0) -> Dict[str, int]:
    return {"input_tokens": prompt, "output_tokens": output, "cache_read_input_tokens": cached, "cache_creation_input_tokens": 0}


def input_of(arguments: str) -> Dict[str, Any]:
    """A tool call's arguments as the tool_use block's input object."""
    try:
        v = json.loads(arguments)
    except ValueError:
        return {}
    return v if isinstance(v, dict) else {}


def tool_use_id(call_id: str) -> str:
    return "toolu_" + call_id[5:] if call_id.startswith("call_") else call_id


def blocks(reasoning: str, text: str, calls) -> List[Dict[str, Any]]:
    out: List[Dict[str, Any]] = []
    if reasoning:
        out.append({"type": "thinking", "thinking": reasoning, "signature": ""})
    if text.strip():
        out.append({"type": "text", "text": text})
    for c in calls:
        out.append({"type": "tool_use", "id": tool_use_id(c.id), "name": c.name, "input": input_of(c.arguments)})
    return out


class BlockStream:
    """Events of a streamed message: a content block per kind of output (thinking, text, each tool call), opened with its
    first delta and stopped when the next one starts.  Every method returns the event payloads to send."""

    def __init__(self, mid: str, model: str, prompt_tokens: int):
        self.mid, self.model, self.prompt_tokens = mid, model, prompt_tokens
        self.open: Optional[Tuple[str, int]] = None
        self.next = 0
        self.reasoning = ""
        self.answered = False
        self.calls = 0

    def start(self):
        return [{"type": "message_start", "message": {"id": self.mid, "type": "message", "role": "assistant", "model": self.model,
                                                      "content": [], "stop_reason": None, "stop_sequence": None,
                                                      "usage": {"input_tokens": self.prompt_tokens, "output_tokens": 0}}},
                {"type": "ping"}]

    def _close(self):
        if self.open is None:
            return []
        kind, i = self.open
        self.open = None
        out = []
        if kind == "thinking":
            out.append({"type": "content_block_delta", "index": i, "delta": {"type": "signature_delta", "signature": ""}})
        out.append({"type": "content_block_stop", "index": i})
        return out

    def _open(self, kind: str, block: Dict[str, Any]):
        out = self._close()
        self.open = (kind, self.next)
        out.append({"type": "content_block_start", "index": self.next, "content_block": block})
        self.next += 1
        return out

    def on_reasoning(self, delta: str):
        if not delta:
            return []
        out = [] if self.open and self.open[0] == "thinking" else self._open("thinking", {"type": "thinking", "thinking": "", "signature": ""})
        self.reasoning += delta
        out.append({"type": "content_block_delta", "index": self.open[1], "delta": {"type": "thinking_delta", "thinking": delta}})
        return out

    def on_text(self, delta: str):
        if not delta:
            return []
        out = []
        if not (self.open and self.open[0] == "text"):
            if not delta.strip():          # the blank line after the thinking opens no block
                return []
            out = self._open("text", {"type": "text", "text": ""})
        self.answered = True
        out.append({"type": "content_block_delta", "index": self.open[1], "delta": {"type": "text_delta", "text": delta}})
        return out

    def on_call(self, call):
        out = self._open("tool_use", {"type": "tool_use", "id": tool_use_id(call.id), "name": call.name, "input": {}})
        self.calls += 1
        if call.arguments:
            out.append({"type": "content_block_delta", "index": self.open[1], "delta": {"type": "input_json_delta", "partial_json": call.arguments}})
        return out

    def error(self, message: str):
        return [{"type": "error", "error": {"type": "api_error", "message": message}}]

    def finish(self, length: bool, stop: Optional[str], output_tokens: int, cached: int = 0):
        out = self._close()
        if not length and not self.answered and not self.calls and self.reasoning.strip():
            # an answer left inside the thinking section: its text
            out += self._open("text", {"type": "text", "text": ""})
            out.append({"type": "content_block_delta", "index": self.open[1], "delta": {"type": "text_delta", "text": self.reasoning}})
            out += self._close()
        reason, sequence = stop_reason(length, self.calls > 0, stop)
        out.append({"type": "message_delta", "delta": {"stop_reason": reason, "stop_sequence": sequence},
                    "usage": {"output_tokens": output_tokens, "input_tokens": self.prompt_tokens, "cache_read_input_tokens": cached}})
        out.append({"type": "message_stop"})
        return out
