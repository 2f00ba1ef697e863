"""The OpenAI Responses API as a view of a chat request: input items to chat messages, tools (function, custom, built-in)
to chat tools, the answer to output items, and the event sequence of a streamed response.  Nothing here touches the model;
the route in ``server/app.py`` runs the chat request these functions produce.

Behaviour follows the reference's adapter (``crates/blaze/src/server/responses.rs``): consecutive calls are one assistant
turn :101, a custom (freeform) tool runs as a function of one string ``input`` and answers as a ``custom_tool_call`` :173-184
:278, built-in tools (web search, file search, computer, shell, MCP) and their items are left out :119 :185, ``tool_choice``
in the flat ``{"type": "function" | "custom", "name"}`` form and ``allowed_tools`` :193-207, ``instructions`` replace a kept
system message :143, events carry ``sequence_number`` from 0 and open/close one item per kind of output :405."""
from __future__ import annotations

import json
import time
import uuid
from typing import Any, Dict, Iterable, List, Optional, Set, Tuple

from ..service import RequestError

TEXT_PARTS = ("input_text", "output_text", "text", "summary_text")
# sampling fields a Responses request may carry under the chat names
PASS_THROUGH = ("model", "temperature", "top_p", "parallel_tool_calls", "top_logprobs", "seed", "samplers", "top_nsigma", "top_h",
                "top_k", "min_p", "presence_penalty", "frequency_penalty", "repetition_penalty", "logit_bias", "stop",
                "chat_template_kwargs", "enable_thinking", "thinking_token_budget", "priority", "user")


def new_id(prefix: str) -> str:
    return f"{prefix}_{uuid.uuid4().hex[:24]}"


def content_of(c: Any) -> Any:
    """Chat content of an item's content: a string stays, parts become chat parts."""
    if not isinstance(c, list):
        return c if isinstance(c, str) else None
    out: List[Dict[str, Any]] = []
    for p in c:
        kind = p.get("type", "") if isinstance(p, dict) else ""
        if kind in TEXT_PARTS:
            out.append({"type": "text", "text": p.get("text") or ""})
        elif kind == "input_image":
            url = p.get("image_url")
            url = url.get("url") if isinstance(url, dict) else url
            if not isinstance(url, str):
                raise RequestError("an input_image needs an image_url (file ids are not supported)", "input")
            img: Dict[str, Any] = {"type": "image_url", "image_url": {"url": url}}
            if p.get("detail") is not None:
                img["image_url"]["detail"] = p["detail"]
            out.append(img)
        elif kind == "refusal":
            out.append({"type": "text", "text": p.get("refusal") or ""})
        else:
            raise RequestError(f"content part {kind!r} is not supported", "input")
    return out


def input_messages(inp: Any) -> List[Dict[str, Any]]:
    """The input (a string or a list of items) as chat messages.  Reasoning items, references and the calls of built-in
    tools are left out."""
    if isinstance(inp, str):
        return [{"role": "user", "content": inp}]
    if inp is None:
        return []
    if not isinstance(inp, list):
        raise RequestError("input must be a string or a list of items", "input")
    out: List[Dict[str, Any]] = []
    for it in inp:
        if not isinstance(it, dict):
            raise RequestError("an input item must be an object", "input")
        kind = it.get("type") or ("message" if "role" in it else "")
        if kind == "message":
            role = it.get("role") or "user"
            out.append({"role": "system" if role == "developer" else role, "content": content_of(it.get("content"))})
        elif kind in ("function_call", "custom_tool_call"):
            args = json.dumps({"input": it.get("input") or ""}) if kind == "custom_tool_call" else (it.get("arguments") or "{}")
            call = {"id": it.get("call_id") or it.get("id") or new_id("call"), "type": "function",
                    "function": {"name": it.get("name") or "", "arguments": args}}
            if out and out[-1]["role"] == "assistant" and isinstance(out[-1].get("tool_calls"), list):
                out[-1]["tool_calls"].append(call)
            else:
                out.append({"role": "assistant", "content": None, "tool_calls": [call]})
        elif kind in ("function_call_output", "custom_tool_call_output"):
            o = it.get("output")
            if isinstance(o, list):
                o = content_of(o)
            elif o is None:
                o = ""
            elif not isinstance(o, str):
                o = json.dumps(o)
            out.append({"role": "tool", "tool_call_id": it.get("call_id") or "", "content": o})
        elif not kind:
            raise RequestError("an input item needs a type or a role", "input")
    return out


def chat_tools(tools: Any) -> Tuple[List[Dict[str, Any]], Set[str]]:
    """Chat tools of the request's tools and the names of its custom ones."""
    out: List[Dict[str, Any]] = []
    custom: Set[str] = set()
    for t in tools or []:
        kind = t.get("type") if isinstance(t, dict) else None
        if kind == "function":
            out.append({"type": "function", "function": {
                "name": t.get("name") or "", "description": t.get("description"),
                "parameters": t.get("parameters") or {"type": "object", "properties": {}}}})
        elif kind == "custom":
            name, about = t.get("name") or "", t.get("description") or ""
            fmt = t.get("format") if isinstance(t.get("format"), dict) else {}
            if isinstance(fmt.get("definition"), str):
                about += f"\n\nThe input follows this grammar ({fmt.get('syntax') or 'lark'}):\n{fmt['definition']}"
            out.append({"type": "function", "function": {"name": name, "description": about, "parameters": {
                "type": "object", "properties": {"input": {"type": "string", "description": "the tool's input, as text"}},
                "required": ["input"]}}})
            custom.add(name)
    return out, custom


def chat_request(body: Dict[str, Any], kept: Optional[List[Dict[str, Any]]] = None
                 ) -> Tuple[Dict[str, Any], List[Dict[str, Any]], Set[str]]:
    """``(chat body, the conversation before the answer, custom tool names)`` of a Responses request; ``kept`` is the
    conversation of ``previous_response_id``."""
    messages = [dict(m) for m in (kept or [])]
    if isinstance(body.get("instructions"), str):
        messages = [m for m in messages if m.get("role") != "system"]
        messages.insert(0, {"role": "system", "content": body["instructions"]})
    messages.extend(input_messages(body.get("input")))
    if not messages:
        raise RequestError("input is empty", "input")
    chat: Dict[str, Any] = {"messages": [dict(m) for m in messages]}
    for k in PASS_THROUGH:
        if body.get(k) is not None:
            chat[k] = body[k]
    if body.get("max_output_tokens") is not None:
        chat["max_tokens"] = body["max_output_tokens"]
    tools, custom = chat_tools(body.get("tools"))
    if tools:
        chat["tools"] = tools
        choice = body.get("tool_choice")
        if isinstance(choice, str):
            chat["tool_choice"] = choice
        elif isinstance(choice, dict):
            if choice.get("type") in ("function", "custom"):
                name = choice.get("name") or (choice.get("function") or {}).get("name") or ""
                chat["tool_choice"] = {"type": "function", "function": {"name": name}}
            elif choice.get("type") == "allowed_tools":
                chat["tool_choice"] = choice.get("mode") or "auto"
    effort = body["reasoning"].get("effort") if isinstance(body.get("reasoning"), dict) else None
    if isinstance(effort, str):
        # "minimal": as little as possible, i.e. no thinking section for a model that has one
        chat["reasoning_effort"] = "none" if effort == "minimal" else effort
    fmt = body["text"].get("format") if isinstance(body.get("text"), dict) else None
    if isinstance(fmt, dict):
        kind = fmt.get("type")
        if kind == "json_object":
            chat["response_format"] = {"type": "json_object"}
        elif kind == "json_schema":
            chat["response_format"] = {"type": "json_schema", "json_schema": {
                "name": fmt.get("name") or "schema", "schema": fmt.get("schema") or {}, "strict": bool(fmt.get("strict", False))}}
        elif kind not in (None, "text"):
            raise RequestError(f"format type {kind!r} is not supported", "text.format")
    if body.get("stream") is True:
        chat["stream"] = True
    return chat, messages, custom


def shell(body: Dict[str, Any], rid: str, model: str, status: str, created: Optional[int] = None) -> Dict[str, Any]:
    """The response object's fixed fields: a copy of the request's settings."""
    return {"id": rid, "object": "response", "created_at": int(time.time()) if created is None else created, "status": status,
            "model": model, "output": [], "error": None, "incomplete_details": None,
            "instructions": body.get("instructions"), "max_output_tokens": body.get("max_output_tokens"),
            "parallel_tool_calls": body.get("parallel_tool_calls", True), "previous_response_id": body.get("previous_response_id"),
            "reasoning": body.get("reasoning") or {"effort": None, "summary": None},
            "temperature": body.get("temperature", 1.0), "text": body.get("text") or {"format": {"type": "text"}},
            "tool_choice": body.get("tool_choice", "auto"), "tools": body.get("tools") or [], "top_p": body.get("top_p", 1.0),
            "store": body.get("store", True), "metadata": body.get("metadata") or {}, "usage": None}


def usage(prompt: int, output: int, cached: int = 0, reasoning: int = 0) -> Dict[str, Any]:
    return {"input_tokens": prompt, "output_tokens": output, "total_tokens": prompt + output,
            "input_tokens_details": {"cached_tokens": cached}, "output_tokens_details": {"reasoning_tokens": reasoning}}


def custom_input(arguments: str) -> str:
    """The input of a custom tool's call: the ``input`` string of its arguments, else the arguments as written."""
    try:
        v = json.loads(arguments)
    except ValueError:
        return arguments
    return v["input"] if isinstance(v, dict) and isinstance(v.get("input"), str) else arguments


def call_item(call_id: str, name: str, arguments: str, custom: Iterable[str], status: str = "completed") -> Dict[str, Any]:
    if name in custom:
        return {"type": "custom_tool_call", "id": new_id("ctc"), "call_id": call_id, "name": name,
                "input": custom_input(arguments), "status": status}
    return {"type": "function_call", "id": new_id("fc"), "call_id": call_id, "name": name, "arguments": arguments, "status": status}


def settle(reasoning: str, text: str, n_calls: int, natural_stop: bool) -> Tuple[str, str]:
    """An answer the model ended inside its thinking section (a natural stop, no text, no call): the reasoning is the
    answer (``responses.rs:268``)."""
    if natural_stop and not text.strip() and not n_calls and reasoning.strip():
        return "", reasoning
    return reasoning, text


def output_items(reasoning: str, text: str, calls, custom: Iterable[str]) -> List[Dict[str, Any]]:
    """Output items of an answer: reasoning, the message, the calls (objects with ``id``, ``name``, ``arguments``)."""
    out: List[Dict[str, Any]] = []
    if reasoning:
        out.append({"type": "reasoning", "id": new_id("rs"), "summary": [], "content": [{"type": "reasoning_text", "text": reasoning}]})
    if text.strip():
        out.append({"type": "message", "id": new_id("msg"), "status": "completed", "role": "assistant",
                    "content": [{"type": "output_text", "text": text, "annotations": []}]})
    for c in calls:
        out.append(call_item(c.id, c.name, c.arguments, custom))
    return out


def kept_messages(messages: List[Dict[str, Any]], reasoning: str, text: str, calls) -> List[Dict[str, Any]]:
    """The conversation after the answer, for a later ``previous_response_id``."""
    m: Dict[str, Any] = {"role": "assistant", "content": text or None}
    if calls:
        m["tool_calls"] = [{"id": c.id, "type": "function", "function": {"name": c.name, "arguments": c.arguments}} for c in calls]
    if reasoning:
        m["reasoning_content"] = reasoning
    return messages + [m]


class EventStream:
    """Events of a streamed response.  One item per kind of output is open at a time: it opens with its first delta and
    closes when another kind starts or the answer ends.  Every method returns the ``(event name, payload)`` pairs to send."""

    def __init__(self, body: Dict[str, Any], rid: str, model: str, custom: Iterable[str]):
        self.resp = shell(body, rid, model, "in_progress")
        self.custom = set(custom)
        self.seq = 0
        self.output: List[Dict[str, Any]] = []
        self.open: Optional[Tuple[str, int]] = None      # (kind, output index)
        self.buf = ""
        self.reasoning = ""
        self.text = ""

    def _ev(self, kind: str, **payload) -> Tuple[str, Dict[str, Any]]:
        out = (kind, {"type": kind, "sequence_number": self.seq, **payload})
        self.seq += 1
        return out

    def start(self):
        return [self._ev("response.created", response=dict(self.resp)), self._ev("response.in_progress", response=dict(self.resp))]

    def _close(self):
        if self.open is None:
            return []
        kind, oi = self.open
        item, text = self.output[oi], self.buf
        self.open, self.buf = None, ""
        out = []
        if kind == "reasoning":
            item["content"] = [{"type": "reasoning_text", "text": text}]
            out.append(self._ev("response.reasoning_text.done", item_id=item["id"], output_index=oi, content_index=0, text=text))
        elif kind == "message":
            part = {"type": "output_text", "text": text, "annotations": []}
            item["content"], item["status"] = [part], "completed"
            out.append(self._ev("response.output_text.done", item_id=item["id"], output_index=oi, content_index=0, text=text))
            out.append(self._ev("response.content_part.done", item_id=item["id"], output_index=oi, content_index=0, part=part))
        out.append(self._ev("response.output_item.done", output_index=oi, item=dict(item)))
        return out

    def _open(self, kind: str, item: Dict[str, Any]):
        out = self._close()
        self.output.append(item)
        oi = len(self.output) - 1
        self.open = (kind, oi)
        out.append(self._ev("response.output_item.added", output_index=oi, item=dict(item)))
        return out, oi

    def on_reasoning(self, delta: str):
        if not delta:
            return []
        out = []
        if self.open is None or self.open[0] != "reasoning":
            out, _ = self._open("reasoning", {"type": "reasoning", "id": new_id("rs"), "summary": [], "content": []})
        oi = self.open[1]
        self.buf += delta
        self.reasoning += delta
        out.append(self._ev("response.reasoning_text.delta", item_id=self.output[oi]["id"], output_index=oi, content_index=0, delta=delta))
        return out

    def on_text(self, delta: str):
        if not delta:
            return []
        out = []
        if self.open is None or self.open[0] != "message":
            if not delta.strip():          # the blank line after the reasoning opens no message
                self.text += delta
                return []
            out, oi = self._open("message", {"type": "message", "id": new_id("msg"), "status": "in_progress", "role": "assistant", "content": []})
            out.append(self._ev("response.content_part.added", item_id=self.output[oi]["id"], output_index=oi, content_index=0,
                                part={"type": "output_text", "text": "", "annotations": []}))
        oi = self.open[1]
        self.buf += delta
        self.text += delta
        out.append(self._ev("response.output_text.delta", item_id=self.output[oi]["id"], output_index=oi, content_index=0, delta=delta))
        return out

    def on_call(self, call):
        """A finished call (the tool parsers hand calls over whole): its item opens, gets its arguments and closes."""
        item = call_item(call.id, call.name, call.arguments, self.custom)
        opened = {**item, "status": "in_progress", **({"input": ""} if item["type"] == "custom_tool_call" else {"arguments": ""})}
        out = self._close()
        self.output.append(item)
        oi = len(self.output) - 1
        out.append(self._ev("response.output_item.added", output_index=oi, item=opened))
        if item["type"] == "custom_tool_call":
            out.append(self._ev("response.custom_tool_call_input.delta", item_id=item["id"], output_index=oi, delta=item["input"]))
            out.append(self._ev("response.custom_tool_call_input.done", item_id=item["id"], output_index=oi, input=item["input"]))
        else:
            if item["arguments"]:
                out.append(self._ev("response.function_call_arguments.delta", item_id=item["id"], output_index=oi, delta=item["arguments"]))
            out.append(self._ev("response.function_call_arguments.done", item_id=item["id"], output_index=oi, arguments=item["arguments"]))
        out.append(self._ev("response.output_item.done", output_index=oi, item=dict(item)))
        return out

    def failed(self, message: str):
        self.resp["status"] = "failed"
        self.resp["error"] = {"code": "server_error", "message": message}
        return [self._ev("response.failed", response=dict(self.resp))]

    def finish(self, length: bool, natural_stop: bool, n_calls: int, use: Dict[str, Any]):
        out = self._close()
        if natural_stop and not self.text.strip() and not n_calls and self.reasoning.strip():
            # an answer left inside the thinking section: a message of the reasoning
            self.text = ""
            out += self.on_text(self.reasoning)
            out += self._close()
        self.resp["status"] = "incomplete" if length else "completed"
        if length:
            self.resp["incomplete_details"] = {"reason": "max_output_tokens"}
        self.resp["output"] = self.output
        self.resp["usage"] = use
        out.append(self._ev("response.incomplete" if length else "response.completed", response=dict(self.resp)))
        return out
