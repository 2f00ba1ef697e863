"""Prompt rendering: the checkpoint's Jinja chat template when it has one, else a built-in renderer of the model
family (ChatML for Qwen, with tools and thinking control; DeepSeek, GLM and Kimi turn markers).  Before either, the
messages are normalised the way the family's template expects them (``normalize_messages``).
Reference: ``crates/blaze-chat/src/render`` (``ChatFormatter``; ``render/models`` — qwen38.rs, deepseek_v4.rs, glm53.rs,
kimi_k3.rs prepare the request for the family's template)."""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional

DEFAULT_SYSTEM_TOOLS = ("# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
                        "You are provided with function signatures within <tools></tools> XML tags:\n<tools>\n{tools}\n</tools>\n\n"
                        "For each function call, return a json object with function name and arguments within "
                        "<tool_call></tool_call> XML tags:\n<tool_call>\n{{\"name\": <function-name>, \"arguments\": <args-json-object>}}\n</tool_call>")


def _text_of(content) -> str:
    """OpenAI message content: a string or a list of parts ({type:text|image_url|...})."""
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    out = []
    for part in content:
        if isinstance(part, str):
            out.append(part)
        elif part.get("type") in ("text", "input_text", "output_text"):
            out.append(part.get("text", ""))
        elif part.get("type") in ("image_url", "image", "input_image"):
            out.append("<|vision_start|><|image_pad|><|vision_end|>")
    return "".join(out)


FAMILIES = ("chatml", "deepseek", "glm", "kimi")


def family_of(model_name: str) -> str:
    """Renderer family from a model or architecture name."""
    n = (model_name or "").lower()
    for key, fam in (("deepseek", "deepseek"), ("glm", "glm"), ("kimi", "kimi"), ("moonshot", "kimi")):
        if key in n:
            return fam
    return "chatml"


def normalize_messages(messages: List[Dict[str, Any]], family: str = "chatml", flatten: bool = False) -> List[Dict[str, Any]]:
    """What the family templates rely on: ``developer`` is ``system``; assistant tool-call arguments are objects
    (a JSON string is parsed, anything else is an error); ``content`` defaults to ""; with ``flatten`` the content
    parts collapse to their text.  DeepSeek and Kimi always get a leading system message (theirs carries the tools),
    and DeepSeek merges a user turn that follows a user or tool turn into one."""
    out: List[Dict[str, Any]] = []
    for m in messages:
        m = dict(m)
        if m.get("role") == "developer":
            m["role"] = "system"
        if m.get("content") is None:
            m["content"] = ""
        if flatten or family in ("deepseek", "kimi", "glm"):
            m["content"] = _text_of(m["content"]) if not isinstance(m["content"], str) else m["content"]
        if m.get("tool_calls"):
            calls = []
            for i, tc in enumerate(m["tool_calls"]):
                fn = dict(tc.get("function", tc))
                args = fn.get("arguments", {})
                if isinstance(args, str):
                    try:
                        args = json.loads(args) if args.strip() else {}
                    except ValueError:
                        raise ValueError("assistant tool arguments must be a JSON object")
                if not isinstance(args, dict):
                    raise ValueError("assistant tool arguments must be a JSON object")
                calls.append({"id": tc.get("id"), "index": tc.get("index", i), "type": "function",
                              "function": {"name": fn.get("name"), "arguments": args}})
            m["tool_calls"] = calls
        elif "tool_calls" in m:
            del m["tool_calls"]
        if family == "deepseek" and out and m["role"] == "user" and out[-1]["role"] == "user":
            out[-1] = dict(out[-1], content=out[-1]["content"] + "\n\n" + m["content"])
            continue
        out.append(m)
    if family in ("deepseek", "kimi") and (not out or out[0]["role"] != "system"):
        out.insert(0, {"role": "system", "content": ""})
    return out


THINK_OPENERS = ("<think>", "<think>\n", "<|open|>think<|sep|>")


class ChatFormatter:
    """Prompt renderer of one checkpoint.  ``encoder`` names a family request encoder: "deepseek_v4", "deepseek_v41" and
    "kimi_k3" build the prompt without a template; "glm53" and "qwen38" (recognised from the template text) prepare the
    request for the checkpoint's template.  Without one, ``render`` runs the template (or the built-in family layout) on
    the messages as given."""

    def __init__(self, chat_template: Optional[str] = None, bos_token: str = "", eos_token: str = "<|im_end|>",
                 family: str = "chatml", encoder: Optional[str] = None, effort_profile: str = "preview"):
        if family not in FAMILIES:
            raise ValueError(f"unknown chat family {family!r}")
        self.family = family
        self.encoder, self.effort_profile = encoder, effort_profile
        if encoder is None and chat_template:
            from . import templated
            self.encoder = ("glm53" if templated.is_glm53(chat_template) else
                            "qwen38" if templated.is_qwen38(chat_template) else None)
        self.template_src = chat_template
        self.bos_token, self.eos_token = bos_token, eos_token
        self._tpl = None
        if chat_template:
            from jinja2.sandbox import ImmutableSandboxedEnvironment

            def raise_exception(msg):
                raise ValueError(msg)

            def tojson(v, ensure_ascii=False, indent=None, separators=None, sort_keys=False):
                return json.dumps(v, ensure_ascii=ensure_ascii, indent=indent, separators=separators, sort_keys=sort_keys)

            def strftime_now(fmt):
                import datetime
                return datetime.datetime.now().strftime(fmt)

            env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=["jinja2.ext.loopcontrols"])
            env.globals["raise_exception"] = raise_exception
            env.globals["strftime_now"] = strftime_now
            env.filters["tojson"] = tojson
            self._tpl = env.from_string(chat_template)

    def render_prepared(self, messages: List[Dict[str, Any]], tools: Optional[List[Dict[str, Any]]], args: Dict[str, Any],
                        add_generation_prompt: bool = True) -> str:
        """Run the template on messages a family encoder has already prepared (no normalisation here)."""
        if self._tpl is None:
            raise ValueError("the checkpoint has no chat template")
        ctx = dict(bos_token=self.bos_token, eos_token=self.eos_token)
        ctx.update(args)
        ctx.update(messages=messages, tools=tools, add_generation_prompt=add_generation_prompt)
        from jinja2.exceptions import TemplateError
        try:
            return self._tpl.render(**ctx)
        except TemplateError as e:
            raise ValueError(f"chat template error: {e}")

    @classmethod
    def for_checkpoint(cls, model_name: str, config: Optional[Dict[str, Any]], chat_template: Optional[str] = None,
                       family: Optional[str] = None, bos_token: str = "", eos_token: str = "<|im_end|>") -> "ChatFormatter":
        """The formatter a checkpoint gets from its name, ``config.json`` fields and template
        (``crates/blaze-chat/src/render/selection.rs``)."""
        from .families import encoder_of
        config = config or {}
        return cls(chat_template, bos_token, eos_token, family or family_of(model_name), encoder_of(model_name, config),
                   str(config.get("dsv4_reasoning_effort_profile") or "preview"))

    def render_request(self, request: Dict[str, Any], defaults: Optional[Dict[str, Any]] = None):
        """``(prompt, continuation prefix, thinking)`` of a chat-completions request body.  ``prefix`` is the text of a final
        assistant turn to continue (tokenised on its own after the prompt); ``thinking`` says whether the prompt leaves the
        model inside its reasoning channel.  ``defaults`` are server-side template arguments a request may override."""
        if self.encoder in ("deepseek_v4", "deepseek_v41"):
            from . import deepseek
            prompt, prefix = deepseek.render_request(request, defaults, self.encoder == "deepseek_v41", self.effort_profile)
        elif self.encoder == "kimi_k3":
            from . import kimi
            prompt, prefix = kimi.render_request(request, defaults)
        elif self.encoder in ("glm53", "qwen38"):
            from . import templated
            prompt, prefix = templated.render_request(self, request, defaults, self.encoder)
        else:
            tools = request.get("tools")
            if request.get("tool_choice", "auto" if tools else "none") == "none":
                tools = None
            from .request import effort_of, thinking_requested
            kw = dict(defaults or {})
            kw.update(request.get("chat_template_kwargs") or {})
            # reasoning_effort / reasoning.{effort,enabled} switch thinking and name the effort the template may announce;
            # explicit template arguments win (``crates/blaze/src/server/chat.rs:176-188``)
            t, e = thinking_requested(request), effort_of(request)
            if t is not None:
                kw.setdefault("thinking", t)
                kw.setdefault("enable_thinking", t)
            if e is not None:
                kw.setdefault("reasoning_effort", e)
            think = kw.pop("enable_thinking", request.get("enable_thinking"))
            for k in ("messages", "tools", "add_generation_prompt"):
                kw.pop(k, None)
            messages = request.get("messages") or []
            if request.get("continue_final_message") not in (None, False, 0):
                # the final assistant turn is rendered closed and the prompt is cut after its text, which leaves it open
                tail = _text_of(messages[-1].get("content")) if messages else ""
                if not tail:
                    raise ValueError("the last message has no text to continue")
                prompt = self.render(messages, tools, False, think, **kw)
                at = prompt.rfind(tail)
                if at < 0:
                    raise ValueError("the last message's text is not in the rendered prompt")
                return prompt[:at + len(tail)], "", False
            prompt = self.render(messages, tools, bool(request.get("add_generation_prompt", True)), think, **kw)
            return prompt, "", think
        return prompt, prefix, prompt.endswith(THINK_OPENERS) and not prefix

    def render(self, messages: List[Dict[str, Any]], tools: Optional[List[Dict[str, Any]]] = None,
               add_generation_prompt: bool = True, enable_thinking: Optional[bool] = None, **kwargs) -> str:
        if self.family != "chatml":
            messages = normalize_messages(messages, self.family)
        if self._tpl is not None:
            ctx = dict(messages=messages, tools=tools, add_generation_prompt=add_generation_prompt,
                       bos_token=self.bos_token, eos_token=self.eos_token, **kwargs)
            if enable_thinking is not None:
                ctx["enable_thinking"] = enable_thinking
            from jinja2.exceptions import TemplateError
            try:
                return self._tpl.render(**ctx)
            except TemplateError as e:
                raise ValueError(f"chat template error: {e}")
        builtin = {"chatml": self._chatml, "deepseek": self._deepseek, "glm": self._glm, "kimi": self._kimi}[self.family]
        return builtin(messages, tools, add_generation_prompt, enable_thinking)

    # ---- built-in family renderers (used when the checkpoint ships no template) ----
    @staticmethod
    def _tool_lines(tools) -> str:
        return "\n".join(json.dumps(t.get("function", t), ensure_ascii=False) for t in tools or [])

    def _deepseek(self, messages, tools, add_generation_prompt, enable_thinking) -> str:
        D = "｜DSML｜"
        out = [self.bos_token or "<｜begin▁of▁sentence｜>"]
        system = messages[0]["content"]
        if tools:
            system += (("\n\n" if system else "") + "## Tools\nYou can call these functions:\n<functions>\n"
                       + self._tool_lines(tools) + f"\n</functions>\nCall them inside one <{D}tool_calls> block of "
                       f'<{D}invoke name="..."> elements with <{D}parameter name="..." string="true|false"> children.')
        out.append(system)
        for m in messages[1:]:
            role = m["role"]
            if role == "assistant":
                body = ""
                if m.get("reasoning_content"):
                    body += "<think>" + m["reasoning_content"] + "</think>"
                body += m["content"]
                if m.get("tool_calls"):
                    body += f"\n\n<{D}tool_calls>\n"
                    for tc in m["tool_calls"]:
                        fn = tc["function"]
                        body += f'<{D}invoke name="{fn["name"]}">\n'
                        for k, v in fn["arguments"].items():
                            is_str = isinstance(v, str)
                            body += (f'<{D}parameter name="{k}" string="{"true" if is_str else "false"}">'
                                     + (v if is_str else json.dumps(v, ensure_ascii=False)) + f"</{D}parameter>\n")
                        body += f"</{D}invoke>\n"
                    body += f"</{D}tool_calls>"
                out.append("<｜Assistant｜>" + body + "<｜end▁of▁sentence｜>")
            elif role == "tool":
                out.append("<｜User｜><function_results>\n<result>" + m["content"] + "</result>\n</function_results>")
            elif role == "system":
                out.append("\n\n" + m["content"])
            else:
                out.append("<｜User｜>" + m["content"])
        if add_generation_prompt:
            out.append("<｜Assistant｜>" + ("</think>" if enable_thinking is False else "<think>"))
        return "".join(out)

    def _glm(self, messages, tools, add_generation_prompt, enable_thinking) -> str:
        out = ["[gMASK]<sop>"]
        if tools:
            out.append("<|system|>\n# Tools\n\nYou may call one or more functions to assist with the user query.\n<tools>\n"
                       + self._tool_lines(tools) + "\n</tools>\n\nFor each function call, output the function name and "
                       "arguments within <tool_call>{function-name}\n<arg_key>{key}</arg_key>\n<arg_value>{value}</arg_value>\n"
                       "...\n</tool_call>")
        for m in messages:
            role = m["role"]
            if role == "assistant":
                body = "\n<think>" + (m.get("reasoning_content") or "") + "</think>\n" + m["content"]
                for tc in m.get("tool_calls") or []:
                    fn = tc["function"]
                    body += "\n<tool_call>" + fn["name"]
                    for k, v in fn["arguments"].items():
                        body += (f"\n<arg_key>{k}</arg_key>\n<arg_value>"
                                 + (v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)) + "</arg_value>")
                    body += "\n</tool_call>"
                out.append("<|assistant|>" + body)
            elif role == "tool":
                out.append("<|observation|>\n<tool_response>\n" + m["content"] + "\n</tool_response>")
            else:
                out.append(f"<|{role}|>\n" + m["content"] + ("/nothink" if role == "user" and enable_thinking is False else ""))
        if add_generation_prompt:
            out.append("<|assistant|>" + ("\n<think></think>\n" if enable_thinking is False else ""))
        return "".join(out)

    def _kimi(self, messages, tools, add_generation_prompt, enable_thinking) -> str:
        O, C, S = "<|open|>", "<|close|>", "<|sep|>"

        def esc(v: str) -> str:
            return v.replace("&", "&amp;").replace('"', "&quot;")

        out: List[str] = []
        for i, m in enumerate(messages):
            role = m["role"]
            out.append(f'{O}message role="{role}"{S}')
            if i == 0 and tools:
                out.append(f"{O}tools{S}" + self._tool_lines(tools) + f"{C}tools{S}")
            if role == "assistant":
                if m.get("reasoning_content"):
                    out.append(f"{O}think{S}" + m["reasoning_content"] + f"{C}think{S}")
                if m["content"]:
                    out.append(f"{O}response{S}" + m["content"] + f"{C}response{S}")
                if m.get("tool_calls"):
                    out.append(f"{O}tools{S}")
                    for tc in m["tool_calls"]:
                        fn = tc["function"]
                        out.append(f'{O}call tool="{esc(fn["name"])}"' + (f' id="{esc(tc["id"])}"' if tc.get("id") else "") + S)
                        for k, v in fn["arguments"].items():
                            typ = ("string" if isinstance(v, str) else "boolean" if isinstance(v, bool) else
                                   "number" if isinstance(v, (int, float)) else "null" if v is None else
                                   "array" if isinstance(v, list) else "object")
                            out.append(f'{O}argument key="{esc(k)}" type="{typ}"{S}'
                                       + (v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)) + f"{C}argument{S}")
                        out.append(f"{C}call{S}")
                    out.append(f"{C}tools{S}")
            elif role == "tool":
                out.append((f'{O}result id="{esc(m["tool_call_id"])}"{S}' if m.get("tool_call_id") else f"{O}result{S}")
                           + m["content"] + f"{C}result{S}")
            else:
                out.append(m["content"])
            out.append(f"{C}message{S}")
        if add_generation_prompt:
            out.append(f'{O}message role="assistant"{S}' + (f"{O}response{S}" if enable_thinking is False else f"{O}think{S}"))
        return "".join(out)

    def _chatml(self, messages, tools, add_generation_prompt, enable_thinking) -> str:
        out: List[str] = []
        msgs = list(messages)
        system = ""
        if msgs and msgs[0].get("role") in ("system", "developer"):
            system = _text_of(msgs.pop(0).get("content"))
        if tools:
            tl = "\n".join(json.dumps(t, ensure_ascii=False) for t in tools)
            system = (system + "\n\n" if system else "") + DEFAULT_SYSTEM_TOOLS.format(tools=tl)
        if system:
            out.append(f"<|im_start|>system\n{system}<|im_end|>\n")
        for m in msgs:
            role = m.get("role", "user")
            text = _text_of(m.get("content"))
            if role == "assistant":
                body = ""
                rc = m.get("reasoning_content")
                if rc:
                    body += f"<think>\n{rc}\n</think>\n\n"
                body += text
                for tc in m.get("tool_calls") or []:
                    fn = tc.get("function", tc)
                    args = fn.get("arguments")
                    if isinstance(args, str):
                        try:
                            args = json.loads(args)
                        except ValueError:
                            pass
                    body += ("\n" if body else "") + "<tool_call>\n" + json.dumps({"name": fn.get("name"), "arguments": args},
                                                                                  ensure_ascii=False) + "\n</tool_call>"
                out.append(f"<|im_start|>assistant\n{body}<|im_end|>\n")
            elif role == "tool":
                out.append(f"<|im_start|>user\n<tool_response>\n{text}\n</tool_response><|im_end|>\n")
            else:
                out.append(f"<|im_start|>{role}\n{text}<|im_end|>\n")
        if add_generation_prompt:
            out.append("<|im_start|>assistant\n")
            if enable_thinking is False:
                out.append("<think>\n\n</think>\n\n")
        return "".join(out)
