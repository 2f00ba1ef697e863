"""Prompt rendering: the checkpoint's Jinja chat template when it has one, else a built-in ChatML renderer
(Qwen style, with tools and thinking control).  Reference: ``crates/blaze-chat/src/render`` (``ChatFormatter``)."""
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


class ChatFormatter:
    def __init__(self, chat_template: Optional[str] = None, bos_token: str = "", eos_token: str = "<|im_end|>"):
        self.template_src = chat_template
        self.bos_token, self.eos_token = bos_token, eos_token
        self._tpl = None
        if chat_template:
            from jinja2.sandbox import ImmutableSandboxedEnvironment

            def raise_exception(msg):
                raise ValueError(msg)

            def tojson(v, ensure_ascii=False, indent=None):
                return json.dumps(v, ensure_ascii=ensure_ascii, indent=indent)

            env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
            env.globals["raise_exception"] = raise_exception
            env.filters["tojson"] = tojson
            self._tpl = env.from_string(chat_template)

    def render(self, messages: List[Dict[str, Any]], tools: Optional[List[Dict[str, Any]]] = None,
               add_generation_prompt: bool = True, enable_thinking: Optional[bool] = None, **kwargs) -> str:
        if self._tpl is not None:
            ctx = dict(messages=messages, tools=tools, add_generation_prompt=add_generation_prompt,
                       bos_token=self.bos_token, eos_token=self.eos_token, **kwargs)
            if enable_thinking is not None:
                ctx["enable_thinking"] = enable_thinking
            return self._tpl.render(**ctx)
        return self._chatml(messages, tools, add_generation_prompt, enable_thinking)

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
