"""A scheduler stand-in that answers from a script, for protocol tests of the HTTP server: a random-init model cannot be asked
to call a tool, think, stop at a string or say "pong".  Generation requests are answered by ``script(prompt, thinking)``
(a string, or several candidates of which the first one the request's grammar accepts is used); everything else (embedding
requests, statistics, shutdown) goes to the real scheduler it wraps.  Tokens arrive a few at a time from a thread, the
way the real scheduler's sink is called, with ``max_tokens``, stop token ids, end-of-sequence, logprobs and aborts honoured."""
import threading
import time
from typing import Callable, List, Sequence, Union

from blaze_b200.sched import Finish, GenEvent

# ChatML with Hermes-style tool text and a thinking section that ``enable_thinking: false`` closes in the prompt.
TEMPLATE = """{%- if tools %}<|im_start|>system
{%- if messages[0].role == 'system' %}
{{ messages[0].content }}
{%- endif %}
# Tools
<tools>
{%- for t in tools %}
{{ t | tojson }}
{%- endfor %}
</tools><|im_end|>
{% elif messages[0].role == 'system' %}<|im_start|>system
{{ messages[0].content }}<|im_end|>
{% endif %}
{%- for m in messages %}
{%- if m.role == 'system' and loop.first %}
{%- elif m.role == 'tool' %}<|im_start|>user
<tool_response>
{{ m.content }}
</tool_response><|im_end|>
{% elif m.role == 'assistant' %}<|im_start|>assistant
{% if m.reasoning_content %}<think>
{{ m.reasoning_content }}
</think>

{% endif %}{{ m.content or '' }}
{%- for c in m.tool_calls or [] %}
<tool_call>
{"name": "{{ c.function.name }}", "arguments": {{ c.function.arguments if c.function.arguments is string else c.function.arguments | tojson }}}
</tool_call>
{%- endfor %}<|im_end|>
{% else %}<|im_start|>{{ m.role }}
{{ m.content }}<|im_end|>
{% endif %}
{%- endfor %}
{%- if add_generation_prompt %}<|im_start|>assistant
{% if enable_thinking is defined and enable_thinking is false %}<think>

</think>

{% else %}<think>
{% endif %}
{%- endif %}"""


def call_text(name: str, arguments: str) -> str:
    """A tool call as the Hermes parser reads it."""
    return '<tool_call>\n{"name": "%s", "arguments": %s}\n</tool_call>' % (name, arguments)


class ScriptedScheduler:
    def __init__(self, real, tokenizer, script: Callable[[str, bool], Union[str, Sequence[str]]], think: str = "Let me see.",
                 step_s: float = 0.001, tokens_per_event: int = 3):
        self._real, self._tok, self._script = real, tokenizer, script
        self._think, self._step_s, self._per = think, step_s, tokens_per_event
        self._aborted = set()
        self.prompts: List[str] = []

    def __getattr__(self, k):
        return getattr(self._real, k)

    def abort(self, rid):
        self._aborted.add(rid)
        self._real.abort(rid)

    def _accepted(self, constraint, ids: List[int]) -> bool:
        """Whether the grammar takes ``ids`` token by token (the constraint itself is not advanced)."""
        for i, t in enumerate(ids):
            if not bool(constraint.mask(ids[:i])[t]):
                return False
        return True

    def submit(self, req):
        if req.embed_only:
            return self._real.submit(req)
        prompt = self._tok.decode(req.prompt, skip_special_tokens=False)
        self.prompts.append(prompt)
        thinking = prompt.rstrip("\n").endswith("<think>")
        answers = self._script(prompt, thinking)
        answers = [answers] if isinstance(answers, str) else list(answers)
        eos = self._tok.eos_ids[-1]
        lead = self._tok.encode(self._think + "\n</think>\n\n") if thinking else []
        ids = None
        for a in answers:
            body = self._tok.encode(a) + [eos]
            if req.constraint is None or self._accepted(req.constraint, body):
                ids = lead + body
                break
        if ids is None:
            ids = lead + self._tok.encode(answers[0]) + [eos]
        p = req.params

        def run():
            n, fin = 0, None
            for i in range(0, len(ids), self._per):
                if req.request_id in self._aborted:
                    req.sink(GenEvent(req.request_id, finish=Finish.ABORT, prompt_tokens=len(req.prompt)))
                    return
                chunk = []
                for t in ids[i:i + self._per]:
                    if n >= p.max_tokens:
                        fin = Finish.LENGTH
                        break
                    chunk.append(t)
                    n += 1
                    if (t in self._tok.eos_ids and not p.ignore_eos) or t in p.stop_token_ids:
                        fin = Finish.STOP
                        break
                lps = None
                if p.logprobs is not None:
                    k = max(int(p.logprobs), 0)
                    lps = [{"token": t, "logprob": -0.1, "top": [(t, -0.1)] + [((t + j) % 256, -2.0 - j) for j in range(1, k)]}
                           for t in chunk]
                if chunk:
                    req.sink(GenEvent(req.request_id, tokens=chunk, logprobs=lps, prompt_tokens=len(req.prompt),
                                      stopped_on=chunk[-1] if fin == Finish.STOP else None))
                if fin:
                    break
                time.sleep(self._step_s)
            req.sink(GenEvent(req.request_id, finish=fin or Finish.STOP, prompt_tokens=len(req.prompt)))
        threading.Thread(target=run, daemon=True).start()
