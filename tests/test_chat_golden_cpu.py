"""Prompt rendering against golden prompts: 850 chat requests over eight checkpoints of five families (DeepSeek-V4 and
V4.1, GLM-5.3, Kimi-K3, Qwen3.8), each with the exact prompt text the reference serving stack produces for it, or the fact
that it must be refused.  ``tests/data/chat_prompt_golden.json.gz`` holds, per checkpoint, its name, the ``config.json``
fields that select the encoder, its Jinja template where it has one, and the cases (request body, server-side default
template arguments, expected prompt).  The expected text is that of the reference's parity fixtures
(``crates/blaze-chat/tests/fixtures/parity``, checked there by ``crates/blaze-chat/tests/parity.rs``)."""
import gzip
import json
import os

import pytest

from blaze_b200.chat import ChatFormatter

with gzip.open(os.path.join(os.path.dirname(__file__), "data", "chat_prompt_golden.json.gz"), "rt", encoding="utf-8") as f:
    GOLDEN = json.load(f)["models"]


@pytest.mark.parametrize("entry", GOLDEN, ids=[m["model"] for m in GOLDEN])
def test_prompts_match_the_golden_text(entry):
    fmt = ChatFormatter.for_checkpoint(entry["model"], entry["config"], entry.get("chat_template"))
    assert fmt.encoder is not None, "every golden checkpoint has a family encoder"
    bad = []
    for case in entry["cases"]:
        try:
            prompt, prefix, _ = fmt.render_request(case["request"], case.get("defaults"))
            got = prompt + prefix
        except (ValueError, TypeError, IndexError, KeyError) as e:
            got = e
        if case.get("error"):
            if not isinstance(got, Exception):
                bad.append((case["name"], "should have been refused", got))
        elif got != case["prompt"]:
            bad.append((case["name"], case["prompt"], got))
    assert not bad, f"{len(bad)} of {len(entry['cases'])} prompts differ; first: {bad[0]}"


def test_thinking_flag_follows_the_prompt_tail():
    ds = ChatFormatter.for_checkpoint("deepseek-ai/DeepSeek-V4-Flash", {"model_type": "deepseek_v4"})
    req = {"messages": [{"role": "user", "content": "Hi"}]}
    assert ds.render_request(req)[2] is False
    assert ds.render_request({**req, "reasoning_effort": "high"})[2] is True
    # a server-side default a request may override
    assert ds.render_request(req, {"thinking": True})[2] is True
    assert ds.render_request({**req, "chat_template_kwargs": {"thinking": False}}, {"thinking": True})[2] is False
    kimi = ChatFormatter.for_checkpoint("moonshotai/Kimi-K3", {"model_type": "kimi_k3"})
    assert kimi.render_request(req)[2] is True
    p, prefix, thinking = kimi.render_request({"messages": req["messages"] + [{"role": "assistant", "content": "It is"}],
                                               "continue_final_message": True})
    assert prefix == "It is" and thinking is False and p.endswith("<|open|>think<|sep|>")


def test_plain_template_checkpoints_keep_the_generic_path():
    fmt = ChatFormatter.for_checkpoint("Qwen/Qwen3-8B", {"model_type": "qwen3", "architectures": ["Qwen3ForCausalLM"]})
    assert fmt.encoder is None
    prompt, prefix, thinking = fmt.render_request({"messages": [{"role": "user", "content": "Hi"}],
                                                   "chat_template_kwargs": {"enable_thinking": False}})
    assert prompt == "<|im_start|>user\nHi<|im_end|>\n<|im_start|>assistant\n<think>\n\n</think>\n\n" and prefix == "" and thinking is False


with gzip.open(os.path.join(os.path.dirname(__file__), "data", "reasoning_split_golden.json.gz"), "rt", encoding="utf-8") as f:
    REASONING = json.load(f)["parsers"]

# Streams in which the recorded step-by-step split disagrees with the recorded split of the whole output (a later <think>
# after the reasoning ended, a quoted <tool_call> inside a line): the splitter here keeps stream and whole output alike,
# as the reference's own splitter does (``think/models/qwen3.rs`` tests), so only the whole-output split is compared.
SELF_INCONSISTENT = {("deepseek-v4", 11), ("deepseek-v41", 11), ("qwen3", 4)}


@pytest.mark.parametrize("entry", REASONING, ids=[p["parser"] for p in REASONING])
def test_reasoning_split_matches_the_golden_steps(entry):
    """304 recorded outputs over five reasoning parsers (``crates/blaze-chat/tests/fixtures/reasoning_parity``): the split of
    the whole output, and the (reasoning, answer) delta of every streamed chunk plus the final flush, with reasoning forced
    on or off, streamed or held until it ends, and the never-empty-answer option."""
    from blaze_b200.chat import get_think_parser
    bad = []
    for case in entry["cases"]:
        chunks = entry["inputs"][case["input"]]
        kw = dict(starts_in_think=bool(case.get("force")), nonempty=bool(case.get("nonempty")))
        whole = list(get_think_parser(entry["parser"], **kw).parse("".join(chunks)))
        p = get_think_parser(entry["parser"], stream_reasoning=bool(case.get("stream")), **kw)
        steps = [list(p.push(c)) for c in chunks] + [list(p.flush())]
        if whole != case["unary"]:
            bad.append((case, "whole", whole))
        elif (entry["parser"], case["input"]) in SELF_INCONSISTENT:
            joined = ["".join(s[0] for s in steps), "".join(s[1] for s in steps)]
            if steps != case["steps"] and joined != whole and not case.get("nonempty"):
                bad.append((case, "stream differs from both the recorded steps and the whole-output split", steps))
        elif steps != case["steps"]:
            bad.append((case, "steps", steps))
    assert not bad, f"{len(bad)} of {len(entry['cases'])} differ; first: {bad[0]}"


with gzip.open(os.path.join(os.path.dirname(__file__), "data", "tool_call_golden.json.gz"), "rt", encoding="utf-8") as f:
    TOOL_CALLS = json.load(f)["parsers"]


@pytest.mark.parametrize("entry", TOOL_CALLS, ids=[p["parser"] for p in TOOL_CALLS])
def test_tool_calls_match_the_golden_parses(entry):
    """134 recorded outputs over the DSML (two tag sets), Kimi-K3 and qwen3_coder tool-call parsers
    (``crates/blaze-chat/tests/fixtures/tool_parity``): answer text and (name, arguments JSON) of every call for the whole
    output, and, for the DSML and Kimi parsers, the same accumulated over the recorded stream chunks.  The qwen3_coder
    stream is compared with the whole-output parse instead (its recorded stream emits argument JSON piecewise, keeps
    duplicate keys and escapes differently; the reference does not pin it either, ``tool_call/models/mod.rs``)."""
    from blaze_b200.chat import get_tool_parser
    bad = []
    for n, case in enumerate(entry["cases"]):
        text = "".join(case["chunks"])
        p = get_tool_parser(entry["parser"], entry["tools"])
        if hasattr(p, "parse"):
            t, calls = p.parse(text)
        else:
            t, calls = p.push(text)
            ft, fc = p.flush()
            t, calls = t + ft, calls + fc
        whole = [t, [[c.name, c.arguments] for c in calls]]
        if whole != case["whole"]:
            bad.append((n, "whole", whole, case["whole"]))
            continue
        p = get_tool_parser(entry["parser"], entry["tools"])
        t, calls = "", []
        for chunk in case["chunks"]:
            a, b = p.push(chunk)
            t, calls = t + a, calls + b
        a, b = p.flush()
        stream = [t + a, [[c.name, c.arguments] for c in calls + b]]
        if entry["parser"] == "qwen3_coder":
            if stream[1] != whole[1] and "<tool_call>" in text:
                bad.append((n, "stream calls differ from the whole-output parse", stream, whole))
        elif stream != case["stream"]:
            # one recorded case feeds the V4.1 parser the other tag set and records an empty stream for it
            if not (entry["parser"] == "deepseekv41" and "｜DSML｜tool_calls" in text):
                bad.append((n, "stream", stream, case["stream"]))
    assert not bad, f"{len(bad)} of {len(entry['cases'])} differ; first: {bad[0]}"
