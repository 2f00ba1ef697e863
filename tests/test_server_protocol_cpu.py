"""Protocol behaviour of the HTTP server with scripted answers: reasoning split, tool calls (free, forced, single), stop
strings, the Responses API (tools of every kind, stored conversations, event order) and the Messages API (tool loop,
thinking, stop sequences).  The checks follow the reference's API test client (``scripts/api_test.py``)."""
import json
import re

import pytest
import torch
from starlette.testclient import TestClient

from blaze_b200.config import named_config
from blaze_b200.llm import LLM
from blaze_b200.server.app import ServerState, create_app
from blaze_b200.service import ServiceArgs
from blaze_b200.text import ByteTokenizer

from scripted import TEMPLATE, ScriptedScheduler, call_text

WEATHER = {"type": "function", "function": {"name": "get_weather", "description": "Weather of a city", "parameters": {
    "type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"]}}}
TIME = {"type": "function", "function": {"name": "get_time", "description": "Local time of a city", "parameters": {
    "type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"]}}}


def script(prompt: str, thinking: bool):
    last = prompt.rsplit("<|im_start|>user\n", 1)[-1]
    names = re.findall(r'"name": "([a-z_]+)"', prompt.split("</tools>")[0]) if "<tools>" in prompt else []
    if "<tool_response>" in last:
        return "The result is " + " and ".join(re.findall(r"<tool_response>\n(.*?)\n</tool_response>", last, re.S)) + "."
    if "both cities" in last:
        return call_text("get_weather", '{"city": "Paris"}') + "\n" + call_text("get_weather", '{"city": "Oslo"}')
    if names and ("weather" in last.lower() or "time" in last.lower()):
        name = next((n for n in names if n.split("_")[-1] in last.lower()), names[0])
        return call_text(name, '{"city": "Oslo"}')
    if "hello.txt" in last:
        return call_text("apply_patch", json.dumps({"input": "*** Add File: hello.txt\n+hi"}))
    if "pong" in last:
        return "pong"
    if "Count" in last:
        return "1, 2, 3, 4, 5, 6"
    if "JSON" in last:
        return ['{"a":1}']
    # a greeting: words first; under a grammar the first candidate it accepts
    return ["Hello to you.", '{"greeting":"hello"}'] + [call_text(n, '{"city": "Rome"}') for n in reversed(names)]


@pytest.fixture(scope="module")
def served():
    st = ServerState(ServiceArgs(default_max_tokens=256, tool_call_parser="hermes", reasoning_parser="qwen3"), "scripted")
    app = create_app(st)
    llm = LLM(named_config("tiny"), device="cpu", dtype=torch.float32, max_seqs=8, max_model_len=2048, use_graphs=False)
    tok = ByteTokenizer(1024)
    tok.chat_template = TEMPLATE
    real = llm.sched
    llm.sched = ScriptedScheduler(real, tok, script)
    st.attach(llm, tok)
    yield TestClient(app), llm.sched
    real.stop()


def chat(c, content, **kw):
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": content}], **kw})
    assert r.status_code == 200, r.text
    return r.json()["choices"][0]


def test_reasoning_is_split_and_the_end_token_hidden(served):
    c, _ = served
    ch = chat(c, "Say pong.")
    # the blank line the model writes after its thinking belongs to the answer, as in the streamed form
    assert ch["message"]["content"] == "\n\npong" and ch["message"]["reasoning_content"].strip() == "Let me see." and ch["finish_reason"] == "stop"
    ch = chat(c, "Say pong.", chat_template_kwargs={"enable_thinking": False})
    assert ch["message"]["content"] == "pong" and not ch["message"].get("reasoning_content")
    ch = chat(c, "Say pong.", include_reasoning=False)
    assert ch["message"]["content"].strip() == "pong" and not ch["message"].get("reasoning_content")
    # separate_reasoning false: the thinking stays in the text
    ch = chat(c, "Say pong.", separate_reasoning=False)
    assert "Let me see." in ch["message"]["content"] and ch["message"]["content"].endswith("pong")
    # streamed: reasoning deltas, then content deltas, no end-of-sequence text
    with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "Say pong."}], "stream": True}) as s:
        deltas = [json.loads(l[6:])["choices"][0]["delta"] for l in s.iter_lines() if l.startswith("data: {")]
    assert "".join(d.get("reasoning_content") or "" for d in deltas).strip() == "Let me see."
    assert "".join(d.get("content") or "" for d in deltas) == "\n\npong"


def test_stop_strings_and_logprob_counts(served):
    c, _ = served
    ch = chat(c, "Count.", stop=["4"], chat_template_kwargs={"enable_thinking": False})
    assert ch["message"]["content"] == "1, 2, 3, " and ch["finish_reason"] == "stop"
    ch = chat(c, "Count.", stop=["4"], include_stop_str_in_output=True, chat_template_kwargs={"enable_thinking": False})
    assert ch["message"]["content"] == "1, 2, 3, 4"
    ch = chat(c, "Count.", max_tokens=4, chat_template_kwargs={"enable_thinking": False})
    assert ch["message"]["content"] == "1, 2" and ch["finish_reason"] == "length"
    ch = chat(c, "Say pong.", logprobs=True, top_logprobs=3, chat_template_kwargs={"enable_thinking": False})
    entries = ch["logprobs"]["content"]
    assert "".join(e["token"] for e in entries) == "pong" and all(len(e["top_logprobs"]) == 3 for e in entries)
    assert bytes(b for e in entries for b in e["bytes"]) == b"pong"


def test_tool_calls_free_forced_and_single(served):
    c, _ = served
    ch = chat(c, "What is the weather in Oslo?", tools=[WEATHER, TIME])
    assert ch["finish_reason"] == "tool_calls" and ch["message"]["tool_calls"][0]["function"]["name"] == "get_weather"
    assert json.loads(ch["message"]["tool_calls"][0]["function"]["arguments"]) == {"city": "Oslo"}
    ch = chat(c, "Weather in both cities?", tools=[WEATHER])
    assert [json.loads(t["function"]["arguments"])["city"] for t in ch["message"]["tool_calls"]] == ["Paris", "Oslo"]
    assert len({t["id"] for t in ch["message"]["tool_calls"]}) == 2
    ch = chat(c, "Weather in both cities?", tools=[WEATHER], parallel_tool_calls=False)
    assert len(ch["message"]["tool_calls"]) == 1
    # none: no call although the question wants one
    ch = chat(c, "What is the weather in Oslo?", tools=[WEATHER], tool_choice="none")
    assert not ch["message"].get("tool_calls")
    # required and named: the greeting would be answered in words; the grammar makes it a call
    ch = chat(c, "Hello there!", tools=[WEATHER, TIME], tool_choice="required", chat_template_kwargs={"enable_thinking": False})
    assert ch["finish_reason"] == "tool_calls" and ch["message"]["tool_calls"][0]["function"]["name"] in ("get_weather", "get_time")
    ch = chat(c, "Hello there!", tools=[WEATHER, TIME], tool_choice={"type": "function", "function": {"name": "get_weather"}},
              chat_template_kwargs={"enable_thinking": False})
    assert ch["finish_reason"] == "tool_calls" and ch["message"]["tool_calls"][0]["function"]["name"] == "get_weather"
    # the result fed back
    call = chat(c, "What is the weather in Oslo?", tools=[WEATHER])["message"]["tool_calls"][0]
    r = c.post("/v1/chat/completions", json={"tools": [WEATHER], "messages": [
        {"role": "user", "content": "What is the weather in Oslo?"}, {"role": "assistant", "content": None, "tool_calls": [call]},
        {"role": "tool", "tool_call_id": call["id"], "content": '{"temp_c": 4}'}]}).json()
    assert "temp_c" in r["choices"][0]["message"]["content"]
    # streamed: name and id first, then the arguments
    with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "Time in Oslo?"}], "tools": [TIME],
                                                        "stream": True}) as s:
        chunks = [json.loads(l[6:]) for l in s.iter_lines() if l.startswith("data: {")]
    tcs = [t for ch in chunks for t in (ch["choices"][0]["delta"].get("tool_calls") or [])]
    assert tcs[0]["function"]["name"] == "get_time" and tcs[0]["id"] and tcs[0]["index"] == 0
    assert json.loads("".join(t["function"].get("arguments") or "" for t in tcs)) == {"city": "Oslo"}
    assert chunks[-1]["choices"][0]["finish_reason"] == "tool_calls"


def test_structured_output_picks_what_the_grammar_accepts(served):
    c, _ = served
    ch = chat(c, "Hello there!", response_format={"type": "json_object"}, chat_template_kwargs={"enable_thinking": False})
    assert json.loads(ch["message"]["content"]) == {"greeting": "hello"}
    ch = chat(c, "Hello there!", structured_outputs={"json": {"type": "object"}, "disable_any_whitespace": True},
              chat_template_kwargs={"enable_thinking": False})
    assert ch["message"]["content"] == '{"greeting":"hello"}'


def items(r, kind):
    return [it for it in r["output"] if it["type"] == kind]


def test_responses_text_store_and_tools(served):
    c, sched = served
    r = c.post("/v1/responses", json={"input": "Say the word pong.", "max_output_tokens": 30, "reasoning": {"effort": "minimal"}}).json()
    assert r["object"] == "response" and r["status"] == "completed" and r["error"] is None
    assert items(r, "message")[0]["content"][0] == {"type": "output_text", "text": "pong", "annotations": []}
    assert r["usage"]["input_tokens"] > 0 and r["usage"]["output_tokens"] > 0 and r["output_text"] == "pong"
    assert not items(r, "reasoning")
    # thinking shows as a reasoning item
    r1 = c.post("/v1/responses", json={"input": "Say the word pong.", "instructions": "Be brief."}).json()
    assert items(r1, "reasoning")[0]["content"][0]["text"].strip() == "Let me see."
    # a stored conversation continues; new instructions replace the old system message
    r2 = c.post("/v1/responses", json={"input": "Count.", "previous_response_id": r1["id"], "instructions": "Be long."}).json()
    assert r2["previous_response_id"] == r1["id"]
    p = sched.prompts[-1]
    assert "Say the word pong." in p and "pong<|im_end|>" in p and "Be long." in p and "Be brief." not in p
    assert c.get("/v1/responses/" + r1["id"]).json()["id"] == r1["id"]
    assert c.post("/v1/responses", json={"input": "x", "previous_response_id": "resp_missing"}).status_code == 404
    assert c.post("/v1/responses", json={"input": []}).status_code == 400
    # incomplete when cut
    r = c.post("/v1/responses", json={"input": "Count.", "max_output_tokens": 4, "reasoning": {"effort": "minimal"}}).json()
    assert r["status"] == "incomplete" and r["incomplete_details"] == {"reason": "max_output_tokens"}
    # a function tool chosen in the flat form, its output fed back
    tool = {"type": "function", "name": "get_time", "description": "Local time of a city", "parameters": TIME["function"]["parameters"]}
    r = c.post("/v1/responses", json={"input": "Hello there!", "tools": [tool], "tool_choice": {"type": "function", "name": "get_time"},
                                      "reasoning": {"effort": "minimal"}}).json()
    call = items(r, "function_call")[0]
    assert call["name"] == "get_time" and "city" in json.loads(call["arguments"]) and call["status"] == "completed"
    r = c.post("/v1/responses", json={"tools": [tool], "input": [
        {"role": "user", "content": [{"type": "input_text", "text": "What time is it in Oslo?"}]},
        {"type": "reasoning", "id": "rs_1", "summary": []}, call,
        {"type": "function_call_output", "call_id": call["call_id"], "output": "13:37"}]}).json()
    assert "13:37" in items(r, "message")[0]["content"][0]["text"]
    assert '"name": "get_time"' in sched.prompts[-1].split("</tools>")[1]          # the call was replayed as an assistant turn
    # a custom tool answers as custom_tool_call with its input as text; a built-in tool is left out
    tools = [{"type": "custom", "name": "apply_patch", "description": "Apply a patch."}, {"type": "web_search"}]
    r = c.post("/v1/responses", json={"input": "Create hello.txt containing hi.", "tools": tools,
                                      "tool_choice": {"type": "custom", "name": "apply_patch"}}).json()
    call = items(r, "custom_tool_call")[0]
    assert call["name"] == "apply_patch" and call["input"] == "*** Add File: hello.txt\n+hi"
    assert "web_search" not in sched.prompts[-1]
    r = c.post("/v1/responses", json={"tools": tools, "input": [
        {"role": "user", "content": "Create hello.txt containing hi."}, call,
        {"type": "custom_tool_call_output", "call_id": call["call_id"], "output": "Done: hello.txt created."},
        {"type": "web_search_call", "id": "ws_1", "status": "completed"}]})
    assert r.status_code == 200 and "Done: hello.txt created." in items(r.json(), "message")[0]["content"][0]["text"]
    # only built-in tools: tool_choice has nothing to choose from and is dropped
    assert c.post("/v1/responses", json={"input": "Say pong.", "tools": [{"type": "web_search"}], "tool_choice": "required"}).status_code == 200


def sse(c, path, body):
    out, name = [], None
    with c.stream("POST", path, json=body) as s:
        for line in s.iter_lines():
            if line.startswith("event:"):
                name = line[6:].strip()
            elif line.startswith("data:"):
                out.append((name, json.loads(line[5:])))
    return out


def test_responses_stream_events(served):
    c, _ = served
    ev = sse(c, "/v1/responses", {"input": "Count.", "stream": True})
    names = [n for n, _ in ev]
    assert names[:2] == ["response.created", "response.in_progress"] and names[-1] == "response.completed"
    assert all(d["sequence_number"] == i and d["type"] == n for i, (n, d) in enumerate(ev))
    # reasoning item, then the message: each opened, filled and closed in order
    order = [n for n in names if n.endswith((".added", ".done"))]
    assert order == ["response.output_item.added", "response.reasoning_text.done", "response.output_item.done",
                     "response.output_item.added", "response.content_part.added", "response.output_text.done",
                     "response.content_part.done", "response.output_item.done"]
    assert "".join(d["delta"] for n, d in ev if n == "response.output_text.delta") == "1, 2, 3, 4, 5, 6"
    final = ev[-1][1]["response"]
    assert [it["type"] for it in final["output"]] == ["reasoning", "message"] and final["usage"]["output_tokens"] > 0
    assert final["output"][1]["status"] == "completed" and final["output"][1]["content"][0]["text"] == "1, 2, 3, 4, 5, 6"
    assert c.get("/v1/responses/" + final["id"]).json()["output"] == final["output"]
    # a call streams as an item with its arguments
    tool = {"type": "function", "name": "get_time", "parameters": TIME["function"]["parameters"]}
    ev = sse(c, "/v1/responses", {"input": "Time in Oslo?", "tools": [tool], "stream": True, "reasoning": {"effort": "minimal"}})
    done = [d for n, d in ev if n == "response.function_call_arguments.done"]
    assert json.loads(done[0]["arguments"]) == {"city": "Oslo"}
    assert [it["type"] for it in ev[-1][1]["response"]["output"]] == ["function_call"]
    ev = sse(c, "/v1/responses", {"input": "Count.", "stream": True, "max_output_tokens": 3, "reasoning": {"effort": "minimal"}})
    assert ev[-1][0] == "response.incomplete" and ev[-1][1]["response"]["status"] == "incomplete"


def test_messages_api(served):
    c, _ = served
    m = c.post("/v1/messages", json={"max_tokens": 40, "messages": [{"role": "user", "content": "Say pong."}]}).json()
    assert m["type"] == "message" and m["content"] == [{"type": "text", "text": "pong"}] and m["stop_reason"] == "end_turn"
    assert m["usage"]["input_tokens"] > 0
    tools = [{"name": "get_time", "description": "Local time of a city", "input_schema": TIME["function"]["parameters"]}]
    m = c.post("/v1/messages", json={"max_tokens": 300, "tools": tools, "tool_choice": {"type": "tool", "name": "get_time"},
                                     "messages": [{"role": "user", "content": "Hello there!"}]}).json()
    use = [b for b in m["content"] if b["type"] == "tool_use"]
    assert m["stop_reason"] == "tool_use" and use[0]["name"] == "get_time" and use[0]["input"] == {"city": "Rome"}
    m2 = c.post("/v1/messages", json={"max_tokens": 200, "tools": tools, "messages": [
        {"role": "user", "content": "Time in Rome?"}, {"role": "assistant", "content": m["content"]},
        {"role": "user", "content": [{"type": "tool_result", "tool_use_id": use[0]["id"], "content": "09:15"}]}]}).json()
    assert "09:15" in m2["content"][0]["text"]
    m = c.post("/v1/messages", json={"max_tokens": 400, "thinking": {"type": "enabled", "budget_tokens": 200},
                                     "messages": [{"role": "user", "content": "Say pong."}]}).json()
    assert [b["type"] for b in m["content"]] == ["thinking", "text"] and m["content"][0]["thinking"].strip() == "Let me see."
    ev = sse(c, "/v1/messages", {"max_tokens": 40, "stream": True, "messages": [{"role": "user", "content": "Count."}]})
    names = [n for n, _ in ev]
    assert names[0] == "message_start" and names[-1] == "message_stop" and "content_block_delta" in names and "message_delta" in names
    m = c.post("/v1/messages", json={"max_tokens": 80, "stop_sequences": ["5"], "messages": [{"role": "user", "content": "Count."}]}).json()
    assert m["stop_reason"] == "stop_sequence" and m["stop_sequence"] == "5" and m["content"][0]["text"] == "1, 2, 3, 4, "
    assert c.post("/v1/messages/count_tokens", json={"messages": [{"role": "user", "content": "Hello there"}]}).json()["input_tokens"] > 0
    e = c.post("/v1/messages", json={"messages": [{"role": "user", "content": "x"}]})
    assert e.status_code == 400 and e.json()["type"] == "error" and e.json()["error"]["type"] == "invalid_request_error"
