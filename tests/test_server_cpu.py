"""HTTP API on CPU with the tiny model and the byte tokenizer (in-process ASGI client)."""
import json

import pytest
import torch
from starlette.testclient import TestClient

from blaze_b200.config import named_config
from blaze_b200.llm import LLM
from blaze_b200.server.app import ServerState, create_app
from blaze_b200.service import ServiceArgs
from blaze_b200.text import ByteTokenizer


@pytest.fixture(scope="module")
def client():
    st = ServerState(ServiceArgs(api_keys=("secret",), default_max_tokens=8), "tiny")
    app = create_app(st)
    c = TestClient(app)
    # while loading: 503 with the load stage
    r = c.get("/v1/models", headers={"authorization": "Bearer secret"})
    assert r.status_code == 503 and r.json()["error"]["code"] == "model_loading"
    llm = LLM(named_config("tiny"), device="cpu", dtype=torch.float32, max_seqs=8, max_model_len=512, use_graphs=False)
    st.attach(llm, ByteTokenizer(1024))
    yield c
    llm.sched.stop()


H = {"authorization": "Bearer secret"}


def test_control_plane(client):
    assert client.get("/health").json() == {"status": "ok"}
    assert client.get("/ping").text == "pong"
    assert client.get("/v1/models").status_code == 401
    assert client.get("/v1/models", headers={"x-api-key": "secret"}).json()["data"][0]["id"] == "tiny"
    assert client.get("/v1/models/nope", headers=H).status_code == 404
    info = client.get("/server_info", headers=H).json()
    assert info["model"] == "tiny" and "stats" in info
    m = client.get("/metrics").text
    assert "blaze_requests_total" in m and "blaze_time_to_first_token_seconds_bucket" in m


def test_tokenize_roundtrip(client):
    r = client.post("/tokenize", json={"prompt": "héllo"}, headers=H).json()
    assert r["count"] == len("héllo".encode())
    assert client.post("/detokenize", json={"tokens": r["tokens"]}, headers=H).json()["prompt"] == "héllo"
    r = client.post("/tokenize", json={"messages": [{"role": "user", "content": "hi"}]}, headers=H).json()
    assert r["count"] > 4


def test_completions_and_validation(client):
    r = client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 5, "temperature": 0}, headers=H)
    assert r.status_code == 200
    j = r.json()
    assert j["usage"]["completion_tokens"] == 5 and j["choices"][0]["finish_reason"] == "length"
    again = client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 5, "temperature": 0}, headers=H).json()
    assert again["choices"][0]["text"] == j["choices"][0]["text"]
    ids = client.post("/v1/completions", json={"prompt": [97, 98, 99], "max_tokens": 5, "temperature": 0, "logprobs": 2}, headers=H).json()
    assert ids["choices"][0]["text"] == j["choices"][0]["text"]
    assert len(ids["choices"][0]["logprobs"]["token_logprobs"]) == 5
    for bad in ({"prompt": "a", "temperature": -1}, {"prompt": "a", "top_p": 0}, {"prompt": "a", "n": 100},
                {"prompt": "a", "logit_bias": {"5": 500}}, {"prompt": "a", "presence_penalty": 3}, {"prompt": 5},
                {"prompt": "a", "samplers": "top_k,top_k"}, {"prompt": "a", "top_h": 0.5}, {"prompt": "a", "model": "other"},
                {"prompt": "a", "min_tokens": 9, "max_tokens": 3}, {"prompt": "x" * 600}):
        rr = client.post("/v1/completions", json=bad, headers=H)
        assert rr.status_code in (400, 404), (bad, rr.text)
        assert "error" in rr.json()
    two = client.post("/v1/completions", json={"prompt": ["ab", "cd"], "n": 2, "max_tokens": 3, "seed": 1}, headers=H).json()
    assert len(two["choices"]) == 4


def test_chat_and_stream(client):
    body = {"messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "temperature": 0}
    r = client.post("/v1/chat/completions", json=body, headers=H).json()
    assert r["object"] == "chat.completion" and r["choices"][0]["message"]["role"] == "assistant"
    assert r["usage"]["completion_tokens"] <= 6
    with client.stream("POST", "/v1/chat/completions", json={**body, "stream": True, "stream_options": {"include_usage": True}}, headers=H) as s:
        lines = [l for l in s.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    text = "".join(c["choices"][0]["delta"].get("content") or "" for c in chunks if c["choices"])
    assert text == (r["choices"][0]["message"]["content"] or "")
    assert chunks[-1]["usage"]["completion_tokens"] == r["usage"]["completion_tokens"]
    assert any(c["choices"] and c["choices"][0]["finish_reason"] for c in chunks)


def test_stop_string_and_choice_constraint(client):
    free = client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 8, "temperature": 0}, headers=H).json()["choices"][0]["text"]
    if len(free) >= 3:
        stop = free[2]
        cut = client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 8, "temperature": 0, "stop": stop}, headers=H).json()
        assert cut["choices"][0]["finish_reason"] == "stop" and stop not in cut["choices"][0]["text"]
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "pick"}], "max_tokens": 8,
                                                  "guided_choice": ["yes", "no"]}, headers=H).json()
    assert r["choices"][0]["message"]["content"] in ("yes", "no")


def test_embeddings_responses_messages(client):
    e = client.post("/v1/embeddings", json={"input": ["hello", "world"], "dimensions": 16}, headers=H).json()
    assert len(e["data"]) == 2 and len(e["data"][0]["embedding"]) == 16
    assert abs(sum(x * x for x in e["data"][0]["embedding"]) - 1.0) < 1e-3
    r = client.post("/v1/responses", json={"input": "hi", "max_output_tokens": 4, "temperature": 0}, headers=H).json()
    assert r["object"] == "response" and r["status"] in ("completed", "incomplete")
    assert client.get(f"/v1/responses/{r['id']}", headers=H).json()["id"] == r["id"]
    r2 = client.post("/v1/responses", json={"input": "more", "previous_response_id": r["id"], "max_output_tokens": 4}, headers=H)
    assert r2.status_code == 200 and r2.json()["usage"]["input_tokens"] > r["usage"]["input_tokens"]
    assert client.post("/v1/responses", json={"input": "x", "previous_response_id": "resp_missing"}, headers=H).status_code == 404
    m = client.post("/v1/messages", json={"max_tokens": 5, "messages": [{"role": "user", "content": "hi"}], "system": "be brief"}, headers=H).json()
    assert m["type"] == "message" and m["stop_reason"] in ("max_tokens", "end_turn") and m["content"][0]["type"] == "text"
    ct = client.post("/v1/messages/count_tokens", json={"messages": [{"role": "user", "content": "hi"}]}, headers=H).json()
    assert ct["input_tokens"] > 0
    with client.stream("POST", "/v1/messages", json={"max_tokens": 4, "stream": True, "messages": [{"role": "user", "content": "hi"}]}, headers=H) as s:
        ev = [l for l in s.iter_lines() if l.startswith("event: ")]
    assert ev[0] == "event: message_start" and ev[-1] == "event: message_stop"


# ---------------------------------------------------------------------------------------------- chat families
_FAMILY_TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {
    "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}, "opts": {"type": "object"}}}}}]
_FAMILY_CALL = {"id": "c1", "type": "function", "function": {
    "name": "get_weather", "arguments": json.dumps({"city": "Paris & \"Lyon\"", "days": 3, "opts": {"unit": "C"}})}}


def _stream(parser, text, step):
    content, calls = "", []
    for i in range(0, len(text), step):
        c, k = parser.push(text[i:i + step])
        content, calls = content + c, calls + k
    c, k = parser.flush()
    return content + c, calls + k


@pytest.mark.parametrize("family,parser", [("chatml", "hermes"), ("deepseek", "deepseek"), ("glm", "glm"), ("kimi", "kimi")])
def test_family_renderer_and_tool_parser_round_trip(family, parser):
    """What a family's renderer writes for an assistant tool call, its parser reads back, at any delta size."""
    from blaze_b200.chat import ChatFormatter, get_tool_parser
    msgs = [{"role": "developer", "content": "Be brief."}, {"role": "user", "content": [{"type": "text", "text": "Weather?"}]},
            {"role": "assistant", "content": "Looking.", "tool_calls": [_FAMILY_CALL, dict(_FAMILY_CALL, id="c2")]},
            {"role": "tool", "tool_call_id": "c1", "content": "sunny"}]
    fmt = ChatFormatter(family=family)
    full = fmt.render(msgs, _FAMILY_TOOLS)
    head = fmt.render(msgs[:2], _FAMILY_TOOLS, add_generation_prompt=False)
    assert full.startswith(head) and "Be brief." in head and "get_weather" in head
    turn = full[len(head):]
    for step in (1, 3, 11, 10_000):
        content, calls = _stream(get_tool_parser(parser, _FAMILY_TOOLS), turn, step)
        assert [c.name for c in calls[:2]] == ["get_weather", "get_weather"], (family, step, turn)
        assert json.loads(calls[0].arguments) == json.loads(_FAMILY_CALL["function"]["arguments"])
        assert "Looking." in content and "get_weather" not in content.split("sunny")[0]


def test_message_normalisation():
    from blaze_b200.chat.template import family_of, normalize_messages
    out = normalize_messages([{"role": "user", "content": "a"}, {"role": "user", "content": "b"},
                              {"role": "assistant", "content": None, "tool_calls": [{"function": {"name": "f", "arguments": ""}}]}],
                             "deepseek")
    assert [m["role"] for m in out] == ["system", "user", "assistant"] and out[1]["content"] == "a\n\nb"
    assert out[2]["content"] == "" and out[2]["tool_calls"][0]["function"]["arguments"] == {}
    with pytest.raises(ValueError):
        normalize_messages([{"role": "assistant", "tool_calls": [{"function": {"name": "f", "arguments": "[1]"}}]}])
    assert family_of("DeepSeek-V3.2") == "deepseek" and family_of("Kimi-K2") == "kimi" and family_of("Qwen3-8B") == "chatml"


def test_dsml_and_kimi_details():
    from blaze_b200.chat import get_think_parser, get_tool_parser
    M = "｜DSML｜"
    spaced = (f'<{M} calls><{M} invoke name="f"><{M} parameter name="s" string="true"> keep </{M} parameter>'
              f'<{M} parameter name="bad" string="false">{{oops</{M} parameter></{M} invoke></{M} calls>')
    _, calls = _stream(get_tool_parser("deepseek_v41"), spaced, 5)
    assert json.loads(calls[0].arguments) == {"s": " keep ", "bad": "{oops"}
    kimi = ('<|open|>tools<|sep|><|open|>call id="x"<|sep|><|close|>call<|sep|>'           # no tool name: dropped
            '<|open|>call tool="g" tool="h"<|sep|><|open|>argument key="v" type="array"<|sep|>[1, 2]<|close|>argument<|sep|>'
            '<|close|>call<|sep|><|close|>tools<|sep|>')
    _, calls = _stream(get_tool_parser("kimi"), kimi, 4)
    assert [(c.name, json.loads(c.arguments)) for c in calls] == [("h", {"v": [1, 2]})]
    think = get_think_parser("kimi_k3", starts_in_think=True)
    r, c = think.push("plan<|close|>think<|sep|>answer")
    fr, fc = think.flush()
    assert (r + fr, c + fc) == ("plan", "answer")


def test_server_with_another_chat_family():
    """A server configured for the Kimi markers renders with them and answers a chat request that carries tools."""
    st = ServerState(ServiceArgs(default_max_tokens=6, chat_family="kimi", tool_call_parser="kimi", reasoning_parser="kimi"), "tiny")
    c = TestClient(create_app(st))
    llm = LLM(named_config("tiny"), device="cpu", dtype=torch.float32, max_seqs=4, max_model_len=1024, use_graphs=False)
    try:
        st.attach(llm, ByteTokenizer(1024))
        assert st.formatter.family == "kimi"
        text = st.formatter.render([{"role": "user", "content": "hi"}])
        assert text.startswith('<|open|>message role="system"<|sep|>') and text.endswith("<|open|>think<|sep|>")
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6,
                                                  "temperature": 0, "tools": _FAMILY_TOOLS})
        assert r.status_code == 200, r.text
        msg = r.json()["choices"][0]["message"]
        assert msg["role"] == "assistant" and r.json()["usage"]["completion_tokens"] == 6
    finally:
        llm.sched.stop()


def test_protocol_details_clients_rely_on(client):
    """Behaviours that OpenAI-style clients and the reference's own API test client check: error objects on unknown routes
    and wrong methods, request ids, metric names, the info route, range checks, token strings, prompt truncation."""
    r = client.get("/v1/nope", headers=H)
    assert r.status_code == 404 and r.json()["error"]["type"] == "invalid_request_error"
    assert client.get("/v1/chat/completions", headers=H).status_code == 405
    r = client.get("/v1/models", headers={**H, "x-request-id": "trace-42"})
    assert r.headers["x-request-id"] == "trace-42"
    r = client.get("/v1/models", headers={**H, "x-request-id": "not a valid id"})
    assert r.headers["x-request-id"] and r.headers["x-request-id"] != "not a valid id"
    m = client.get("/metrics").text
    for name in ("blaze_requests_total", "blaze_requests_running", "blaze_requests_waiting", "blaze_requests_cancelled_total",
                 "blaze_prefill_tokens_total"):
        assert name in m, name
    info = client.get("/server_info", headers=H).json()
    assert "sampling_defaults" in info and "scheduler" in info and info["config"].get("api-key") == "[REDACTED]"
    assert "secret" not in json.dumps(info)
    for extra in ({"seed": -1}, {"stop_token_ids": [2 ** 64 - 1]}, {"stop_token_ids": ["bad"]}, {"top_logprobs": "many"},
                  {"stream": "yes"}, {"top_k": 1.5}, {"max_tokens": "ten"}, {"logit_bias": {"0": 101}}, {"echo": True, "logprobs": 1}):
        r = client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 2, **extra}, headers=H)
        assert r.status_code == 400 and "error" in r.json(), extra
    t = client.post("/tokenize", json={"prompt": "Hi", "return_token_strs": True}, headers=H).json()
    assert "".join(t["token_strs"]) == "Hi"
    assert client.post("/detokenize", json={"tokens": [10 ** 9]}, headers=H).status_code == 400
    # the chat form of /tokenize counts what the chat route uses as its prompt
    body = {"messages": [{"role": "user", "content": "Say hi."}], "chat_template_kwargs": {"enable_thinking": False}}
    n = client.post("/tokenize", json=body, headers=H).json()["count"]
    r = client.post("/v1/chat/completions", json={**body, "max_tokens": 2}, headers=H).json()
    assert r["usage"]["prompt_tokens"] == n
    big = "the " * 600
    r = client.post("/v1/completions", json={"prompt": big, "max_tokens": 3}, headers=H)
    assert r.status_code == 400 and r.json()["error"]["code"] == "context_length_exceeded"
    r = client.post("/v1/completions", json={"prompt": big, "max_tokens": 3, "truncate_prompt_tokens": 100}, headers=H)
    assert r.status_code == 200 and r.json()["usage"]["prompt_tokens"] == 100
    r = client.post("/v1/completions", json={"prompt": "Count: 1, 2,", "max_tokens": 5, "temperature": 0, "logprobs": 2}, headers=H).json()
    lp = r["choices"][0]["logprobs"]
    assert len(lp["tokens"]) == len(lp["token_logprobs"]) == len(lp["top_logprobs"]) == len(lp["text_offset"]) >= 2
    assert lp["text_offset"][0] == 0


TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {"city": {"type": "string"}}}}},
         {"type": "function", "function": {"name": "search", "parameters": {"type": "object", "properties": {"q": {"type": "string"}}}}}]


def test_tool_choice_and_continuation_are_validated(client):
    chat = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "temperature": 0}

    def err(extra):
        r = client.post("/v1/chat/completions", json={**chat, **extra}, headers=H)
        assert r.status_code == 400, r.text
        return r.json()["error"]

    assert err({"tool_choice": "required"})["param"] == "tool_choice"
    assert "not present in tools" in err({"tools": TOOLS, "tool_choice": {"type": "function", "function": {"name": "nope"}}})["message"]
    assert err({"tools": TOOLS, "tool_choice": "sometimes"})["param"] == "tool_choice"
    assert err({"continue_final_message": True})["param"] == "continue_final_message"          # last message is not the assistant's
    both = {"messages": chat["messages"] + [{"role": "assistant", "content": "It is"}], "continue_final_message": True,
            "add_generation_prompt": True}
    assert "cannot both be true" in err(both)["message"]
    # a continued assistant turn: the prompt ends with its text, the turn left open
    body = {"messages": chat["messages"] + [{"role": "assistant", "content": "It is"}], "continue_final_message": True}
    toks = client.post("/tokenize", json=body, headers=H).json()["tokens"]
    text = client.post("/detokenize", json={"tokens": toks, "skip_special_tokens": False}, headers=H).json()["prompt"]
    assert text.endswith("<|im_start|>assistant\nIt is")
    r = client.post("/v1/chat/completions", json={**chat, **body}, headers=H)
    assert r.status_code == 200 and r.json()["usage"]["prompt_tokens"] == len(toks)


def test_structured_output_on_the_byte_tokenizer(client):
    """Grammar constraints run through llguidance with any tokenizer that can name its tokens' bytes."""
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 24, "temperature": 0,
                                                  "chat_template_kwargs": {"enable_thinking": False},
                                                  "guided_regex": "(yes|no), [0-9]{3}!"}, headers=H)
    assert r.status_code == 200, r.text
    import re
    assert re.fullmatch(r"(yes|no), [0-9]{3}!", r.json()["choices"][0]["message"]["content"]), r.json()
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 200, "temperature": 0,
                                                  "chat_template_kwargs": {"enable_thinking": False},
                                                  "response_format": {"type": "json_schema", "json_schema": {"name": "s", "schema": {
                                                      "x-guidance": {"whitespace_flexible": False},     # a random model would pad forever
                                                      "type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer", "minimum": 0, "maximum": 9}},
                                                      "required": ["ok", "n"], "additionalProperties": False}}}}, headers=H)
    assert r.status_code == 200, r.text
    obj = json.loads(r.json()["choices"][0]["message"]["content"])
    assert set(obj) == {"ok", "n"} and isinstance(obj["ok"], bool) and 0 <= obj["n"] <= 9


def test_forced_tool_call_is_constrained_to_the_call_syntax():
    """``tool_choice`` naming a function (or "required") constrains the answer to calls of the listed tools in the parser's
    syntax, so even a random-init model answers with a call to the right tool."""
    st = ServerState(ServiceArgs(default_max_tokens=8, tool_call_parser="qwen3_coder", reasoning_parser=None), "tiny")
    c = TestClient(create_app(st))
    llm = LLM(named_config("tiny"), device="cpu", dtype=torch.float32, max_seqs=4, max_model_len=1024, use_graphs=False)
    st.attach(llm, ByteTokenizer(1024))
    try:
        body = {"messages": [{"role": "user", "content": "weather?"}], "tools": TOOLS, "max_tokens": 48, "temperature": 0,
                "chat_template_kwargs": {"enable_thinking": False}, "parallel_tool_calls": False}
        r = c.post("/v1/chat/completions", json={**body, "tool_choice": {"type": "function", "function": {"name": "search"}}})
        assert r.status_code == 200, r.text
        msg = r.json()["choices"][0]["message"]
        assert msg.get("tool_calls") and msg["tool_calls"][0]["function"]["name"] == "search", r.json()
        r = c.post("/v1/chat/completions", json={**body, "tool_choice": "required"})
        names = [t["function"]["name"] for t in r.json()["choices"][0]["message"]["tool_calls"]]
        assert names and set(names) <= {"get_weather", "search"}
    finally:
        llm.sched.stop()


def test_structured_output_fields_and_bounded_white_space():
    """``grammar_of``: every spelling of a structured-output request, and the white-space policy for JSON."""
    from blaze_b200.structured import ConstraintError, grammar_of
    ws64 = {"whitespace_pattern": "[\\x20\\x0A\\x0D\\x09]{1,64}"}
    assert grammar_of({"response_format": {"type": "json_object"}}) == {"kind": "json_schema", "schema": {"type": "object", "x-guidance": ws64}}
    s = {"type": "object", "properties": {"a": {"type": "integer"}}}
    for body in ({"response_format": {"type": "json_schema", "json_schema": {"name": "x", "schema": s}}}, {"guided_json": s},
                 {"structured_outputs": {"json": s}}, {"guided_decoding": {"json": json.dumps(s)}}, {"json_schema": s}):
        assert grammar_of(body)["schema"] == {**s, "x-guidance": ws64}, body
    assert grammar_of({"guided_json": s}, max_ws=0)["schema"] == s                                   # unbounded: the schema as given
    assert grammar_of({"guided_json": s, "disable_any_whitespace": True})["schema"]["x-guidance"] == {"whitespace_flexible": False}
    assert grammar_of({"structured_outputs": {"json": s, "whitespace_pattern": "[ ]?"}})["schema"]["x-guidance"] == {"whitespace_pattern": "[ ]?"}
    own = {**s, "x-guidance": {"whitespace_flexible": True}}
    assert grammar_of({"guided_json": own})["schema"] == own                                          # a schema's own setting wins
    assert grammar_of({"structured_outputs": {"json_object": True}})["schema"]["type"] == "object"
    assert grammar_of({"regex": "a+"}) == {"kind": "regex", "regex": "a+"}
    assert grammar_of({"structured_outputs": {"choice": ["a", "b"]}}) == {"kind": "choice", "choices": ["a", "b"]}
    assert grammar_of({"guided_grammar": 'start: "x"'})["kind"] == "grammar"
    assert grammar_of({"response_format": {"type": "text"}}) is None and grammar_of({}) is None
    for bad in ({"response_format": {"type": "json_schema"}}, {"response_format": {"type": "json_schema", "json_schema": {"name": "x"}}},
                {"response_format": {"type": "yaml"}}, {"guided_choice": []}, {"guided_regex": 5}):
        with pytest.raises(ConstraintError):
            grammar_of(bad)


def test_service_flags_layers_and_limits(tmp_path, capsys):
    from blaze_b200.cli import build_parser, main
    from blaze_b200.server.run import service_args_of
    model = tmp_path / "ckpt"
    model.mkdir()
    (model / "generation_config.json").write_text(json.dumps({"temperature": 0.6, "top_k": 20, "top_p": 0.95}))
    keys = tmp_path / "keys.txt"
    keys.write_text("k1\n\nk2\n")
    ns = build_parser().parse_args(["serve", "--model", str(model), "--override-generation-config", '{"top_k": 40, "min_p": 0.1}',
                                    "--instruct-sampling", '{"temperature": 0.7, "presence_penalty": 1.5}', "--top-p", "0.8",
                                    "--api-key", "k0", "--api-key-file", str(keys), "--allowed-origins", "https://a.example, https://b.example",
                                    "--max-queued-requests", "7", "--max-concurrent-requests", "3", "--shutdown-timeout", "2",
                                    "--max-request-body-mib", "1", "--disable-log-requests", "--log-inputs", "--repetition-penalty", "1.1"])
    svc = service_args_of(ns)
    # generation_config.json < --override-generation-config < explicit flags
    assert svc.defaults["temperature"] == 0.6 and svc.defaults["top_k"] == 40 and svc.defaults["min_p"] == 0.1 and svc.defaults["top_p"] == 0.8
    assert svc.defaults["repetition_penalty"] == 1.1 and svc.instruct_sampling == {"temperature": 0.7, "presence_penalty": 1.5}
    assert svc.api_keys == ("k0", "k1", "k2") and svc.cors_origins == ("https://a.example", "https://b.example")
    assert (svc.max_queue, svc.max_concurrency, svc.shutdown_timeout, svc.max_request_body_mib) == (7, 3, 2.0, 1)
    assert svc.log_requests is False and svc.log_inputs is True
    assert service_args_of(build_parser().parse_args(["serve", "--model", "tiny", "--allowed-origins", "none"])).cors_origins == ()
    with pytest.raises(SystemExit, match="unknown sampling parameter"):
        service_args_of(build_parser().parse_args(["serve", "--model", "tiny", "--instruct-sampling", '{"temperatur": 0.7}']))
    # --print-config shows the effective settings without the keys and loads nothing
    assert main(["serve", "--model", "tiny", "--api-key", "topsecret", "--print-config", "--top-k", "5"]) == 0
    out = capsys.readouterr().out
    assert "topsecret" not in out and '"top_k": 5' in out and "[REDACTED]" in out


def test_instruct_defaults_body_limit_and_cors():
    from blaze_b200.service import sampling_of
    svc = ServiceArgs(defaults={"temperature": 0.6, "top_p": 0.95}, instruct_sampling={"temperature": 0.7, "presence_penalty": 1.5},
                      max_request_body_mib=1, cors_origins=("https://a.example",), reasoning_parser="qwen3")
    think, plain = sampling_of({}, svc, 1024), sampling_of({}, svc, 1024, instruct=True)
    assert (think.temperature, think.presence_penalty) == (0.6, 0.0) and (plain.temperature, plain.presence_penalty, plain.top_p) == (0.7, 1.5, 0.95)
    assert sampling_of({"temperature": 0.1}, svc, 1024, instruct=True).temperature == 0.1          # the request wins
    st = ServerState(svc, "tiny")
    c = TestClient(create_app(st))
    llm = LLM(named_config("tiny"), device="cpu", dtype=torch.float32, max_seqs=4, max_model_len=256, use_graphs=False)
    st.attach(llm, ByteTokenizer(1024))
    try:
        r = c.post("/v1/completions", content=b'{"prompt": "' + b"x" * (1 << 20) + b'"}', headers={"content-type": "application/json"})
        assert r.status_code == 413 and r.json()["error"]["code"] == "request_too_large"
        r = c.get("/v1/models", headers={"origin": "https://a.example"})
        assert r.headers["access-control-allow-origin"] == "https://a.example"
        st.svc.cors_origins = ()
        assert "access-control-allow-origin" not in c.get("/v1/models").headers
    finally:
        llm.sched.stop()
