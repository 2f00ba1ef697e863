"""The HTTP server under traffic, with the real scheduler and the tiny model on CPU: an agent's growing conversation is
served from the prefix cache while side requests compete for it, more long generations than the KV pool holds all finish
(preemption and resume), and a mixed soak (streams, cancels mid-stream, JSON schemas, repeated prompts) leaves no request,
page or gauge behind.  The checks are those of the reference's ``scripts/prefix_cache_test.py``, ``kv_pressure_test.py``
and ``soak_test.py``, which run against a live server."""
import json
import random
import threading
import time

import torch
from starlette.testclient import TestClient

from blaze_b200.config import named_config
from blaze_b200.llm import LLM
from blaze_b200.server.app import ServerState, create_app
from blaze_b200.service import ServiceArgs
from blaze_b200.text import ByteTokenizer

WORDS = "module parser kernel cache tensor stream request batch graph token prefix router layer".split()


def _serve(**llm_kw):
    st = ServerState(ServiceArgs(default_max_tokens=16), "tiny")
    app = create_app(st)
    kw = dict(device="cpu", dtype=torch.float32, max_seqs=8, max_model_len=2048, use_graphs=False)
    kw.update(llm_kw)
    llm = LLM(named_config("tiny"), **kw)
    st.attach(llm, ByteTokenizer(1024))
    return TestClient(app), llm, st


def _chat_stream(c, messages, max_tokens):
    body = {"messages": messages, "max_tokens": max_tokens, "temperature": 0, "stream": True, "ignore_eos": True,
            "stream_options": {"include_usage": True}}
    text, usage = "", {}
    with c.stream("POST", "/v1/chat/completions", json=body) as s:
        assert s.status_code == 200
        for line in s.iter_lines():
            if not line.startswith("data: {"):
                continue
            ch = json.loads(line[6:])
            usage = ch.get("usage") or usage
            if ch["choices"] and ch["choices"][0]["delta"].get("content"):
                text += ch["choices"][0]["delta"]["content"]
    return text, usage["prompt_tokens"], (usage.get("prompt_tokens_details") or {}).get("cached_tokens", 0)


def test_an_agents_conversation_is_served_from_the_prefix_cache():
    c, llm, _ = _serve()
    rng = random.Random(3)
    system = "You are a coding agent. Project notes: " + " ".join(rng.choice(WORDS) for _ in range(60))
    msgs = [{"role": "system", "content": system}]
    try:
        for turn in range(4):
            msgs.append({"role": "user", "content": f"Step {turn + 1}: how does the {rng.choice(WORDS)} talk to the {rng.choice(WORDS)}?"})
            text, prompt, cached = _chat_stream(c, msgs, 12)
            msgs.append({"role": "assistant", "content": text})
            if turn:
                # every turn after the first starts from the previous turn's conversation: at least its prompt is cached
                assert cached >= last_prompt - 32, (turn, cached, last_prompt)
                assert cached < prompt
            last_prompt = prompt
            for _ in range(2):
                side = [{"role": "user", "content": "Give a five-word title for: " + " ".join(rng.choice(WORDS) for _ in range(12))}]
                _chat_stream(c, side, 4)
    finally:
        llm.sched.stop()


def test_more_long_generations_than_the_kv_pool_holds_all_finish():
    # 4 x (40-byte prompt + 150 tokens) needs about 800 slots; the pool has 512: the newest request is preempted and resumed
    c, llm, st = _serve(kv_tokens=512, max_seqs=4, max_model_len=512)
    out = [None] * 4

    def run(i):
        body = {"messages": [{"role": "user", "content": f"Write a long story number {i}."}], "max_tokens": 150, "temperature": 0.8,
                "seed": i, "ignore_eos": True}
        r = c.post("/v1/chat/completions", json=body)
        out[i] = (r.status_code, r.json())
    try:
        ts = [threading.Thread(target=run, args=(i,)) for i in range(4)]
        [t.start() for t in ts]
        [t.join(timeout=600) for t in ts]
        for status, body in out:
            assert status == 200, body
            ch = body["choices"][0]
            assert ch["finish_reason"] == "length" and body["usage"]["completion_tokens"] == 150
        assert llm.sched.stats.preemptions > 0, "the pool was meant to be too small"
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "Say ok."}], "max_tokens": 4})
        assert r.status_code == 200
    finally:
        llm.sched.stop()


def test_mixed_soak_leaves_nothing_behind():
    c, llm, st = _serve()
    schema = {"type": "object", "properties": {"title": {"type": "string", "maxLength": 8}, "score": {"type": "integer"}},
              "required": ["title", "score"], "additionalProperties": False}
    errors = []
    done = [0]

    def client(seed):
        rng = random.Random(seed)
        for _ in range(6):
            kind = rng.choice(["plain", "stream", "cancel", "schema", "repeat", "completion"])
            try:
                if kind == "plain":
                    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": " ".join(rng.choice(WORDS) for _ in range(20))}],
                                                             "max_tokens": rng.randint(1, 24), "temperature": 0.7, "seed": seed})
                    assert r.status_code == 200 and r.json()["choices"][0]["finish_reason"] in ("stop", "length")
                elif kind == "stream":
                    _chat_stream(c, [{"role": "user", "content": " ".join(rng.choice(WORDS) for _ in range(40))}], rng.randint(2, 30))
                elif kind == "cancel":
                    body = {"messages": [{"role": "user", "content": "a long one"}], "max_tokens": 400, "stream": True, "ignore_eos": True}
                    with c.stream("POST", "/v1/chat/completions", json=body) as s:
                        for n, line in enumerate(s.iter_lines()):
                            if n >= 6:
                                break           # the client walks away mid-stream
                elif kind == "schema":
                    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "rate this"}], "max_tokens": 120,
                                                             "response_format": {"type": "json_schema", "json_schema": {"schema": {**schema, "x-guidance": {"whitespace_flexible": False}}}}})
                    assert r.status_code == 200
                    ch = r.json()["choices"][0]
                    if ch["finish_reason"] == "stop":
                        j = json.loads(ch["message"]["content"])
                        assert set(j) == {"title", "score"} and isinstance(j["score"], int)
                elif kind == "repeat":
                    m = [{"role": "system", "content": "shared notes: " + " ".join(WORDS * 3)}, {"role": "user", "content": "again"}]
                    r = c.post("/v1/chat/completions", json={"messages": m, "max_tokens": 5})
                    assert r.status_code == 200
                else:
                    r = c.post("/v1/completions", json={"prompt": ["abc", "abd"], "max_tokens": 6, "n": 2, "seed": seed})
                    assert r.status_code == 200 and len(r.json()["choices"]) == 4
                done[0] += 1
            except Exception as e:          # noqa: BLE001 — collected and reported by the main thread
                errors.append((kind, repr(e)))
    try:
        ts = [threading.Thread(target=client, args=(s,)) for s in range(5)]
        [t.start() for t in ts]
        [t.join(timeout=900) for t in ts]
        assert not errors, errors
        assert done[0] == 30
        # nothing is left running, waiting or holding pages (the prefix cache's snapshots aside)
        t0 = time.monotonic()
        while (llm.sched.active or st.totals.inflight) and time.monotonic() - t0 < 30:
            time.sleep(0.05)
        assert not llm.sched.active and st.totals.inflight == 0 and st.waiting == 0
        eng = llm.engine
        held = sum(len(e.snap.pages) for e in llm.sched.cache.entries)
        assert eng.pages.free_count >= eng.num_pages - 1 - held
        assert c.get("/health").json() == {"status": "ok"}
        m = c.get("/metrics").text
        assert "blaze_requests_running 0" in m
    finally:
        llm.sched.stop()
