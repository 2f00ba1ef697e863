"""The HTTP load generator against a live server (uvicorn on a loop-back port, tiny model on CPU)."""
import json
import socket
import threading
import time

import torch

from blaze_b200.benchmarks import client as bc


def test_percentiles_and_prompts():
    assert bc.percentile([1, 2, 3, 4], 0.5) == 2.5 and bc.percentile([], 0.5) == 0.0
    import random
    a = bc.make_prompt(random.Random(0), 20, shared_prefix=8)
    b = bc.make_prompt(random.Random(1), 20, shared_prefix=8)
    assert len(a) == 20 and a[:8] == b[:8] and a[8:] != b[8:]


def test_client_against_live_server(capsys):
    import uvicorn

    from blaze_b200.config import named_config
    from blaze_b200.llm import LLM
    from blaze_b200.server.app import ServerState, create_app
    from blaze_b200.service import ServiceArgs
    from blaze_b200.text import ByteTokenizer

    st = ServerState(ServiceArgs(default_max_tokens=8), "tiny")
    app = create_app(st)
    llm = LLM(named_config("tiny"), device="cpu", dtype=torch.float32, max_seqs=8, max_model_len=512, use_graphs=False)
    st.attach(llm, ByteTokenizer(1024))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    try:
        for _ in range(100):
            if server.started:
                break
            time.sleep(0.05)
        assert server.started
        # token ids below the tiny model's vocabulary
        orig = bc.make_prompt
        bc.make_prompt = lambda rng, n, shared_prefix=0, prefix_seed=1: [rng.randrange(10, 250) for _ in range(n)]
        try:
            rc = bc.main(["--url", f"http://127.0.0.1:{port}", "--requests", "6", "--concurrency", "3", "--prompt-tokens", "24",
                          "--max-tokens", "5", "--warm"])
        finally:
            bc.make_prompt = orig
        assert rc == 0
        out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        warm = out["warm"]
        assert warm["failed"] == 0 and warm["requests"] == 6
        assert warm["output_tok_per_s"] > 0 and warm["ttft_s"]["p50"] > 0 and warm["e2e_s"]["p95"] >= warm["ttft_s"]["p50"]
    finally:
        server.should_exit = True
        th.join(timeout=10)
        llm.sched.stop()
