"""Pipeline parallelism on CPU: remote stage over TCP, and NCCL-style p2p stages as gloo ranks."""
import socket
import threading

import torch

from blaze_b200.config import named_config
from blaze_b200.engine import Engine, EngineConfig
from blaze_b200.models.qwen3 import Model
from blaze_b200.parallel.pp import cut_parts, stage_layers
from blaze_b200.remote import RemoteStage, get_plan, put_plan, serve_connection


def _engine(first, last):
    cfg = named_config("tiny")
    m = Model.random_init(cfg, seed=0, device="cpu", dtype=torch.float32, first_layer=first, last_layer=last)
    return Engine(m, EngineConfig(max_seqs=4, max_model_len=64, kv_dtype="fp32", use_graphs=False)), m


def test_split_helpers_and_wire_format():
    assert [stage_layers(48, 2, s) for s in range(2)] == [(0, 24), (24, 48)]
    assert [stage_layers(5, 2, s) for s in range(2)] == [(0, 2), (2, 5)]
    assert cut_parts(1100, 512) == [(0, 512), (512, 1024), (1024, 1100)]
    from blaze_b200.batch import SeqChunk
    chunks = [SeqChunk(2, [5, 6, 7], 10, 1), SeqChunk(0, [9], 3, 1)]
    back = get_plan(put_plan(chunks))
    assert [(c.slot, list(c.tokens), c.start_pos, c.want_logits) for c in back] == [(2, [5, 6, 7], 10, 1), (0, [9], 3, 1)]


def test_remote_stage_matches_single_process():
    full_eng, full = _engine(0, None)
    e0, m0 = _engine(0, 1)
    e1, m1 = _engine(1, 2)
    srv = socket.create_server(("127.0.0.1", 0))
    port = srv.getsockname()[1]

    def worker():
        conn, _ = srv.accept()
        try:
            serve_connection(conn, e1, m1)
        finally:
            conn.close()
    th = threading.Thread(target=worker, daemon=True)
    th.start()
    remote = RemoteStage("127.0.0.1", port)
    prompts = torch.randint(0, 1024, (2, 12), generator=torch.Generator().manual_seed(3)).tolist()
    fs = [full_eng.open_from() for _ in prompts]
    ss = [e0.open_from() for _ in prompts]
    want = full_eng.forward(full_eng.plan([(s, p, 1) for s, p in zip(fs, prompts)]), "greedy").tolist()
    got_all, want_all = [], [want]
    chunks = e0.plan([(s, p, 1) for s, p in zip(ss, prompts)])
    x = m0.forward(e0._build(chunks), e0.kv)
    got = remote.step(chunks, x).tolist()
    got_all.append(got)
    for _ in range(4):
        want = full_eng.forward(full_eng.plan([(s, [t], 1) for s, t in zip(fs, want)]), "greedy").tolist()
        want_all.append(want)
        chunks = e0.plan([(s, [t], 1) for s, t in zip(ss, got)])
        x = m0.forward(e0._build(chunks), e0.kv)
        got = remote.step(chunks, x).tolist()
        got_all.append(got)
    remote.close()
    th.join(timeout=5)
    assert got_all == want_all
