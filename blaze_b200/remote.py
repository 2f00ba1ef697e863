"""Remote pipeline stage over TCP: a coordinator relays step plans and hidden rows to a ``stage-worker`` process.

Reference: ``crates/blaze/src/remote.rs`` — binary wire format :13-70, ``put_meta`` / ``get_meta`` :72/:92, ``connect`` :358
(two connections: commands and data), ``serve`` :455 (the stage worker).  The only process/host boundary of the system.
Frames: ``magic u32 | kind u8 | len u64 | payload``; plans are length-prefixed little-endian int32 arrays, rows raw bf16.
"""
from __future__ import annotations

import socket
import struct
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

MAGIC = 0x424C5A31   # "BLZ1"
K_PLAN, K_ROWS, K_RESULT, K_QUIT, K_ERROR = 1, 2, 3, 4, 5
_HDR = struct.Struct("<IBQ")


def _send(sock: socket.socket, kind: int, payload: bytes) -> None:
    sock.sendall(_HDR.pack(MAGIC, kind, len(payload)) + payload)


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        part = sock.recv(min(n - len(buf), 1 << 20))
        if not part:
            raise ConnectionError("peer closed the connection")
        buf += part
    return bytes(buf)


def _recv(sock: socket.socket) -> Tuple[int, bytes]:
    magic, kind, n = _HDR.unpack(_recv_exact(sock, _HDR.size))
    if magic != MAGIC:
        raise ConnectionError("bad frame magic")
    return kind, _recv_exact(sock, n)


def put_plan(chunks) -> bytes:
    """SeqChunk list → bytes: count, then per chunk (slot, start_pos, want_logits, n, tokens…)."""
    out = [struct.pack("<i", len(chunks))]
    for c in chunks:
        toks = np.asarray(c.tokens, dtype=np.int32)
        out.append(struct.pack("<iiii", c.slot, c.start_pos, c.want_logits, toks.size))
        out.append(toks.tobytes())
    return b"".join(out)


def get_plan(data: bytes):
    from .batch import SeqChunk
    (n,) = struct.unpack_from("<i", data, 0)
    off, chunks = 4, []
    for _ in range(n):
        slot, start, want, k = struct.unpack_from("<iiii", data, off)
        off += 16
        toks = np.frombuffer(data, dtype=np.int32, count=k, offset=off).tolist()
        off += 4 * k
        chunks.append(SeqChunk(slot, toks, start, want))
    return chunks


def put_rows(x: torch.Tensor) -> bytes:
    t = x.detach().to(torch.bfloat16).contiguous().cpu()
    return struct.pack("<ii", t.shape[0], t.shape[1]) + t.view(torch.uint8).numpy().tobytes()


def get_rows(data: bytes, device) -> torch.Tensor:
    r, c = struct.unpack_from("<ii", data, 0)
    a = np.frombuffer(data, dtype=np.uint8, offset=8).copy()
    return torch.from_numpy(a).view(torch.bfloat16).view(r, c).to(device)


class RemoteStage:
    """Coordinator side: forwards each step's plan and hidden rows, returns the worker's result."""

    def __init__(self, host: str, port: int, timeout: float = 30.0):
        self.sock = socket.create_connection((host, port), timeout=timeout)
        self.sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)

    def step(self, chunks, rows: torch.Tensor, mode: str = "greedy") -> torch.Tensor:
        _send(self.sock, K_PLAN, mode.encode().ljust(8, b"\0") + put_plan(chunks))
        _send(self.sock, K_ROWS, put_rows(rows))
        kind, data = _recv(self.sock)
        if kind == K_ERROR:
            raise RuntimeError("remote stage failed: " + data.decode("utf-8", "replace"))
        n = len(data) // 8
        return torch.from_numpy(np.frombuffer(data, dtype=np.int64, count=n).copy())

    def close(self) -> None:
        try:
            _send(self.sock, K_QUIT, b"")
        finally:
            self.sock.close()


def serve_connection(conn: socket.socket, engine, model) -> None:
    """Worker side of one coordinator connection."""
    mode = "greedy"
    chunks = None
    while True:
        kind, data = _recv(conn)
        if kind == K_QUIT:
            return
        if kind == K_PLAN:
            mode = data[:8].rstrip(b"\0").decode()
            chunks = get_plan(data[8:])
            for c in chunks:     # the worker mirrors the coordinator's page bookkeeping from the plan
                s = engine.seqs.get(c.slot)
                if s is None:
                    while engine.free_rows and engine.free_rows[-1] != c.slot:
                        engine.free_rows.insert(0, engine.free_rows.pop())
                    s = engine.open_from()
                engine.reserve(s, c.start_pos + len(c.tokens))
                s.length = c.start_pos + len(c.tokens)
        elif kind == K_ROWS:
            try:
                x = get_rows(data, engine.device).to(model.dtype)
                batch = engine._build(chunks)
                h = model.forward(batch, engine.kv, x)
                out = model.greedy(h, batch.logit_rows) if mode == "greedy" else model.head(h, batch.logit_rows).argmax(-1)
                _send(conn, K_RESULT, out.to(torch.int64).cpu().numpy().tobytes())
            except Exception as e:  # report, keep the worker alive for the next step
                _send(conn, K_ERROR, repr(e).encode())


def serve_stage(ns) -> int:
    """``stage-worker`` command: load the last stage's layers and serve coordinators one at a time."""
    from .cli import build_llm
    from .parallel.pp import stage_layers
    llm = build_llm(ns)
    host, _, port = ns.listen.rpartition(":")
    srv = socket.create_server((host or "127.0.0.1", int(port)))
    while True:
        conn, _ = srv.accept()
        conn.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        try:
            serve_connection(conn, llm.engine, llm.model)
        except ConnectionError:
            pass
        finally:
            conn.close()
