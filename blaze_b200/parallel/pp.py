"""Pipeline parallelism: an even split of the layers over stages, rows handed from stage to stage in chunks.

Reference: ``crates/blaze/src/engine.rs`` (``pp_parts`` :1328, ``cut_parts`` :1612 — a step is cut into ``--pp-chunk`` row
chunks; even split ``s*L/stages`` :826-1020; lm_head only on the last stage ``model.rs:1278``) and
``kernels/src/cuda/pp_link.cu`` (two-slot mailbox in mapped host memory with an unbounded device-side wait).
Here the hand-off is NCCL ``isend`` / ``irecv`` on a side stream, double-buffered so the transfer of chunk i overlaps the
compute of chunk i+1; nothing waits on the device without the library's own timeout.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def stage_layers(num_layers: int, stages: int, stage: int) -> Tuple[int, int]:
    """Layers [first, last) of ``stage`` (even split, ``s * L / stages``)."""
    return stage * num_layers // stages, (stage + 1) * num_layers // stages


def cut_parts(rows: int, chunk: int) -> List[Tuple[int, int]]:
    """Row ranges of at most ``chunk`` rows."""
    return [(i, min(rows, i + chunk)) for i in range(0, max(rows, 1), max(chunk, 1))] if rows else []


class StageLink:
    """Point-to-point hand-off between consecutive pipeline stages."""

    def __init__(self, rank: int, prev_rank: Optional[int], next_rank: Optional[int], hidden: int, max_rows: int, device,
                 dtype=torch.bfloat16, group=None):
        self.rank, self.prev, self.next, self.group = rank, prev_rank, next_rank, group
        self.device = torch.device(device)
        self.side = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self.bufs = [torch.empty(max_rows, hidden, dtype=dtype, device=device) for _ in range(2)]
        self.meta = torch.zeros(2, dtype=torch.int64, device=device)
        self.pending: List = []
        self.k = 0

    def send(self, rows: torch.Tensor) -> None:
        """Ship ``rows`` to the next stage without blocking the compute stream."""
        if self.next is None:
            return
        buf = self.bufs[self.k & 1][:rows.shape[0]]
        self.k += 1
        if self.side is not None:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.side):
                self.side.wait_event(ev)
                buf.copy_(rows, non_blocking=True)
                self.pending.append(dist.isend(buf, self.next, group=self.group))
        else:
            buf.copy_(rows)
            self.pending.append(dist.isend(buf, self.next, group=self.group))
        while len(self.pending) > 2:
            self.pending.pop(0).wait()

    def recv(self, n_rows: int) -> torch.Tensor:
        if self.prev is None:
            raise RuntimeError("first stage has nothing to receive")
        buf = self.bufs[self.k & 1][:n_rows]
        self.k += 1
        dist.recv(buf, self.prev, group=self.group)
        return buf

    def flush(self) -> None:
        for w in self.pending:
            w.wait()
        self.pending = []


def pipeline_step(model, engine, link: StageLink, chunks, mode: str, pp_chunk: int = 512):
    """Run one engine step on this stage: receive rows (unless first), run the stage's layers chunk by chunk, send on
    (unless last).  Every stage builds the same batch metadata from the same plan."""
    from ..batch import build_batch
    batch = engine._build(chunks)
    T = batch.num_rows
    if model.is_first_stage:
        x = model.forward(batch, engine.kv)
    else:
        x_in = link.recv(T)
        x = model.forward(batch, engine.kv, x_in)
    if not model.is_last_stage:
        for lo, hi in cut_parts(T, pp_chunk):
            link.send(x[lo:hi])
        return None
    rows = batch.logit_rows
    if mode == "greedy":
        return model.greedy(x, rows)
    if mode == "logits":
        return model.head(x, rows)
    return None
