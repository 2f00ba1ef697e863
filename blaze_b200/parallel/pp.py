"""Pipeline parallelism: an even split of the layers over stages; a step's rows flow from stage to stage in micro-batches
of at most ``--pp-chunk`` rows, so that stage s+1 works on micro-batch i while stage s computes micro-batch i+1.

Reference: ``crates/blaze/src/engine.rs`` (``pp_parts`` :1328, ``cut_parts`` :1612 — a step is cut into ``--pp-chunk`` row
chunks; even split ``s*L/stages`` :826-1020; lm_head only on the last stage ``model.rs:1278``) and
``kernels/src/cuda/pp_link.cu`` (two-slot mailbox in mapped host memory with an unbounded device-side wait).
Here ranks are processes (one per GPU), laid out stage-major: global rank = stage * tp + tp_rank.  The hand-off between
rank r and r + tp is a ``torch.distributed`` ``isend`` / ``irecv`` pair per micro-batch (NCCL on GPUs, gloo on CPU),
posted on a side stream and double-buffered; nothing waits on the device without the library's own timeout.  Every rank
executes the same step plan (published by global rank 0 over the control group); the last stage returns the step's
result (tokens or logits) to global rank 0.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..batch import SeqChunk


def stage_layers(num_layers: int, stages: int, stage: int) -> Tuple[int, int]:
    """Layers [first, last) of ``stage`` (even split, ``s * L / stages``)."""
    return stage * num_layers // stages, (stage + 1) * num_layers // stages


def cut_parts(rows: int, chunk: int) -> List[Tuple[int, int]]:
    """Row ranges of at most ``chunk`` rows."""
    return [(i, min(rows, i + chunk)) for i in range(0, max(rows, 1), max(chunk, 1))] if rows else []


def split_step(chunks: Sequence[SeqChunk], pp_chunk: int) -> List[List[SeqChunk]]:
    """Cut a step into micro-batches of at most ``pp_chunk`` rows.  Whole sequence chunks are kept together when they fit;
    a longer prompt chunk is cut into consecutive pieces (later pieces attend to the KV the earlier ones wrote, because the
    micro-batches run in order on every stage); only the piece that holds a chunk's last rows keeps its logit rows.
    Draft-tree and deferred-state chunks are never cut."""
    pp_chunk = max(int(pp_chunk), 1)
    out: List[List[SeqChunk]] = []
    cur: List[SeqChunk] = []
    room = pp_chunk
    for c in chunks:
        n = len(c.tokens)
        if c.parents is not None or c.defer_state or n <= room:
            if n > room and cur:
                out.append(cur)
                cur, room = [], pp_chunk
            cur.append(c)
            room -= n
            if room <= 0:
                out.append(cur)
                cur, room = [], pp_chunk
            continue
        a = 0
        while a < n:
            if room <= 0:
                out.append(cur)
                cur, room = [], pp_chunk
            b = min(n, a + room)
            keep = max(0, c.want_logits - (n - b))          # logit rows that fall inside [a, b)
            keep = min(keep, b - a)
            cur.append(SeqChunk(slot=c.slot, tokens=list(c.tokens[a:b]), start_pos=c.start_pos + a, want_logits=keep))
            room -= b - a
            a = b
    if cur:
        out.append(cur)
    return out


class StageLink:
    """Point-to-point hand-off of hidden rows between consecutive pipeline stages (same tensor-parallel rank)."""

    def __init__(self, prev_rank: Optional[int], next_rank: Optional[int], hidden: int, max_rows: int, device,
                 dtype=torch.bfloat16, group=None):
        self.prev, self.next, self.group = prev_rank, next_rank, group
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.side = torch.cuda.Stream(self.device) if self.cuda else None
        self.hidden, self.dtype, self.max_rows = hidden, dtype, max_rows
        self.send_bufs = [torch.empty(max_rows, hidden, dtype=dtype, device=device) for _ in range(2)] if next_rank is not None else []
        self.recv_bufs = [torch.empty(max_rows, hidden, dtype=dtype, device=device) for _ in range(2)] if prev_rank is not None else []
        self.sends: List = []
        self.ks = self.kr = 0
        self.posted = None            # (work, buffer view, event) of the receive posted ahead

    # ------------------------------------------------------------------ sending
    def send(self, rows: torch.Tensor) -> None:
        """Ship ``rows`` to the next stage without blocking the compute stream."""
        if self.next is None:
            return
        n = rows.shape[0]
        if n > self.max_rows:
            raise ValueError(f"micro-batch of {n} rows exceeds the link buffers ({self.max_rows})")
        while len(self.sends) >= 2:             # the buffer about to be reused must have left
            self.sends.pop(0).wait()
        buf = self.send_bufs[self.ks & 1][:n]
        self.ks += 1
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.side):
                self.side.wait_event(ev)
                buf.copy_(rows, non_blocking=True)
                self.sends.append(dist.isend(buf, self.next, group=self.group))
        else:
            buf.copy_(rows)
            self.sends.append(dist.isend(buf, self.next, group=self.group))

    # ------------------------------------------------------------------ receiving
    def post_recv(self, n_rows: int) -> None:
        """Post the receive of the next micro-batch (called before the current one is computed, so the transfer overlaps)."""
        if self.prev is None or self.posted is not None:
            return
        if n_rows > self.max_rows:
            raise ValueError(f"micro-batch of {n_rows} rows exceeds the link buffers ({self.max_rows})")
        buf = self.recv_bufs[self.kr & 1][:n_rows]
        self.kr += 1
        if self.cuda:
            with torch.cuda.stream(self.side):
                work = dist.irecv(buf, self.prev, group=self.group)
                work.wait()                                    # orders the side stream after the transfer, not the host
                ev = torch.cuda.Event()
                ev.record(self.side)
            self.posted = (work, buf, ev)
        else:
            self.posted = (dist.irecv(buf, self.prev, group=self.group), buf, None)

    def recv(self, n_rows: int) -> torch.Tensor:
        if self.prev is None:
            raise RuntimeError("the first stage has nothing to receive")
        if self.posted is None:
            self.post_recv(n_rows)
        work, buf, ev = self.posted
        self.posted = None
        if buf.shape[0] != n_rows:
            raise RuntimeError("receive posted for a different micro-batch size")
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
        else:
            work.wait()
        return buf

    def flush(self) -> None:
        for w in self.sends:
            w.wait()
        self.sends = []


class Pipeline:
    """Wraps one rank's engine so that ``engine.forward`` runs this stage's part of a pipelined step.

    ``group`` is the rank layout from ``TPGroup.from_env(..., pp=stages)``: ``stage``, ``stages``, ``global_rank``, ``tp``
    (ranks per stage).  The wrapped ``forward`` has the engine's signature and result on global rank 0; on other ranks it
    returns what the stage produced (hidden rows, or the result on the last stage)."""

    def __init__(self, engine, group, pp_chunk: int = 512):
        self.engine, self.group, self.pp_chunk = engine, group, max(int(pp_chunk), 1)
        self.stage, self.stages, self.tpw = group.stage, group.stages, group.world
        g = group.global_rank
        prev = g - self.tpw if self.stage > 0 else None
        nxt = g + self.tpw if self.stage < self.stages - 1 else None
        cfg = engine.model.cfg
        self.link = StageLink(prev, nxt, cfg.hidden_size, max(self.pp_chunk, 64), engine.device, engine.model.dtype)
        self.last_root = (self.stages - 1) * self.tpw           # global rank of the last stage's first tensor-parallel rank
        self._local = engine.forward
        engine.forward = self.forward
        self.micro_batches = 0

    def forward(self, chunks, mode: str = "greedy", hidden_in=None, feedback: bool = False):
        if feedback:
            raise RuntimeError("token feedback is not available with pipeline stages")
        if mode not in ("greedy", "logits", "none"):
            raise ValueError(f"mode {mode!r} is not available with pipeline stages (a drafter needs the hidden rows)")
        eng, link = self.engine, self.link
        parts = split_step(chunks, self.pp_chunk)
        first, last = self.stage == 0, self.stage == self.stages - 1
        outs = []
        if not first and parts:
            link.post_recv(sum(len(c.tokens) for c in parts[0]))
        for i, mb in enumerate(parts):
            rows = sum(len(c.tokens) for c in mb)
            x_in = None
            if not first:
                x_in = link.recv(rows)
                if i + 1 < len(parts):
                    link.post_recv(sum(len(c.tokens) for c in parts[i + 1]))
            want = any(c.want_logits for c in mb)
            out = self._local(mb, (mode if want else "none") if last else "none", hidden_in=x_in)   # earlier stages return hidden rows
            self.micro_batches += 1
            if not last:
                link.send(out)
            elif out is not None:
                outs.append(out)
        link.flush()
        result = torch.cat(outs) if len(outs) > 1 else (outs[0] if outs else None)
        return self._return_to_root(result, chunks, mode)

    def _return_to_root(self, result, chunks, mode):
        """The last stage's first tensor-parallel rank sends the step's result to global rank 0 (which plans the steps)."""
        if mode == "none" or self.stages == 1:
            return result
        g = self.group.global_rank
        R = sum(c.want_logits for c in chunks)
        if R == 0:
            return result
        if g == self.last_root and g != 0:
            dist.send(result.contiguous(), 0)
        elif g == 0 and self.last_root != 0:
            eng = self.engine
            if mode == "greedy":
                result = torch.empty(R, dtype=torch.int64, device=eng.device)
            else:
                result = torch.empty(R, eng.model.cfg.vocab_size, dtype=torch.float32, device=eng.device)
            dist.recv(result, self.last_root)
        return result
