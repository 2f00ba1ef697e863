"""Tensor-parallel group: one process per GPU, ``torch.distributed`` for bootstrap, NCCL as the library
baseline, and the fused peer-memory kernels (``parallel/symm.py``) as the product path.

The reference runs ranks as threads and reduces through pinned host memory (``kernels/src/cuda/host_allreduce.cu``,
``crates/blaze/src/model.rs:2555-2716``: ``reduce_norm``, ``all_reduce``, ``head``, ``greedy_sharded``); the
placements are the same here (two reductions per layer, sharded lm_head with a (value, index) merge for greedy
decoding), the transport is NVLink.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist


class TPGroup:
    def __init__(self, rank: int, world: int, pg=None, device=None, fused=None):
        self.rank, self.world, self.pg, self.device = rank, world, pg, device
        self.fused = fused           # parallel.symm.SymmAllReduce or None
        self.bytes_reduced = 0
        self.calls = 0

    # pipeline layout (one stage unless from_env is given pp > 1): ranks are stage-major, global rank = stage * world + rank
    stage, stages = 0, 1

    @property
    def global_rank(self) -> int:
        return self.stage * self.world + self.rank

    @classmethod
    def from_env(cls, device=None, backend: Optional[str] = None, pp: int = 1) -> Optional["TPGroup"]:
        """Join the process group described by RANK / WORLD_SIZE / MASTER_* (torchrun).  With ``pp`` pipeline stages the
        WORLD_SIZE ranks form ``pp`` stages of ``WORLD_SIZE / pp`` tensor-parallel ranks each; the returned group does the
        collectives of this rank's stage, ``ctrl`` spans every rank (step plans), and point-to-point hand-offs between
        stages use the default group."""
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world == 1:
            return None
        rank = int(os.environ["RANK"])
        if pp > 1:
            return cls._from_env_pp(device, backend, pp, rank, world)
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            if backend is None:
                backend = "nccl" if (device is not None and torch.device(device).type == "cuda") else "gloo"
            kw = {}
            if backend == "nccl":
                kw["device_id"] = torch.device(device)
            dist.init_process_group(backend, rank=rank, world_size=world, **kw)
        g = cls(rank, world, dist.group.WORLD, device)
        if dist.get_backend() == "nccl":
            # Control messages (step plans, quit) travel over a host-side group: an object broadcast over NCCL is ordered
            # behind the kernels already queued on the stream and would make every rank wait for the GPU each step.
            g.ctrl = dist.new_group(backend="gloo")
        return g

    @classmethod
    def _from_env_pp(cls, device, backend, pp: int, grank: int, gworld: int) -> "TPGroup":
        if gworld % pp:
            raise ValueError(f"{gworld} ranks do not split into {pp} pipeline stages")
        tpw = gworld // pp
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            if backend is None:
                backend = "nccl" if (device is not None and torch.device(device).type == "cuda") else "gloo"
            kw = {"device_id": torch.device(device)} if backend == "nccl" else {}
            dist.init_process_group(backend, rank=grank, world_size=gworld, **kw)
        stage, tpr = grank // tpw, grank % tpw
        mine = None
        for s in range(pp):                       # every rank takes part in the creation of every stage's group
            ranks = list(range(s * tpw, (s + 1) * tpw))
            pg = dist.new_group(ranks) if tpw > 1 else None
            if s == stage:
                mine = pg
        g = cls(tpr, tpw, mine, device)
        g.stage, g.stages = stage, pp
        g.ctrl = dist.new_group(backend="gloo") if dist.get_backend() == "nccl" else dist.group.WORLD
        return g

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        self.calls += 1
        self.bytes_reduced += x.numel() * x.element_size()
        if self.fused is not None and x.is_cuda:
            y = self.fused.all_reduce(x)
            if y is not None:
                return y
        dist.all_reduce(x, group=self.pg)
        return x

    def all_gather_cols(self, x: torch.Tensor) -> torch.Tensor:
        """[R, n] shards → [R, n * world] (vocab-sharded logits)."""
        parts = [torch.empty_like(x) for _ in range(self.world)]
        dist.all_gather(parts, x.contiguous(), group=self.pg)
        return torch.cat(parts, dim=1)

    def argmax_sharded(self, ops, logits: torch.Tensor, shard: int) -> torch.Tensor:
        """Each rank reduces its vocab shard to (value, global index); the pairs are merged with the lowest index
        winning ties — 16 bytes per row per rank on the wire instead of the logits (``model.rs:2669``)."""
        off = self.rank * shard
        if ops.is_cuda:
            idx, val = ops.argmax(logits, index_offset=off, want_values=True)
        else:
            val, i = logits.max(dim=1)
            m = logits == val.unsqueeze(1)
            ar = torch.arange(logits.shape[1], device=logits.device).expand_as(logits)
            idx = torch.where(m, ar, torch.full_like(ar, logits.shape[1])).min(1).values + off
        return self.merge_pairs(idx, val)

    def merge_pairs(self, idx: torch.Tensor, val: torch.Tensor) -> torch.Tensor:
        """Merge every rank's per-row (global index, value) winner: largest value, lowest index among equals."""
        pair = torch.stack([val.double(), idx.double()], dim=1).contiguous()
        parts = [torch.empty_like(pair) for _ in range(self.world)]
        dist.all_gather(parts, pair, group=self.pg)
        allp = torch.stack(parts)                     # [world, R, 2]
        best_val = allp[:, :, 0].max(dim=0).values
        cand = torch.where(allp[:, :, 0] == best_val.unsqueeze(0), allp[:, :, 1], torch.full_like(allp[:, :, 1], 1e18))
        return cand.min(dim=0).values.long()

    def broadcast(self, t, src: int = 0):
        """Broadcast a tensor from tensor-parallel rank ``src`` of this stage over the data group."""
        dist.broadcast(t, src=dist.get_global_rank(self.pg, src) if self.pg is not None else src, group=self.pg)
        return t

    def broadcast_object(self, obj, src: int = 0):
        box = [obj]
        dist.broadcast_object_list(box, src=src, group=getattr(self, "ctrl", None) or self.pg)
        return box[0]

    def barrier(self):
        if self.pg is not None or self.stages == 1:
            dist.barrier(group=self.pg)
