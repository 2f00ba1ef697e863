"""Host tier of the paged KV cache: snapshots pushed out of the device prefix cache are parked in pinned host memory and
brought back when a later prompt matches them.

One pool per attention layer, ``[host pages, bytes of one device page of that layer]``; an entry occupies a contiguous run
of host pages, so a spill or a restore is one gather / scatter kernel on the device side and ONE asynchronous copy per
layer over the copy engine, ordered on the stream that also runs the model (a page is never reused before the copy that
reads it).  Reference: ``kernels/src/cuda/kv_host.cu`` (gather :57, clear :83, claim :90) and ``--kv-host``
(``crates/blaze/src/model.rs:1666``) — there a device row cache over zero-copy host pools; here whole 16-token pages move.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .kv import KVCache


class HostKVTier:
    def __init__(self, kv: KVCache, host_pages: int):
        self.kv, self.capacity = kv, int(host_pages)
        pin = kv.device.type == "cuda"
        self.pools: Dict[Tuple[str, int], torch.Tensor] = {}
        for name, d in (("kv", kv.kv), ("k", kv.k), ("v", kv.v)):
            for layer, t in d.items():
                self.pools[(name, layer)] = torch.empty((self.capacity,) + tuple(t.shape[1:]), dtype=t.dtype, pin_memory=pin)
        self.free: List[Tuple[int, int]] = [(0, self.capacity)] if self.capacity > 0 else []     # (start, count) runs
        self.spilled_pages = self.restored_pages = 0

    # ------------------------------------------------------------------ run allocator
    @property
    def free_pages(self) -> int:
        return sum(n for _, n in self.free)

    def _alloc(self, n: int) -> Optional[int]:
        for i, (s, c) in enumerate(self.free):
            if c >= n:
                if c == n:
                    self.free.pop(i)
                else:
                    self.free[i] = (s + n, c - n)
                return s
        return None

    def drop(self, run: Tuple[int, int]) -> None:
        """Give a run back; neighbouring free runs are merged."""
        runs = sorted(self.free + [run])
        out: List[Tuple[int, int]] = []
        for s, c in runs:
            if out and out[-1][0] + out[-1][1] == s:
                out[-1] = (out[-1][0], out[-1][1] + c)
            else:
                out.append((s, c))
        self.free = out

    # ------------------------------------------------------------------ data movement
    def _device_pool(self, name: str, layer: int) -> torch.Tensor:
        return getattr(self.kv, name)[layer]

    def spill(self, dev_pages: List[int]) -> Optional[Tuple[int, int]]:
        """Copy the given device pages to the host; returns the host run, or None when there is no room."""
        n = len(dev_pages)
        if n == 0 or self.kv.gdn_layers or getattr(self.kv, "idx_k", None):
            # recurrent state rows are not paged, and an indexer's key pages are not copied here: such models keep their
            # snapshots on the device
            return None
        s0 = self._alloc(n)
        if s0 is None:
            return None
        idx = torch.as_tensor(dev_pages, dtype=torch.long, device=self.kv.device)
        for (name, layer), host in self.pools.items():
            host[s0:s0 + n].copy_(self._device_pool(name, layer).index_select(0, idx), non_blocking=True)
        self.spilled_pages += n
        return (s0, n)

    def restore(self, run: Tuple[int, int], dev_pages: List[int]) -> None:
        """Copy a host run into freshly allocated device pages (same count)."""
        s0, n = run
        assert n == len(dev_pages)
        idx = torch.as_tensor(dev_pages, dtype=torch.long, device=self.kv.device)
        for (name, layer), host in self.pools.items():
            self._device_pool(name, layer).index_copy_(0, idx, host[s0:s0 + n].to(self.kv.device, non_blocking=True))
        self.restored_pages += n
