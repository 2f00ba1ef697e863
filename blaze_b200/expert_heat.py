"""Routing heat of a mixture-of-experts model: how many routed rows every expert of every layer has received, recent and
long-term, kept across restarts in a profile file, and what that load means for a placement of the experts over ranks.

The reference uses the same statistic to decide which experts live in which memory tier (``kernels/src/runtime/swap.cpp``:
``HeatProfile`` with a recent and a long-term score per (layer, expert) :139-184, written back periodically and merged per
pipeline stage :173-190, a periodic log line of where routes were served :528).  Here every expert is resident in HBM; the
tiers are the ranks of an expert-parallel group, so the profile answers: how uneven is the load under the contiguous
placement (experts ``r * E / world ..`` on rank r, what ``--ep`` uses), and how even could a heat-aware placement be.
``placement`` computes that assignment (largest load first onto the least loaded rank that still has a free slot);
``imbalance`` reports max-over-mean rank load for both.

Collection: ``observe(layer, ids)`` adds one step's routed expert ids into a device-resident ``[layers, experts]`` counter
(one ``scatter_add``; capturable in a CUDA graph); ``fold`` moves the counters to the host scores.  Off unless the model
is given a profile (``LLM(expert_heat=...)`` / ``--expert-heat PATH``)."""
from __future__ import annotations

import os
import struct
from typing import Any, Dict, Optional, Tuple

import numpy as np
import torch

MAGIC = b"BLZHEAT2"


class ExpertHeat:
    def __init__(self, num_layers: int, num_experts: int, device="cpu", half_life: float = 65536.0):
        """``half_life``: routed rows per layer after which an observation counts half in the recent score."""
        self.L, self.E = int(num_layers), int(num_experts)
        self.device = torch.device(device)
        self.half_life = float(half_life)
        self.recent = np.zeros((self.L, self.E), dtype=np.float64)
        self.longterm = np.zeros((self.L, self.E), dtype=np.float64)
        self._pending = torch.zeros(self.L, self.E, dtype=torch.int64, device=self.device)
        # allocated up front so that a first observation inside a graph capture allocates nothing
        self._ones: Optional[torch.Tensor] = torch.ones(1 << 17, dtype=torch.int64, device=self.device)
        self.path: Optional[str] = None
        self.layer_range: Optional[Tuple[int, int]] = None      # a pipeline stage's layers (others are kept as the file has them)

    # ------------------------------------------------------------------ collection
    def observe(self, layer: int, ids: torch.Tensor) -> None:
        """Add one step's routed expert ids (``[rows, top_k]``, global expert numbers) of ``layer``."""
        flat = ids.reshape(-1).long()
        if self._ones is None or self._ones.numel() < flat.numel():
            self._ones = torch.ones(flat.numel(), dtype=torch.int64, device=flat.device)
        self._pending[layer].scatter_add_(0, flat, self._ones[:flat.numel()])

    def fold(self) -> None:
        """Move the device counters into the host scores (one device→host copy)."""
        counts = self._pending.cpu().numpy().astype(np.float64)
        self._pending.zero_()
        rows = counts.sum(axis=1, keepdims=True)                 # routed rows per layer since the last fold
        decay = np.power(0.5, rows / self.half_life)
        self.recent = self.recent * decay + counts
        self.longterm += counts

    # ------------------------------------------------------------------ persistence
    def save(self, path: Optional[str] = None) -> None:
        """Write ``magic, layers, experts, recent[L*E], longterm[L*E]`` (little endian, float64) atomically.  With a
        ``layer_range`` only those layers are replaced in an existing profile of the same shape."""
        path = path or self.path
        if not path:
            return
        self.fold()
        recent, longterm = self.recent, self.longterm
        if self.layer_range is not None:
            old = ExpertHeat.load(path, self.L, self.E)
            if old is not None:
                a, b = self.layer_range
                recent, longterm = old.recent.copy(), old.longterm.copy()
                recent[a:b], longterm[a:b] = self.recent[a:b], self.longterm[a:b]
        tmp = path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(MAGIC + struct.pack("<II", self.L, self.E))
            f.write(np.ascontiguousarray(recent, dtype="<f8").tobytes())
            f.write(np.ascontiguousarray(longterm, dtype="<f8").tobytes())
        os.replace(tmp, path)

    @classmethod
    def load(cls, path: str, num_layers: int, num_experts: int, device="cpu") -> Optional["ExpertHeat"]:
        """The profile at ``path``; None when there is none or it is not a profile of ``num_experts`` experts.  A profile
        of another layer count (a drafter layer added or left out) keeps the layers that exist here, the rest start cold."""
        try:
            with open(path, "rb") as f:
                head = f.read(16)
                if len(head) != 16 or head[:8] != MAGIC:
                    return None
                L, E = struct.unpack("<II", head[8:])
                if E != num_experts or L == 0:
                    return None
                body = f.read()
        except OSError:
            return None
        n = L * E
        if len(body) != 2 * n * 8:
            return None
        arr = np.frombuffer(body, dtype="<f8")
        h = cls(num_layers, num_experts, device)
        keep = min(L, num_layers)
        h.recent[:keep] = arr[:n].reshape(L, E)[:keep]
        h.longterm[:keep] = arr[n:].reshape(L, E)[:keep]
        h.path = path
        return h

    @classmethod
    def open(cls, path: Optional[str], num_layers: int, num_experts: int, device="cpu") -> "ExpertHeat":
        """Load ``path`` if it holds a matching profile, else start cold; either way later ``save()`` calls write there."""
        h = (cls.load(path, num_layers, num_experts, device) if path else None) or cls(num_layers, num_experts, device)
        h.path = path
        return h

    # ------------------------------------------------------------------ placement
    def _load(self, recent: bool) -> np.ndarray:
        return self.recent if recent else self.longterm

    def placement(self, world: int, recent: bool = True) -> np.ndarray:
        """``[layers, experts]`` rank of every expert: per layer the experts go, heaviest first, to the rank with the least
        load so far among those holding fewer than ``experts / world`` experts (every rank holds the same number)."""
        if world <= 0 or self.E % world:
            raise ValueError(f"{self.E} experts do not split over {world} ranks")
        cap = self.E // world
        load = self._load(recent)
        out = np.zeros((self.L, self.E), dtype=np.int32)
        for l in range(self.L):
            order = np.argsort(-load[l], kind="stable")
            rank_load = np.zeros(world)
            held = np.zeros(world, dtype=np.int64)
            for e in order:
                open_ranks = np.nonzero(held < cap)[0]
                r = open_ranks[np.argmin(rank_load[open_ranks])]
                out[l, e] = r
                rank_load[r] += load[l, e]
                held[r] += 1
        return out

    @staticmethod
    def order_for(where: np.ndarray) -> np.ndarray:
        """Slot order that realises placement ``where`` (``[layers, experts]`` ranks) with contiguous slots per rank:
        slot j of a layer holds expert ``order[layer][j]``; experts keep their relative order inside a rank."""
        return np.stack([np.argsort(where[l], kind="stable") for l in range(where.shape[0])]).astype(np.int64)

    def contiguous(self, world: int) -> np.ndarray:
        """The placement expert parallelism uses: expert e on rank ``e // (experts / world)``."""
        if world <= 0 or self.E % world:
            raise ValueError(f"{self.E} experts do not split over {world} ranks")
        return np.broadcast_to((np.arange(self.E) // (self.E // world)).astype(np.int32), (self.L, self.E)).copy()

    def imbalance(self, world: int, where: Optional[np.ndarray] = None, recent: bool = True) -> np.ndarray:
        """Per layer: load of the busiest rank over the mean rank load under placement ``where`` (default contiguous);
        1.0 is perfectly even, ``world`` is everything on one rank.  Layers without observations report 1.0."""
        where = self.contiguous(world) if where is None else where
        load = self._load(recent)
        out = np.ones(self.L)
        for l in range(self.L):
            total = load[l].sum()
            if total <= 0:
                continue
            per_rank = np.bincount(where[l], weights=load[l], minlength=world)
            out[l] = per_rank.max() / (total / world)
        return out

    def report(self, world: int = 0, top: int = 4, fold: bool = False) -> Dict[str, Any]:
        """Summary for the info route and logs: observed rows, hottest experts, and for ``world`` ranks the worst and mean
        layer imbalance of the contiguous and of the heat-aware placement.  ``fold``: bring in the device counters first
        (only from the thread that runs the model)."""
        if fold:
            self.fold()
        seen = self.longterm.sum(axis=1)
        layers = [int(l) for l in np.nonzero(seen > 0)[0]]
        out: Dict[str, Any] = {"layers": self.L, "experts": self.E, "observed_layers": len(layers),
                               "routed_rows": float(seen.sum())}
        if layers:
            share = self.longterm[layers] / seen[layers, None]
            out["hottest_share_max"] = float(share.max())
            out["uniform_share"] = 1.0 / self.E
            l0 = layers[0]
            hot = np.argsort(-self.longterm[l0], kind="stable")[:top]
            out["hottest_in_first_layer"] = [(int(e), float(self.longterm[l0, e] / seen[l0])) for e in hot]
        if world > 1 and self.E % world == 0 and layers:
            for name, where in (("contiguous", self.contiguous(world)), ("balanced", self.placement(world))):
                im = self.imbalance(world, where)[layers]
                out[f"imbalance_{name}"] = {"worst": float(im.max()), "mean": float(im.mean())}
        return out


def attach(model, path: Optional[str], half_life: float = 65536.0) -> Optional[ExpertHeat]:
    """Give a mixture-of-experts model a heat profile (loaded from ``path`` when it exists); returns None for dense models.
    Under pipeline parallelism each stage records, and writes back, only its own layers."""
    cfg = model.cfg
    E = int(getattr(cfg, "num_experts", 0) or 0)
    if E <= 0:
        return None
    h = ExpertHeat.open(path, cfg.num_layers, E, model.device)
    h.half_life = half_life
    first, n = getattr(model, "first_layer", 0), len(model.layers)
    if first > 0 or n < cfg.num_layers:
        h.layer_range = (first, first + n)
    model.heat = h
    return h
