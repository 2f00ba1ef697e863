"""Ordered sampler chain: parameters, the row program, the host RNG and the fp64 reference distribution.

Semantics follow the reference (``crates/blaze/src/sampler.rs:8-216`` and
``kernels/src/cuda/sampling_pipeline.cu:74-283``): stages penalties=1, logit_bias=2, temperature=3,
top_k=4, top_p=5, min_p=6, top_nsigma=7, top_h=8 run in the order the request gives; inactive stages
are dropped; temperature 0 keeps exactly one token *at that position of the chain*; filters act on
the descending sort with lower id first among equals; the draw is an inverse-CDF pick with a
host-supplied uniform number from xorshift64*; log-probs come from a canonical copy that received
penalties then bias whatever the stage order.
"""
from __future__ import annotations

import enum
import json
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

TOPK_OUT = 64          # (logit, id) pairs exported per row
MAX_LOGPROBS = 20


class Stage(enum.IntEnum):
    PENALTIES = 1
    LOGIT_BIAS = 2
    TEMPERATURE = 3
    TOP_K = 4
    TOP_P = 5
    MIN_P = 6
    TOP_NSIGMA = 7
    TOP_H = 8


_NAMES = {"penalties": Stage.PENALTIES, "logit_bias": Stage.LOGIT_BIAS, "temperature": Stage.TEMPERATURE,
          "top_k": Stage.TOP_K, "top_p": Stage.TOP_P, "min_p": Stage.MIN_P, "top_nsigma": Stage.TOP_NSIGMA,
          "top_n_sigma": Stage.TOP_NSIGMA, "top_h": Stage.TOP_H}
DEFAULT_PIPELINE = (Stage.PENALTIES, Stage.LOGIT_BIAS, Stage.TEMPERATURE, Stage.TOP_K, Stage.TOP_P, Stage.MIN_P)


def parse_pipeline(spec) -> Tuple[Stage, ...]:
    """Accept a JSON array, a python list or a comma list of stage names; at most 8, no duplicates."""
    if spec is None:
        return DEFAULT_PIPELINE
    if isinstance(spec, str):
        s = spec.strip()
        items = json.loads(s) if s.startswith("[") else [x for x in (p.strip() for p in s.split(",")) if x]
    else:
        items = list(spec)
    out: List[Stage] = []
    for it in items:
        key = str(it).strip().lower()
        if key not in _NAMES:
            raise ValueError(f"unknown sampler stage {it!r}")
        st = _NAMES[key]
        if st in out:
            raise ValueError(f"sampler stage {key} listed twice")
        out.append(st)
    if len(out) > 8:
        raise ValueError("at most 8 sampler stages")
    return tuple(out)


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    top_nsigma: float = 1.0
    top_h: float = 0.4
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    logit_bias: Dict[int, float] = field(default_factory=dict)
    pipeline: Tuple[Stage, ...] = DEFAULT_PIPELINE
    seed: Optional[int] = None
    max_tokens: int = 16
    min_tokens: int = 0
    stop_token_ids: Tuple[int, ...] = ()
    bad_words: Tuple[Tuple[int, ...], ...] = ()
    ignore_eos: bool = False
    logprobs: Optional[int] = None          # number of alternatives wanted (None = no logprobs)
    n: int = 1

    def active_stages(self) -> Tuple[Stage, ...]:
        """The row program: stages that can change the outcome (``sampler.rs:150-160``)."""
        out = []
        for st in self.pipeline:
            if st == Stage.PENALTIES and not self.has_penalties():
                continue
            if st == Stage.LOGIT_BIAS and not self.logit_bias:
                continue
            if st == Stage.TEMPERATURE and self.temperature == 1.0:
                continue
            if st == Stage.TOP_K and self.top_k <= 0:
                continue
            if st == Stage.TOP_P and self.top_p >= 1.0:
                continue
            if st == Stage.MIN_P and self.min_p <= 0.0:
                continue
            if st == Stage.TOP_H and self.top_h >= 1.0:
                continue
            out.append(st)
        return tuple(out)

    def has_penalties(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0
                or bool(self.bad_words) or self.min_tokens > 0)

    def is_greedy(self) -> bool:
        """Temperature stage with T=0, or a top_k stage with k=1 (``sampler.rs:174-176``)."""
        st = self.pipeline
        return (Stage.TEMPERATURE in st and self.temperature == 0.0) or (Stage.TOP_K in st and self.top_k == 1)

    def needs_candidates(self) -> bool:
        """False → plain sharded argmax is enough (``sampler.rs:177-187``)."""
        if not self.is_greedy():
            return True
        if self.logprobs is not None or self.logit_bias or self.has_penalties():
            return True
        return self.pipeline != DEFAULT_PIPELINE

    def execution_mask(self) -> int:
        m = 0
        for i, st in enumerate(self.active_stages()):
            m |= int(st) << (4 * i)
        return m

    def bounded(self) -> bool:
        """True when the first active filter is top_k <= 64: a radix top-64 replaces the full sort."""
        for st in self.active_stages():
            if st in (Stage.TOP_P, Stage.MIN_P, Stage.TOP_NSIGMA, Stage.TOP_H):
                return False
            if st == Stage.TOP_K:
                return self.top_k <= TOPK_OUT
        return False


# ------------------------------------------------------------------------------------- RNG
_M64 = (1 << 64) - 1


class Rng:
    """xorshift64* seeded by ``seed * 0x9E3779B97F4A7C15 | 1``; 24-bit uniform draws (``sampler.rs:191-214``)."""

    def __init__(self, seed: int):
        self.state = ((seed * 0x9E3779B97F4A7C15) & _M64) | 1

    def next_u64(self) -> int:
        x = self.state
        x ^= x >> 12
        x ^= (x << 25) & _M64
        x ^= x >> 27
        self.state = x
        return (x * 0x2545F4914F6CDD1D) & _M64

    def uniform(self) -> float:
        return (self.next_u64() >> 40) / float(1 << 24)

    def lookahead(self, depth: int) -> float:
        """The draw that will be made ``depth`` steps from now, without consuming state (draft rows)."""
        saved = self.state
        u = 0.0
        for _ in range(depth + 1):
            u = self.uniform()
        self.state = saved
        return u


# ------------------------------------------------------------------------------------- logit edits
def penalty_edits(params: SamplingParams, prompt: Sequence[int], generated: Sequence[int], eos_ids: Sequence[int],
                  draft_prefix: Sequence[int] = ()) -> Dict[int, Tuple[float, float, float, float, float]]:
    """Per-token-id edits ``(mul if x>0, mul if x<=0, subtract, bias, banned)`` (``sched.rs:2490-2530``)."""
    edits: Dict[int, List[float]] = {}

    def e(t):
        return edits.setdefault(int(t), [1.0, 1.0, 0.0, 0.0, 0.0])

    gen = list(generated) + list(draft_prefix)
    if params.repetition_penalty != 1.0:
        r = params.repetition_penalty
        for t in set(prompt) | set(gen):
            x = e(t)
            x[0], x[1] = 1.0 / r, r
    if params.presence_penalty != 0.0 or params.frequency_penalty != 0.0:
        counts: Dict[int, int] = {}
        for t in gen:
            counts[t] = counts.get(t, 0) + 1
        for t, c in counts.items():
            e(t)[2] += params.presence_penalty + params.frequency_penalty * c
    for t, b in params.logit_bias.items():
        e(t)[3] += float(b)
    if len(gen) < params.min_tokens:
        for t in list(eos_ids) + list(params.stop_token_ids):
            e(t)[4] = 1.0
    for bw in params.bad_words:
        if not bw:
            continue
        pre = list(bw[:-1])
        if not pre or (len(gen) >= len(pre) and gen[-len(pre):] == pre):
            e(bw[-1])[4] = 1.0
    return {k: tuple(v) for k, v in edits.items()}


# ------------------------------------------------------------------------------------- reference pipeline
@dataclass
class SampleResult:
    token: int
    logprob: float                       # canonical log-prob of the chosen token
    top: List[Tuple[int, float]]         # canonical (id, logprob) alternatives, descending
    status: int = 0                      # 0 ok, -1 empty support, -2 non-finite logit on an allowed token


def _apply_edits(x: torch.Tensor, edits, what: str) -> None:
    for tid, (mp, mn, sub, bias, banned) in edits.items():
        if tid >= x.numel():
            continue
        v = x[tid].item()
        if what == "penalties":
            if banned:
                x[tid] = -math.inf
                continue
            v = v * mp if v > 0 else v * mn
            x[tid] = v - sub
        else:
            x[tid] = v + bias


def sample_reference(logits: torch.Tensor, params: SamplingParams, draw: float, edits=None,
                     allowed: Optional[torch.Tensor] = None, vocab: Optional[int] = None) -> SampleResult:
    """fp64 reference of one row (the oracle of the CUDA sampler; ``sampler.rs:223`` ``distribution``)."""
    x = logits.detach().double().cpu().clone()
    V = x.numel()
    edits = edits or {}
    ok = torch.ones(V, dtype=torch.bool)
    if vocab is not None:
        ok[vocab:] = False
    if allowed is not None:
        ok &= allowed.cpu().bool()
    if not torch.isfinite(x[ok]).all() and (torch.isnan(x[ok]).any() or (x[ok] == math.inf).any()):
        return SampleResult(-1, 0.0, [], -2)
    x[~ok] = -math.inf
    if not ok.any():
        return SampleResult(-1, 0.0, [], -1)
    canon = x.clone()
    _apply_edits(canon, edits, "penalties")
    _apply_edits(canon, edits, "bias")
    alive = torch.isfinite(x)
    for st in params.active_stages():
        if st == Stage.PENALTIES:
            _apply_edits(x, edits, "penalties")
            alive &= torch.isfinite(x)
        elif st == Stage.LOGIT_BIAS:
            _apply_edits(x, edits, "bias")
        elif st == Stage.TEMPERATURE:
            if params.temperature == 0.0:
                xm = torch.where(alive, x, torch.full_like(x, -math.inf))
                best = int(torch.argmax(xm))          # first maximum = lowest id
                alive = torch.zeros_like(alive)
                alive[best] = True
            else:
                x = x / params.temperature
        else:
            xm = torch.where(alive, x, torch.full_like(x, -math.inf))
            order = torch.argsort(-xm, stable=True)
            n_alive = int(alive.sum())
            order = order[:n_alive]
            vals = xm[order]
            keep = n_alive
            if st == Stage.TOP_K:
                keep = min(params.top_k, n_alive)
            elif st == Stage.TOP_P:
                p = torch.softmax(vals, 0)
                c = torch.cumsum(p, 0)
                keep = int((c < params.top_p * c[-1]).sum()) + 1
            elif st == Stage.MIN_P:
                p = torch.softmax(vals, 0)
                keep = int((p / p[0] >= params.min_p).sum())
            elif st == Stage.TOP_NSIGMA:
                sigma = vals.std(unbiased=False) if n_alive > 1 else torch.tensor(0.0, dtype=torch.float64)
                keep = int((vals >= vals[0] - params.top_nsigma * sigma).sum())
            elif st == Stage.TOP_H:
                p = torch.softmax(vals, 0)
                H = float(-(p * torch.log(p.clamp_min(1e-300))).sum())
                keep = 1
                for j in range(1, n_alive + 1):
                    pj = p[:j] / p[:j].sum()
                    hj = float(-(pj * torch.log(pj.clamp_min(1e-300))).sum())
                    if hj <= params.top_h * H + 1e-12:
                        keep = j
                    else:
                        break
            keep = max(1, min(keep, n_alive))
            alive = torch.zeros_like(alive)
            alive[order[:keep]] = True
    xm = torch.where(alive, x, torch.full_like(x, -math.inf))
    order = torch.argsort(-xm, stable=True)[:int(alive.sum())]
    p = torch.softmax(xm[order], 0)
    c = torch.cumsum(p, 0)
    pick = int((c < draw * c[-1]).sum())
    pick = min(pick, order.numel() - 1)
    tok = int(order[pick])
    lse = torch.logsumexp(canon[torch.isfinite(canon)], 0)
    top_n = min(MAX_LOGPROBS, V)
    tv, ti = torch.topk(canon, top_n)
    top = [(int(i), float(v - lse)) for v, i in zip(tv, ti) if math.isfinite(float(v))]
    return SampleResult(tok, float(canon[tok] - lse), top, 0)
