"""Sampler chain on torch tensors (any device): one row at a time with the full stage semantics, and a
batched path for rows that share the default stage order.

Same semantics as :func:`blaze_b200.sampler.sample_reference` (the fp64 oracle) but in fp32 on the logits'
device; this is the functional path behind the CUDA sampler kernels and what CPU runs use.
Reference: ``kernels/src/cuda/sampling_pipeline.cu:74-283``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

from .sampler import MAX_LOGPROBS, SampleResult, SamplingParams, Stage


def _edits_tensors(edits: Dict[int, tuple], V: int, device):
    ids = torch.tensor([i for i in edits if i < V], dtype=torch.long, device=device)
    vals = torch.tensor([edits[int(i)] for i in ids.tolist()], dtype=torch.float32, device=device).view(-1, 5)
    return ids, vals


def _penalties(x: torch.Tensor, ids, vals) -> None:
    if ids.numel() == 0:
        return
    v = x[ids]
    v = torch.where(v > 0, v * vals[:, 0], v * vals[:, 1]) - vals[:, 2]
    v = torch.where(vals[:, 4] > 0, torch.full_like(v, -math.inf), v)
    x[ids] = v


def _bias(x: torch.Tensor, ids, vals) -> None:
    if ids.numel():
        x[ids] = x[ids] + vals[:, 3]


def sample_row(logits: torch.Tensor, params: SamplingParams, draw: float, edits=None,
               allowed: Optional[torch.Tensor] = None, vocab: Optional[int] = None) -> SampleResult:
    x = logits.detach().float().clone()
    V = x.numel()
    dev = x.device
    ok = torch.ones(V, dtype=torch.bool, device=dev)
    if vocab is not None and vocab < V:
        ok[vocab:] = False
    if allowed is not None:
        ok &= allowed.to(dev).bool()
    xa = x[ok]
    if xa.numel() == 0:
        return SampleResult(-1, 0.0, [], -1)
    if torch.isnan(xa).any() or (xa == math.inf).any():
        return SampleResult(-1, 0.0, [], -2)
    x = torch.where(ok, x, torch.full_like(x, -math.inf))
    ids, vals = _edits_tensors(edits or {}, V, dev)
    canon = x.clone()
    _penalties(canon, ids, vals)
    _bias(canon, ids, vals)
    alive = torch.isfinite(x)
    for st in params.active_stages():
        if st == Stage.PENALTIES:
            _penalties(x, ids, vals)
            alive &= torch.isfinite(x)
        elif st == Stage.LOGIT_BIAS:
            _bias(x, ids, vals)
        elif st == Stage.TEMPERATURE:
            if params.temperature == 0.0:
                xm = torch.where(alive, x, torch.full_like(x, -math.inf))
                m = xm.max()
                best = int(torch.nonzero(xm == m)[0])
                alive = torch.zeros_like(alive)
                alive[best] = True
            else:
                x = x / params.temperature
        else:
            xm = torch.where(alive, x, torch.full_like(x, -math.inf))
            n_alive = int(alive.sum())
            vals_s, order = torch.sort(xm, descending=True, stable=True)
            vals_s, order = vals_s[:n_alive], order[:n_alive]
            keep = n_alive
            if st == Stage.TOP_K:
                keep = min(params.top_k, n_alive)
            elif st == Stage.TOP_P:
                p = torch.softmax(vals_s.double(), 0)
                c = torch.cumsum(p, 0)
                keep = int((c < params.top_p * c[-1]).sum()) + 1
            elif st == Stage.MIN_P:
                p = torch.softmax(vals_s.double(), 0)
                keep = int((p / p[0] >= params.min_p).sum())
            elif st == Stage.TOP_NSIGMA:
                sigma = vals_s.double().std(unbiased=False) if n_alive > 1 else torch.zeros((), dtype=torch.float64, device=dev)
                keep = int((vals_s.double() >= vals_s[0].double() - params.top_nsigma * sigma).sum())
            elif st == Stage.TOP_H:
                p = torch.softmax(vals_s.double(), 0)
                plogp = p * torch.log(p.clamp_min(1e-300))
                H = float(-plogp.sum())
                cs = torch.cumsum(p, 0)
                cpl = torch.cumsum(plogp, 0)
                # entropy of the renormalised prefix j: log(cs_j) - cpl_j / cs_j
                hj = torch.log(cs) - cpl / cs
                good = hj <= params.top_h * H + 1e-12
                bad = torch.nonzero(~good)
                keep = int(bad[0]) if bad.numel() else n_alive
            keep = max(1, min(keep, n_alive))
            alive = torch.zeros_like(alive)
            alive[order[:keep]] = True
    xm = torch.where(alive, x, torch.full_like(x, -math.inf))
    n_alive = int(alive.sum())
    vals_s, order = torch.sort(xm, descending=True, stable=True)
    vals_s, order = vals_s[:n_alive], order[:n_alive]
    p = torch.softmax(vals_s.double(), 0)
    c = torch.cumsum(p, 0)
    pick = min(int((c < draw * c[-1]).sum()), n_alive - 1)
    tok = int(order[pick])
    lp, top = 0.0, []
    if params.logprobs is not None:
        lse = torch.logsumexp(canon[torch.isfinite(canon)].double(), 0)
        tv, ti = torch.topk(canon, min(MAX_LOGPROBS, V))
        top = [(int(i), float(v.double() - lse)) for v, i in zip(tv, ti) if math.isfinite(float(v))]
        lp = float(canon[tok].double() - lse)
    return SampleResult(tok, lp, top, 0)


def sample_batch_default(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                         min_p: torch.Tensor, draws: torch.Tensor) -> torch.Tensor:
    """Rows that all use the default order temperature → top_k → top_p → min_p with no edits, sampled together.

    ``temperature == 0`` rows return the lowest-index argmax.  All parameter tensors are ``[R]`` on the logits'
    device; returns int64 token ids ``[R]``.
    """
    x = logits.float()
    R, V = x.shape
    greedy = temperature == 0
    t = torch.where(greedy, torch.ones_like(temperature), temperature).view(R, 1)
    vals, order = torch.sort(x / t, dim=1, descending=True, stable=True)
    rank = torch.arange(V, device=x.device).view(1, V)
    k = torch.where(top_k <= 0, torch.full_like(top_k, V), top_k).view(R, 1)
    keep = rank < k
    p = torch.softmax(vals.masked_fill(~keep, -math.inf).double(), 1)
    c = torch.cumsum(p, 1)
    keep &= (c - p) < top_p.view(R, 1).double() * c[:, -1:]
    p = torch.softmax(vals.masked_fill(~keep, -math.inf).double(), 1)
    keep &= (p / p[:, :1]) >= min_p.view(R, 1).double()
    keep[:, 0] = True
    p = torch.softmax(vals.masked_fill(~keep, -math.inf).double(), 1)
    c = torch.cumsum(p, 1)
    pick = (c < draws.view(R, 1).double() * c[:, -1:]).sum(1).clamp(max=V - 1)
    last = keep.sum(1) - 1
    pick = torch.minimum(pick, last)
    tok = order.gather(1, pick.view(R, 1)).squeeze(1)
    m = x.max(dim=1, keepdim=True).values
    idx = torch.arange(V, device=x.device).expand(R, V)
    arg = torch.where(x == m, idx, torch.full_like(idx, V)).min(1).values
    return torch.where(greedy, arg, tok)
