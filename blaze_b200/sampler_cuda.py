"""Batched CUDA sampler for rows whose chain is "transforms, then top_k <= 64, then top_p / min_p".

One kernel launch samples every such row of a step (``csrc/kernels/sampling.cu``: mask → penalties / bias → top-64 by
block arg-max → filters on the sorted candidates → inverse-CDF draw → canonical log-probs); the rows come back with one
device→host copy.  Rows with any other chain (no top_k, top_k > 64, top-nσ, top-H, transforms after a filter) keep the
full-sort torch path.  Reference: ``kernels/src/cuda/sampling_pipeline.cu:74-283`` (the "bounded" pipeline,
``sampler.rs:160-172``).
"""
from __future__ import annotations

import ctypes
import struct
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .sampler import MAX_LOGPROBS, SampleResult, SamplingParams, Stage, TOPK_OUT

_ORDER = {Stage.PENALTIES: 0, Stage.LOGIT_BIAS: 1, Stage.TEMPERATURE: 2, Stage.TOP_K: 3, Stage.TOP_P: 4, Stage.MIN_P: 5}
VP = ctypes.c_void_p


def eligible(p: SamplingParams) -> bool:
    """The kernel covers chains that keep the default relative order, have a top_k stage with k <= 64, and put every
    penalty / bias the request carries into the chain (so that the working logits equal the canonical ones)."""
    st = p.active_stages()
    if any(s not in _ORDER for s in st):
        return False
    idx = [_ORDER[s] for s in st]
    if idx != sorted(idx):
        return False
    greedy = Stage.TEMPERATURE in st and p.temperature == 0.0
    if not greedy and (Stage.TOP_K not in st or not (0 < p.top_k <= TOPK_OUT)):
        return False
    if p.has_penalties() and Stage.PENALTIES not in st:
        return False
    if p.logit_bias and Stage.LOGIT_BIAS not in st:
        return False
    return True


class CudaSampler:
    def __init__(self, ops):
        self.ops = ops
        lib = ops.lib
        lib.blz_sample_bounded.restype = ctypes.c_int
        lib.blz_sample_bounded.argtypes = [VP, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, VP, VP, VP, ctypes.c_int,
                                           VP, VP, VP, VP, VP, VP, VP, VP]
        self.lib = lib

    def sample(self, logits: torch.Tensor, rows: Sequence[Tuple[SamplingParams, float, Optional[Dict[int, tuple]], Optional[torch.Tensor]]],
               vocab: int) -> List[SampleResult]:
        """``logits`` fp32 ``[R, >=vocab]`` on the device; ``rows[i] = (params, uniform draw, edits, allowed mask)``."""
        R = len(rows)
        if R == 0:
            return []
        dev = logits.device
        assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[0] >= R
        V = min(vocab, logits.shape[1])
        rec = bytearray()
        ed = bytearray()
        n_ed = 0
        any_mask = any(r[3] is not None for r in rows)
        words = (V + 31) // 32
        mask = torch.full((R, words), -1, dtype=torch.int32) if any_mask else None
        for i, (p, draw, edits, allowed) in enumerate(rows):
            edits = edits or {}
            begin = n_ed
            for tid, (mp, mn, sub, bias, banned) in edits.items():
                ed += struct.pack("<ifffff", int(tid), mp, mn, sub, bias, banned)
                n_ed += 1
            rec += struct.pack("<ffffiiiii", float(p.temperature), float(p.top_p), float(p.min_p), float(draw),
                               int(p.top_k), int(p.execution_mask()), begin, n_ed - begin, 2 if p.logprobs is not None else 1)
            if allowed is not None:
                a = allowed[:V].to(torch.bool).cpu()
                pad = torch.zeros(words * 32, dtype=torch.bool)
                pad[:V] = a
                bits = pad.view(words, 32).to(torch.int64)
                w = (bits << torch.arange(32, dtype=torch.int64)).sum(1)
                w = torch.where(w >= (1 << 31), w - (1 << 32), w)
                mask[i] = w.to(torch.int32)
        rows_d = torch.frombuffer(rec, dtype=torch.uint8).to(dev)
        edits_d = torch.frombuffer(ed, dtype=torch.uint8).to(dev) if n_ed else None
        mask_d = mask.to(dev) if mask is not None else None
        out_tok = torch.empty(R, dtype=torch.int64, device=dev)
        f = torch.empty(R * (2 + TOPK_OUT), dtype=torch.float32, device=dev)
        ids = torch.empty(R * TOPK_OUT + R, dtype=torch.int32, device=dev)
        work = self.ops._buf("sampler_work", R * V * 4).view(torch.float32)
        ptr = lambda t: VP(t.data_ptr()) if t is not None else VP(0)   # noqa: E731
        rc = self.lib.blz_sample_bounded(ptr(logits), logits.stride(0), R, V, ptr(rows_d), ptr(edits_d), ptr(mask_d), words,
                                         ptr(out_tok), VP(f.data_ptr()), VP(f.data_ptr() + R * 4),
                                         VP(f.data_ptr() + 2 * R * 4), VP(ids.data_ptr()), VP(ids.data_ptr() + R * TOPK_OUT * 4),
                                         ptr(work), VP(torch.cuda.current_stream(dev).cuda_stream))
        if rc != 0:
            raise RuntimeError(f"blz_sample_bounded failed: cuda error {rc}")
        self.ops.launches += 1
        tok = out_tok.tolist()
        fh = f.tolist()
        ih = ids.tolist()
        out: List[SampleResult] = []
        for i, (p, _, _, _) in enumerate(rows):
            status = ih[R * TOPK_OUT + i]
            if status != 0:
                out.append(SampleResult(-1, 0.0, [], status))
                continue
            lse = fh[R + i]
            top = []
            for j in range(min(MAX_LOGPROBS, TOPK_OUT)):
                tid = ih[i * TOPK_OUT + j]
                if tid < 0:
                    break
                top.append((tid, fh[2 * R + i * TOPK_OUT + j] - lse))
            out.append(SampleResult(int(tok[i]), fh[i], top, 0))
        return out
