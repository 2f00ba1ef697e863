"""Batched CUDA sampler against the fp64 oracle of the stage chain."""
import math

import pytest
import torch

from blaze_b200.sampler import Rng, SamplingParams, penalty_edits, sample_reference
from blaze_b200.sampler_cuda import CudaSampler, eligible

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def sampler():
    from blaze_b200.ops import get_ops
    return CudaSampler(get_ops("cuda"))


def test_sampler_matches_oracle(sampler):
    g = torch.Generator(device=DEV).manual_seed(31)
    V, Vpad = 5003, 5120
    cases = [
        SamplingParams(temperature=0.8, top_k=40, top_p=0.9, min_p=0.02, logprobs=5),
        SamplingParams(temperature=1.3, top_k=64),
        SamplingParams(temperature=0.0, logprobs=3, repetition_penalty=1.3),
        SamplingParams(temperature=0.7, top_k=8, presence_penalty=0.5, frequency_penalty=0.2, logit_bias={17: 4.0, 99: -3.0}),
        SamplingParams(temperature=1.0, top_k=5, min_tokens=4),
        SamplingParams(temperature=0.9, top_k=20, top_p=0.5),
        SamplingParams(temperature=0.6, top_k=3, min_p=0.4, logprobs=20),
    ] * 3
    R = len(cases)
    logits = torch.randn(R, Vpad, generator=g, device=DEV) * 3.0
    rows, want = [], []
    for i, p in enumerate(cases):
        rng = Rng(100 + i)
        draw = rng.uniform()
        prompt = torch.randint(0, V, (30,), generator=torch.Generator().manual_seed(i)).tolist()
        gen = prompt[:3]
        edits = penalty_edits(p, prompt, gen, eos_ids=(2,)) if (p.has_penalties() or p.logit_bias) else {}
        allowed = None
        if i % 5 == 4:
            allowed = torch.rand(V, generator=torch.Generator().manual_seed(50 + i)) < 0.7
        rows.append((p, draw, edits, allowed))
        want.append(sample_reference(logits[i, :V].cpu(), p, draw, edits, allowed, V))
    got = sampler.sample(logits, rows, V)
    torch.cuda.synchronize()
    for i, (g_, w_) in enumerate(zip(got, want)):
        assert g_.status == 0 and w_.status == 0
        assert g_.token == w_.token, f"row {i}: {cases[i]}"
        assert abs(g_.logprob - w_.logprob) < 2e-3
        n = cases[i].logprobs or 0
        assert [t for t, _ in g_.top[:n]] == [t for t, _ in w_.top[:n]]
        for (_, a), (_, b) in zip(g_.top[:n], w_.top[:n]):
            assert abs(a - b) < 2e-3


def test_sampler_status_codes(sampler):
    V = 1000
    logits = torch.randn(3, V, device=DEV)
    logits[1, 5] = float("nan")
    p = SamplingParams(temperature=0.5, top_k=10)
    none_allowed = torch.zeros(V, dtype=torch.bool)
    got = sampler.sample(logits, [(p, 0.3, {}, None), (p, 0.3, {}, None), (p, 0.3, {}, none_allowed)], V)
    assert got[0].status == 0 and 0 <= got[0].token < V
    assert got[1].status == -2
    assert got[2].status == -1
