"""Speculative-decoding benchmark: a drafter proposing ``k`` tokens per step, verify steps through the product path, a shared
prompt prefix served from the prefix cache, and a seeded synthetic acceptance pattern.

A random-init drafter next to a random-init target is almost never right, so acceptance is imposed: the benchmark first
decodes every request without speculation (which is also the exactness oracle), then runs the speculative pass with a
wrapper around the real drafter that still runs it (its cost is paid) but replaces its proposals by the known continuation for
the first ``j`` positions and by wrong tokens after them, ``j`` uniform in ``0..k`` from a seeded generator.  Every emitted
stream must equal the non-speculative one.

The reference's counterpart is ``scripts/spec_bench.py`` driving ``--spec-method mtp`` (``crates/blaze/src/main.rs:933-947``,
acceptance statistics ``sched.rs:235``).
"""
from __future__ import annotations

import random
import time
from typing import Dict, List, Sequence


class SyntheticAcceptance:
    """Wraps a drafter: same hooks, same cost, proposals rewritten so that exactly the first ``j`` of them are accepted."""

    def __init__(self, inner, streams: Dict[str, List[int]], vocab: int, seed: int = 4):
        self.inner, self.streams, self.vocab = inner, streams, vocab
        self.rng = random.Random(seed)
        self.kind = getattr(inner, "kind", "mtp")
        self.hist = [0] * 17

    def __getattr__(self, name):
        return getattr(self.inner, name)

    def propose(self, actives, ks: Sequence[int]):
        real = self.inner.propose(actives, ks)
        out = []
        for a, k, r in zip(actives, ks, real):
            if k <= 0:
                out.append([])
                continue
            full = self.streams.get(a.req.request_id)
            done = len(a.tokens) - a.n_prompt                       # tokens already emitted
            j = self.rng.randint(0, k)
            self.hist[j] += 1
            d = []
            for i in range(k):
                nxt = full[done + i] if (full is not None and done + i < len(full)) else 0
                d.append(nxt if i < j else (nxt + 1) % self.vocab)
            out.append(d)
        return out


def run(llm, prompts: List[List[int]], out_tokens: int, k: int, seed: int = 4, sync=None, shared: int = 0,
        max_passes: int = 3) -> dict:
    """Plain pass (oracle + timing), then the speculative pass with imposed acceptance; returns timings and statistics.

    ``shared``: the first ``shared`` tokens are common to every prompt (a system prompt).  Before each timed pass the prefix
    cache is emptied and one untimed request leaves the shared head in it, as earlier traffic would have; every timed request
    names the head as its cache point, so both passes prefill only what follows it."""
    import torch
    from ..sampler import SamplingParams
    from ..sched import GenRequest
    sp = SamplingParams(temperature=0.0, max_tokens=out_tokens, ignore_eos=True)
    sched = llm.sched
    drafter, sched.drafter = sched.drafter, None
    method, sched.cfg.spec_method = sched.cfg.spec_method, "none"

    def warm():
        sched.cache.clear()
        if shared <= 0:
            return
        one = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
        sched.submit(GenRequest("warm", list(prompts[0][:shared]) + [prompts[0][0]], one, cache_point=shared))
        sched.run_until_idle()

    def timed(tag):
        outs: Dict[str, List[int]] = {}
        warm()
        if sync:
            sync()
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cuda = llm.device.type == "cuda"
        if cuda:
            e0.record()
        for i, p in enumerate(prompts):
            rid = f"{tag}-{i}"
            outs[rid] = []
            sched.submit(GenRequest(rid, list(p), sp, cache_point=shared or None,
                                    sink=lambda ev, rid=rid: outs[rid].extend(ev.tokens or [])))
        sched.run_until_idle()
        if cuda:
            e1.record()
        if sync:
            sync()
        ms = e0.elapsed_time(e1) if cuda else (time.perf_counter() - t0) * 1e3
        return outs, ms
    cached0 = sched.stats.cached_tokens
    plain, plain_ms = timed("plain")
    cached_plain = sched.stats.cached_tokens - cached0
    sched.drafter, sched.cfg.spec_method = None, "none"          # (the warm-up of the second pass runs without the drafter too)
    real_warm = warm

    def agreement(x: Dict[str, List[int]], xt: str, y: Dict[str, List[int]], yt: str) -> float:
        """Share of emitted tokens before a stream's first difference from the other run's stream (1.0 when equal)."""
        same = total = 0
        for i in range(len(prompts)):
            u, v = x[f"{xt}-{i}"], y[f"{yt}-{i}"]
            n = 0
            while n < min(len(u), len(v)) and u[n] == v[n]:
                n += 1
            same += n
            total += max(len(v), 1)
        return same / max(total, 1)

    # The drafts follow a known continuation.  The first speculative pass takes the plain pass's streams.  On a GPU the
    # verify rows and the decode rows go through different kernels and split the KV range differently, so near-ties of
    # random-init logits flip and the speculative stream leaves the plain one early; the imposed pattern then no longer
    # describes it.  Verify steps, however, reproduce verify steps (every step has the same shape), so the pass is repeated
    # with the previous speculative pass's own streams as the continuation until the two agree (at most `max_passes` times).
    # Every pass is a full, really verified run; the last one is reported.
    oracle, otag = plain, "plain"
    passes = 0
    while True:
        tag = f"spec{passes}"
        streams = {f"{tag}-{i}": oracle[f"{otag}-{i}"] for i in range(len(prompts))}
        wrapped = SyntheticAcceptance(drafter, streams, llm.model.cfg.vocab_size, seed)

        def warm():                                    # noqa: F811  the drafter goes in after the untimed warm-up request
            sched.drafter, sched.cfg.spec_method = None, "none"
            real_warm()
            sched.drafter, sched.cfg.spec_method, sched.cfg.max_draft = wrapped, method, k
        d0, a0, s0 = sched.stats.draft_tokens, sched.stats.accepted_tokens, sched.stats.steps
        cached1 = sched.stats.cached_tokens
        spec, spec_ms = timed(tag)
        passes += 1
        agree_oracle = agreement(spec, tag, oracle, otag)
        if agree_oracle >= 0.9 or passes >= max_passes:
            break
        oracle, otag = spec, tag
    stag = tag
    exact = all(spec[f"{stag}-{i}"] == plain[f"plain-{i}"] for i in range(len(prompts)))
    agree_plain = agreement(spec, stag, plain, "plain")
    n_out = sum(len(v) for v in spec.values())
    drafted, accepted = sched.stats.draft_tokens - d0, sched.stats.accepted_tokens - a0
    return {"plain_ms": plain_ms, "spec_ms": spec_ms, "output_tokens": n_out, "exact": exact,
            "plain_tok_s": n_out / (plain_ms / 1e3), "spec_tok_s": n_out / (spec_ms / 1e3),
            "draft_tokens": drafted, "accepted_tokens": accepted, "acceptance": accepted / max(drafted, 1),
            "accepted_per_step_hist": wrapped.hist[:k + 1], "steps": sched.stats.steps - s0, "agreement": agree_plain,
            "agreement_with_continuation": agree_oracle, "passes": passes,
            "cached_prompt_tokens_plain": cached_plain, "cached_prompt_tokens_spec": sched.stats.cached_tokens - cached1}
