"""HTTP load generator for a running server (any OpenAI-compatible endpoint):

    python -m blaze_b200.benchmarks.client --url http://127.0.0.1:8000 --requests 64 --concurrency 16 \
        --prompt-tokens 1024 --max-tokens 256

Sends streaming ``/v1/completions`` requests with synthetic prompts, ``--concurrency`` at a time, and reports time to
first token, time per output token, end-to-end latency (p50 / p95 / mean) and request / token throughput as one JSON
line.  ``--warm`` first sends every prompt once with ``max_tokens=1`` so that the timed pass hits the prefix cache
("warm"), the default measures a cold pass.  Reference: ``crates/blaze/src/bin/blaze-bench.rs`` (cold / warm passes,
TTFT / TPOT / E2E percentiles, JSON output).
"""
from __future__ import annotations

import argparse
import asyncio
import json
import random
import time
from typing import Dict, List, Optional


def percentile(xs: List[float], q: float) -> float:
    if not xs:
        return 0.0
    s = sorted(xs)
    k = (len(s) - 1) * q
    lo, hi = int(k), min(int(k) + 1, len(s) - 1)
    return s[lo] + (s[hi] - s[lo]) * (k - lo)


def summary(xs: List[float]) -> Dict[str, float]:
    return {"p50": percentile(xs, 0.5), "p95": percentile(xs, 0.95), "mean": sum(xs) / len(xs) if xs else 0.0}


def make_prompt(rng: random.Random, n_tokens: int, shared_prefix: int = 0, prefix_seed: int = 1) -> List[int]:
    """Token-id prompts (the server accepts id lists), optionally with a prefix shared by all requests."""
    pre = random.Random(prefix_seed)
    ids = [pre.randrange(1000, 30000) for _ in range(min(shared_prefix, n_tokens))]
    ids += [rng.randrange(1000, 30000) for _ in range(n_tokens - len(ids))]
    return ids


async def one_request(session, url: str, model: str, prompt: List[int], max_tokens: int, api_key: Optional[str],
                      temperature: float) -> Dict[str, float]:
    body = {"model": model, "prompt": prompt, "max_tokens": max_tokens, "temperature": temperature, "stream": True,
            "ignore_eos": True}
    headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
    t0 = time.perf_counter()
    first = last = None
    n = 0
    async with session.post(url + "/v1/completions", json=body, headers=headers) as resp:
        if resp.status != 200:
            return {"error": resp.status, "detail": (await resp.text())[:200]}
        async for raw in resp.content:
            line = raw.decode("utf-8", "replace").strip()
            if not line.startswith("data:"):
                continue
            data = line[5:].strip()
            if data == "[DONE]":
                break
            try:
                ev = json.loads(data)
            except json.JSONDecodeError:
                continue
            ch = (ev.get("choices") or [{}])[0]
            if ch.get("text") or ch.get("token_ids") or (ch.get("delta") or {}).get("content"):
                now = time.perf_counter()
                first = first or now
                last = now
                n += 1
            usage = ev.get("usage")
            if usage and usage.get("completion_tokens"):
                n = max(n, int(usage["completion_tokens"]))
    t1 = time.perf_counter()
    if first is None:
        return {"error": -1, "detail": "no tokens"}
    return {"ttft": first - t0, "e2e": t1 - t0, "tokens": n, "tpot": (last - first) / max(n - 1, 1)}


async def run_pass(url: str, model: str, prompts: List[List[int]], max_tokens: int, concurrency: int, api_key: Optional[str],
                   temperature: float) -> Dict[str, object]:
    import aiohttp
    sem = asyncio.Semaphore(concurrency)
    results: List[Dict[str, float]] = []
    timeout = aiohttp.ClientTimeout(total=None, sock_read=600)
    async with aiohttp.ClientSession(timeout=timeout) as session:
        async def worker(p):
            async with sem:
                results.append(await one_request(session, url, model, p, max_tokens, api_key, temperature))
        t0 = time.perf_counter()
        await asyncio.gather(*(worker(p) for p in prompts))
        wall = time.perf_counter() - t0
    ok = [r for r in results if "error" not in r]
    out_tokens = sum(int(r["tokens"]) for r in ok)
    return {"requests": len(prompts), "failed": len(results) - len(ok), "wall_s": wall,
            "requests_per_s": len(ok) / wall if wall else 0.0, "output_tok_per_s": out_tokens / wall if wall else 0.0,
            "prompt_tok_per_s": sum(len(p) for p in prompts) / wall if wall else 0.0,
            "ttft_s": summary([r["ttft"] for r in ok]), "tpot_s": summary([r["tpot"] for r in ok]),
            "e2e_s": summary([r["e2e"] for r in ok]),
            "errors": [r for r in results if "error" in r][:3]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="default")
    ap.add_argument("--requests", type=int, default=32)
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--prompt-tokens", type=int, default=512)
    ap.add_argument("--shared-prefix", type=int, default=0, help="leading tokens common to every prompt")
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--warm", action="store_true", help="send every prompt once first (max_tokens=1), then time the warm pass")
    ap.add_argument("--api-key", default=None)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    rng = random.Random(a.seed)
    prompts = [make_prompt(rng, a.prompt_tokens, a.shared_prefix) for _ in range(a.requests)]
    out: Dict[str, object] = {"url": a.url, "concurrency": a.concurrency, "prompt_tokens": a.prompt_tokens, "max_tokens": a.max_tokens}
    if a.warm:
        out["cold_fill"] = asyncio.run(run_pass(a.url, a.model, prompts, 1, a.concurrency, a.api_key, a.temperature))
    out["warm" if a.warm else "cold"] = asyncio.run(run_pass(a.url, a.model, prompts, a.max_tokens, a.concurrency, a.api_key,
                                                                 a.temperature))
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
