#!/usr/bin/env python
"""Headline benchmark: output tokens/s of Qwen3-8B-shape NVFP4 serving (256 concurrent requests, 1024-token prompts,
FP8 paged KV in 16-token pages, greedy decode) on N GPUs of one node with tensor parallelism N.

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus 8 --steps 64 --warmup 8

A timed "step" is one decode iteration over all 256 sequences (one new token each) at context >= 1024; the step is
the engine's real serving step (embedding → 36 layers → lm_head → argmax, KV append included).  `value` is
device-timed with CUDA events (max over ranks).  `e2e` runs the whole workload — prefill of every prompt, then
decoding — through the public API `blaze_b200.LLM.generate`, with each step's inputs staged in pinned host memory
and copied to the device, and each step's tokens read back.  Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

REFERENCE_UNAVAILABLE = ("the reference engine is a Rust workspace (Cargo.toml, no setup.py/pyproject.toml): pip cannot install it "
                         "and no Rust toolchain (cargo/rustc) exists in this image, so its serving step cannot run; its CUDA kernel "
                         "library does build (baseline/build_reference_kernels.sh) and is timed kernel by kernel against this "
                         "library by `python -m blaze_b200.benchmarks.reference_kernels`")


def clocks_sampler(path, gpu_index):
    q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    try:
        return subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "100",
                                 "-i", str(gpu_index)], stdout=open(path, "w"), stderr=subprocess.DEVNULL)
    except OSError:
        return None


def clocks_summary(path):
    sm, mx, reasons = [], 0.0, set()
    try:
        for line in open(path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = max(mx, float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
    except OSError:
        pass
    return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
            "samples": len(sm)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--weights", default="nvfp4")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--e2e-out", type=int, default=0, help="output tokens per request in the end-to-end run (0 = the workload's 256)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the model (marks the line invalid)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--chunk", type=int, default=0,
                    help="prompt tokens per prefill step; 0 = 8192 on one or two GPUs (measured, Qwen3-8B NVFP4, one GPU: 4096 -> "
                         "153 k, 8192 -> 158 k, 16384 -> 153 k prompt tok/s; two GPUs: 19.1 -> 20.5 k tok/s end to end), 4096 on "
                         "more (the size the exchange buffers were measured with there)")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--schedule", default="prefill_first", choices=["interleave", "prefill_first"],
                    help="scheduler policy of the end-to-end run (LLM(schedule=...)): prompts first, or decode rows + one chunk per step")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"], help="TP collectives: in-kernel peer memory, or NCCL")
    ap.add_argument("--ep", action="store_true", help="mixture-of-experts models: whole experts per rank (expert parallel) instead "
                    "of every expert cut over the ranks")
    ap.add_argument("--spec", default=None, choices=["mtp", "eagle", "dflash"],
                    help="speculative-decoding benchmark: a one-layer drafter proposing --draft-k tokens, verify steps through the "
                         "scheduler, acceptance imposed by a seeded pattern (first j of k accepted, j uniform in 0..k), prompts "
                         "sharing --shared-prefix tokens through the prefix cache; exactness against plain decoding is checked")
    ap.add_argument("--draft-k", type=int, default=4)
    ap.add_argument("--shared-prefix", type=int, default=0)
    ap.add_argument("--out-tokens", type=int, default=0, help="output tokens per request of the --spec run (0 = 512)")
    ap.add_argument("--cuda-profiler", nargs="?", const="decode", default=None, choices=["decode", "prefill"],
                    help="bracket the timed decode steps (or the second prefill chunk) with cudaProfilerStart/Stop "
                         "(for ncu --profile-from-start off)")
    args = ap.parse_args()
    if args.chunk <= 0:
        args.chunk = 8192 if args.gpus <= 2 else 4096

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0

    if os.environ.get("BLAZE_BENCH_DEBUG"):
        import faulthandler
        faulthandler.dump_traceback_later(float(os.environ["BLAZE_BENCH_DEBUG"]), repeat=True, file=sys.stderr)

    def note(msg):
        if os.environ.get("BLAZE_BENCH_DEBUG"):
            print(f"[bench r{os.environ.get('RANK', '0')} +{time.time() - T0:.1f}s] {msg}", file=sys.stderr, flush=True)
    T0 = time.time()
    import torch
    from blaze_b200.config import named_config
    from blaze_b200.llm import LLM
    from blaze_b200.models.qwen3 import TPInfo
    from blaze_b200.parallel.tp import TPGroup
    from blaze_b200.sampler import SamplingParams

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    assert torch.cuda.is_available(), "bench.py needs CUDA devices"
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    group = TPGroup.from_env(dev)
    tp = TPInfo(rank, world, group, ep=bool(args.ep and world > 1))
    cfg = named_config(args.model)
    comm = "none"
    if group is not None:
        comm = "nccl"
        if args.comm == "fused":
            try:
                from blaze_b200.parallel.symm import SymmAllReduce
                spec_rows = args.batch * (args.draft_k + 1) if args.spec else 0
                group.fused = SymmAllReduce.create(group, dev, max_rows=max(args.batch, spec_rows) + args.chunk + 64, hidden=cfg.hidden_size)
                comm = "fused peer-memory kernels (" + ("multimem" if group.fused.use_mc else "p2p") + ")"
            except Exception as e:  # the NCCL path stays available
                if rank == 0:
                    print(f"[bench] fused collectives unavailable ({e!r}); using NCCL", file=sys.stderr)

    invalid = None
    if args.layers:
        cfg.num_layers = args.layers
        cfg.layer_types = cfg.layer_types[:args.layers]
        invalid = f"truncated to {args.layers} layers"
    B, P, K, W = args.batch, args.prompt_len, args.steps, args.warmup
    if args.spec:
        return spec_bench(args, cfg, dev, tp, group, comm, rank)
    out_tokens = args.e2e_out or 256
    max_len = P + max(out_tokens, K + W) + 32
    kv_tokens = B * (max_len + 16)
    t_load = time.time()
    llm = LLM(cfg, weight_format=args.weights, device=dev, tp=tp, kv_cache_dtype="fp8", kv_tokens=kv_tokens, max_seqs=B,
              max_model_len=max_len, chunk=args.chunk, enable_prefix_caching=False, use_graphs=not args.no_graphs, seed=1,
              max_step_tokens=B + args.chunk, warm_graphs=not args.no_graphs, schedule=args.schedule)
    note("model built")
    eng = llm.engine
    ops = llm.model.ops
    torch.cuda.synchronize()
    t_load = time.time() - t_load

    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=g).tolist()

    def sync_all():
        if group is not None:
            group.barrier()
        torch.cuda.synchronize()

    # ---------------------------------------------------------------- device-timed decode steps
    seqs = [eng.open_from() for _ in range(B)]
    ttft_ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    sync_all()
    ttft_ev[0].record()
    toks = None
    per = max(1, args.chunk // P)
    last = {}
    for i in range(0, B, per):          # prefill in chunks of ~args.chunk tokens
        part = list(range(i, min(B, i + per)))
        prof_this = args.cuda_profiler == "prefill" and i == per
        if prof_this:
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
        out = eng.forward(eng.plan([(seqs[j], prompts[j], 1) for j in part]), "greedy")
        if prof_this:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        for j, t in zip(part, out.tolist()):
            last[j] = t
    ttft_ev[1].record()
    sync_all()
    note("prefill done")
    prefill_ms = ttft_ev[0].elapsed_time(ttft_ev[1])
    cur = [last[j] for j in range(B)]

    def decode_step(cur):
        out = eng.forward(eng.plan([(seqs[j], [cur[j]], 1) for j in range(B)]), "greedy")
        return out

    # With captured graphs the next step's input tokens are fed back on the device (as the scheduler's run-ahead loop
    # does), so the host's planning of step k+1 overlaps the GPU's step k; every step's tokens are still copied to the host.
    feed = eng.can_feed_back(B)
    host_tok = [torch.empty(B, dtype=torch.int64, pin_memory=True) for _ in range(2)]
    zeros = [0] * B

    host_ev = [None, None]

    def decode_step_fed(k):
        # the host stays at most one step ahead of the GPU, as the scheduler's run-ahead loop does: before step k is
        # issued, the token copy of step k-2 (same pinned buffer) must have landed
        if host_ev[k & 1] is not None:
            host_ev[k & 1].synchronize()
        out = eng.forward(eng.plan([(seqs[j], zeros[j:j + 1], 1) for j in range(B)]), "greedy", feedback=True)
        host_tok[k & 1].copy_(out, non_blocking=True)
        host_ev[k & 1] = torch.cuda.Event()
        host_ev[k & 1].record()
        return out

    for _ in range(max(W, 3)):
        cur = decode_step(cur).tolist()
    note("warmup done")
    l0 = ops.launches
    clk_path = os.path.join(tempfile.gettempdir(), f"blaze_clocks_{rank}.csv")
    sampler = clocks_sampler(clk_path, local) if rank == 0 else None
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.cuda_profiler == "decode":
        torch.cuda.profiler.start()
    e0.record()
    for k in range(K):
        if feed:
            decode_step_fed(k)
        else:
            cur = decode_step(cur).tolist()
    e1.record()
    note("timed steps issued")
    if args.cuda_profiler == "decode":
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    sync_all()
    ms = e0.elapsed_time(e1)
    if sampler is not None:
        time.sleep(0.15)
        sampler.terminate()
    t = torch.tensor([ms], device=dev)
    if group is not None:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms = float(t.item())
    status = ops.take_status()
    for s in seqs:
        eng.close(s)

    # ---------------------------------------------------------------- end to end through the public API
    e2e = None
    if not args.no_e2e:
        eng.h2d_bytes = eng.d2h_bytes = 0
        steps0 = llm.sched.stats.steps
        sync_all()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # With several ranks the public path is the served one: rank 0 schedules (its decisions depend on wall-clock time, so
        # they cannot be re-derived on every rank) and publishes each step, the other ranks replay the steps.
        lead = None
        if group is not None:
            from blaze_b200.parallel.worker import attach, follow
            lead = attach(llm, group)
            sync_all()
        a0.record()
        t_start = time.monotonic()
        if rank == 0:
            outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=out_tokens, ignore_eos=True))
            if lead is not None:
                lead.quit()
        else:
            follow(llm)
            outs = []
        a1.record()
        sync_all()
        ems = a0.elapsed_time(a1)
        t = torch.tensor([ems], device=dev)
        if group is not None:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ems = float(t.item())
        n_out = sum(len(o.token_ids) for o in outs)
        nsteps = max(llm.sched.stats.steps - steps0, 1)
        # per-request latencies on rank 0's host clock (when the request's events reached the caller), not histogram edges
        ttfts = sorted((o.t_first - t_start) * 1e3 for o in outs if o.t_first)
        tpots = sorted((o.t_done - o.t_first) * 1e3 / (len(o.token_ids) - 1) for o in outs
                       if o.t_done and o.t_first and len(o.token_ids) > 1)

        def p50(v):
            return round(v[len(v) // 2], 3) if v else None
        e2e = {"value": n_out / (ems / 1e3), "unit": "output tok/s (prefill + decode, through LLM.generate)",
               "h2d_bytes_per_step": eng.h2d_bytes // nsteps, "d2h_bytes_per_step": eng.d2h_bytes // nsteps,
               "total_ms": ems, "output_tokens": n_out, "steps": nsteps,
               "ttft_p50_ms": p50(ttfts), "tpot_p50_ms": p50(tpots), "latency_clock": "host, rank 0, per request"}
        status = status or ops.take_status()

    if rank == 0:
        value = B * K / (ms / 1e3)
        line = {
            "metric": "output tok/s (device-timed decode steps, max over ranks)", "value": value, "unit": "tok/s",
            "n_gpus": args.gpus, "steps": K, "warmup": max(W, 3), "ms_per_step": ms / K, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": f"{args.weights} weights, fp8 KV, bf16 activations",
            "data": "synthetic token ids, random-init N(0,0.02) weights", "impl": "ours",
            "config": {"model": args.model, "global_batch": B, "seq_len": P, "prefill_chunk": args.chunk, "parallelism": (f"tp{args.gpus} attention + ep{args.gpus} experts" if args.ep and args.gpus > 1 else f"tp{args.gpus}"), "collectives": comm,
                       "kv": "fp8 e4m3, 16-token pages", "l2": "inputs larger than L2 (KV + weights read per step >> 126 MB)",
                       "layers": cfg.num_layers, "schedule": args.schedule, "decode_tokens": "fed back on the device, copied to the host every step" if feed else "read by the host every step"},
            "clocks": clocks_summary(clk_path),
            "e2e": e2e, "gpu_launches": ops.launches - l0 if not eng._graphs else eng.graph_kernel_count() * K,
            "prefill_ms": prefill_ms, "prefill_tok_s": B * P / (prefill_ms / 1e3), "load_s": t_load,
            "device_status": status,
        }
        if invalid:
            line["invalid"] = invalid
        print(json.dumps(line))
    if group is not None:
        # captured graphs hold NCCL work; tearing the process group down under them can block, so leave together instead
        sys.stdout.flush()
        sys.stderr.flush()
        eng._graphs.clear()
        sync_all()
        os._exit(0)
    return 0


def spec_bench(args, cfg, dev, tp, group, comm, rank):
    """``--spec``: BASELINE config 5's shape of run (drafter k tokens, shared prefix, verify-timed, seeded acceptance)."""
    import torch
    from blaze_b200.benchmarks import spec
    from blaze_b200.llm import LLM
    B, P = args.batch, args.prompt_len
    out_tokens = args.out_tokens or 512
    shared = min(args.shared_prefix, P)
    max_len = P + out_tokens + 64
    llm = LLM(cfg, weight_format=args.weights, device=dev, tp=tp, kv_cache_dtype="fp8", kv_tokens=B * (max_len + 16) + shared + 4096,
              max_seqs=B, max_model_len=max_len, chunk=4096, enable_prefix_caching=shared > 0, cache_slots=8, use_graphs=not args.no_graphs,
              seed=4, max_step_tokens=B * (args.draft_k + 1) + 4096, spec_method=args.spec, max_draft=args.draft_k,
              max_verify=args.draft_k + 1, schedule=args.schedule)
    # Decode rows and verify rows must go through the same GEMM kernels here: random-init logits are nearly flat, and sums
    # taken in another order (the small-batch kernel splits K over a cluster) flip near-ties, after which the seeded
    # acceptance pattern (drafts follow the plain stream) no longer describes the speculative stream.
    llm.model.ops.NARROW_ROWS = 0
    g = torch.Generator().manual_seed(4)
    head = torch.randint(0, cfg.vocab_size, (shared,), generator=g).tolist()
    prompts = [head + torch.randint(0, cfg.vocab_size, (P - shared,), generator=g).tolist() for _ in range(B)]

    def sync_all():
        if group is not None:
            group.barrier()
        torch.cuda.synchronize()
    clk_path = os.path.join(tempfile.gettempdir(), f"blaze_clocks_spec_{rank}.csv")
    sampler = clocks_sampler(clk_path, int(os.environ.get("LOCAL_RANK", "0"))) if rank == 0 else None
    # several ranks: rank 0 schedules and drafts (its draft lengths follow measured step times), the others replay its steps
    if group is not None:
        from blaze_b200.parallel.worker import attach, follow
        lead = attach(llm, group)
        sync_all()
        if rank == 0:
            r = spec.run(llm, prompts, out_tokens, args.draft_k, seed=4, sync=torch.cuda.synchronize, shared=shared)
            lead.quit()
        else:
            follow(llm)
            r = {"spec_ms": 0.0, "plain_ms": 0.0}
        sync_all()
    else:
        r = spec.run(llm, prompts, out_tokens, args.draft_k, seed=4, sync=sync_all, shared=shared)
    if sampler is not None:
        time.sleep(0.15)
        sampler.terminate()
    t = torch.tensor([r["spec_ms"], r["plain_ms"]], device=dev)
    if group is not None:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    spec_ms, plain_ms = float(t[0]), float(t[1])
    status = llm.model.ops.take_status()
    if rank == 0:
        line = {"metric": "output tok/s (speculative decoding end to end: prefill + draft + verify, max over ranks)",
                "value": r["output_tokens"] / (spec_ms / 1e3), "unit": "tok/s", "n_gpus": args.gpus, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "impl": "ours", "dtype": f"{args.weights} weights, fp8 KV, bf16 activations",
                "data": "synthetic token ids, random-init N(0,0.02) weights, acceptance imposed by a seeded pattern",
                "config": {"model": args.model, "global_batch": B, "seq_len": P, "shared_prefix": shared, "out_tokens": out_tokens,
                           "parallelism": f"tp{args.gpus}", "collectives": comm, "drafter": args.spec, "draft_k": args.draft_k,
                           "small_batch_gemm": "off (decode and verify rows through the same GEMM kernels)"},
                "plain_tok_s": r["output_tokens"] / (plain_ms / 1e3), "spec_ms": spec_ms, "plain_ms": plain_ms,
                "exact_vs_plain_decoding": r["exact"], "agreement_with_plain_decoding": r["agreement"],
                "agreement_with_draft_continuation": r["agreement_with_continuation"], "speculative_passes": r["passes"], "acceptance": r["acceptance"], "accepted_per_step_hist": r["accepted_per_step_hist"],
                "draft_tokens": r["draft_tokens"], "accepted_tokens": r["accepted_tokens"], "target_steps": r["steps"],
                "cached_prompt_tokens": r["cached_prompt_tokens_spec"], "cached_prompt_tokens_plain": r["cached_prompt_tokens_plain"], "clocks": clocks_summary(clk_path), "device_status": status}
        print(json.dumps(line))
    if group is not None:
        sys.stdout.flush()
        llm.engine._graphs.clear()
        sync_all()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
