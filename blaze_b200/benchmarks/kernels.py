"""Kernel micro-benchmarks (device-timed with CUDA events, L2 flushed between iterations).

    python -m blaze_b200.benchmarks.kernels attention --batch 256 --ctx 1024 --hq 32 --hkv 8
    python -m blaze_b200.benchmarks.kernels gemm --kind nvfp4 --m 256 --n 24576 --k 4096
    python -m blaze_b200.benchmarks.kernels norm --rows 256 --hidden 4096

Each prints one JSON line with the achieved bandwidth / FLOP rate and its fraction of the measured peaks in
``MEASURED_PEAKS.json`` when that file is present.  Plays the role of the reference's manual kernel benches
(``kernels/tests/bench_attn_prefill.cu``, ``bench_mma_peak.cu``, ``kernels/tools/membw.cpp``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "src": "fallback"}


def timeit(fn, iters: int, warmup: int = 3, flush: bool = True):
    scratch = torch.empty(192 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            scratch.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2], times[0]


def bench_attention(a):
    from ..batch import SeqChunk, build_batch
    from ..config import ModelConfig, RopeConfig
    from ..kv import KVCache
    from ..ops import get_ops
    ops = get_ops("cuda")
    D = 128
    cfg = ModelConfig(hidden_size=a.hq * D, num_heads=a.hq, num_kv_heads=a.hkv, head_dim=D, num_layers=1, rope=RopeConfig(theta=1e6))
    cfg.layer_types = ["full_attention"]
    B = a.batch
    pages_per = (a.ctx + 15) // 16 + 1
    kv = KVCache(cfg, 1 + B * pages_per, B, pages_per, "fp8", "cuda", "umma")
    perm = torch.randperm(B * pages_per).tolist()
    for b in range(B):
        kv.set_pages(b, [1 + p for p in perm[b * pages_per:(b + 1) * pages_per]])
    kv.kv[0].copy_(torch.randint(0, 120, kv.kv[0].shape, dtype=torch.uint8, device="cuda"))   # finite e4m3 codes
    tpb = 128 // (a.hq // a.hkv)
    chunks = [SeqChunk(b, [0] * a.qlen, a.ctx - a.qlen) for b in range(B)]
    batch = build_batch(chunks, kv.block_table_host, "cuda", attn_group=a.hq // a.hkv)
    q = torch.randn(B * a.qlen, a.hq, D, device="cuda").bfloat16()

    class M:
        pass
    fn = lambda: ops.attention(q, M, batch, kv, 0, D ** -0.5, splits=a.splits)  # noqa: E731
    med, best = timeit(fn, a.iters)
    if a.prof:
        ops.attn_prof = torch.zeros(8 * 3 * 16, dtype=torch.int64, device="cuda")
        fn()
        torch.cuda.synchronize()
        names = ["kv_empty", "k_full", "s_empty", "v_full", "p_full", "o_empty", "q_full", "s_full", "wm_bar", "o_full",
                 "q_empty", "fin", "total"]
        pr = ops.attn_prof.view(8, 3, 16).cpu()
        for blk in range(2):
            for w, role in enumerate(["loader", "mma", "softmax"]):
                print(f"[prof] block {blk} {role}: " + " ".join(f"{n}={int(pr[blk, w, i])}" for i, n in enumerate(names) if int(pr[blk, w, i])),
                      file=sys.stderr)
        ops.attn_prof = None
    causal = 1.0 if a.qlen == 1 else (a.ctx - a.qlen / 2) / a.ctx
    kv_bytes = B * a.ctx * a.hkv * 2 * D * (1.0 if a.qlen <= tpb else 1.0)
    flops = 4.0 * B * a.qlen * a.hq * a.ctx * causal * D
    pk = peaks()
    print(json.dumps({"kernel": "attn_tc", "batch": B, "ctx": a.ctx, "qlen": a.qlen, "hq": a.hq, "hkv": a.hkv,
                      "ms_median": med, "ms_best": best, "kv_gbs": kv_bytes / med / 1e6,
                      "frac_hbm_" + pk["src"]: kv_bytes / med / 1e6 / pk["hbm_gbs"], "tflops": flops / med / 1e9,
                      "status": ops.take_status()}))


def bench_gemm(a):
    """Times the GEMM inside a captured graph of ``copies`` calls, each on its own weight tensor (together larger than L2):
    a single small launch timed from the host measures the host, not the kernel."""
    from ..linear import Linear
    from ..ops import get_ops
    from ..quant import Format
    ops = get_ops("cuda")
    fmt = {"bf16": Format.DENSE, "nvfp4": Format.NVFP4, "mxfp8": Format.MXFP8, "fp8": Format.FP8_CHANNEL,
           "fp8_block": Format.FP8_BLOCK, "fp8_block_mx": Format.FP8_BLOCK}[a.kind]
    if a.kind.startswith("fp8_block"):          # exact per-K-block promotion, or the weight re-expressed in MXFP8
        ops._fp8_block_exact = a.kind == "fp8_block"
    w = torch.randn(a.n, a.k, device="cuda") * 0.02
    lin0 = Linear.from_dense(w, fmt)
    del w
    wbytes = lin0.nbytes()
    copies = max(1, min(64, (300 << 20) // max(wbytes, 1) + 1))
    lins = [lin0]
    for _ in range(copies - 1):
        c = Linear.__new__(Linear)
        c.__dict__.update(lin0.__dict__)
        c.w = lin0.w.clone()
        c.cuda_pack = None
        lins.append(c)
    x = torch.randn(a.m, a.k, device="cuda").bfloat16()
    xin = ops.quantize_rows(x, lin0) if ops._qmode(lin0) else x
    if a.kind == "fp8_block" and not a.with_quant:
        from ..linear import QuantAct
        q, sc = ops.quantize_fp8_block(x)
        xin = QuantAct(Format.FP8_BLOCK, q, sc, None, a.m, a.k, dense=x)
    wide = {"auto": None, "on": True, "off": False}[a.wide]
    sk = None if a.sk == "auto" else (False if a.sk == "off" else (True if a.sk == "on" else int(a.sk)))
    out = torch.empty(a.m, a.n, dtype=torch.float32 if a.f32 else torch.bfloat16, device="cuda")

    def run():
        for lin in lins:
            ops.linear(lin, xin, out=out, bn=a.bn, wide=wide, ksplit=a.ksplit, out_dtype=torch.float32 if a.f32 else None, sk=sk)

    run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    med, best = timeit(g.replay, a.iters, flush=copies == 1)
    med, best = med / copies, best / copies
    flops = 2.0 * a.m * a.n * a.k
    pk = peaks()
    print(json.dumps({"kernel": f"gemm {a.kind}", "m": a.m, "n": a.n, "k": a.k, "bn": a.bn, "wide": a.wide, "ksplit": a.ksplit, "sk": a.sk,
                      "copies": copies, "us_median": med * 1e3, "us_best": best * 1e3,
                      "tflops": flops / med / 1e9, "x_bf16_cublas_" + pk["src"]: flops / med / 1e9 / pk["bf16_tflops"],
                      "weight_gbs": wbytes / med / 1e6, "x_hbm_" + pk["src"]: wbytes / med / 1e6 / pk["hbm_gbs"],
                      "status": ops.take_status()}))


def bench_norm(a):
    from ..linear import Linear
    from ..ops import get_ops
    from ..quant import Format
    ops = get_ops("cuda")
    x = torch.randn(a.rows, a.hidden, device="cuda").bfloat16()
    r = torch.randn(a.rows, a.hidden, device="cuda").bfloat16()
    w = torch.ones(a.hidden, device="cuda").bfloat16()
    lin = Linear.from_dense(torch.randn(128, a.hidden, device="cuda") * 0.02, Format.NVFP4)
    fn = lambda: ops.norm(x, r, w, 1e-6, quant_for=lin)  # noqa: E731
    med, best = timeit(fn, a.iters)
    nbytes = a.rows * a.hidden * (2 + 2 + 2 + 0.5625)
    pk = peaks()
    print(json.dumps({"kernel": "rmsnorm+nvfp4", "rows": a.rows, "hidden": a.hidden, "ms_median": med,
                      "gbs": nbytes / med / 1e6, "frac_hbm_" + pk["src"]: nbytes / med / 1e6 / pk["hbm_gbs"]}))


def bench_moe(a):
    """Routed experts of one layer (scatter, two expert GEMMs, activation, combine) at decode-sized routing."""
    from ..linear import Linear
    from ..models.qwen3 import Experts
    from ..ops import get_ops
    from ..quant import Format
    ops = get_ops("cuda")
    fmt = {"nvfp4": Format.NVFP4, "mxfp8": Format.MXFP8, "bf16": Format.DENSE}[a.kind]
    ex = Experts()
    ex.num_experts, ex.first, ex.count = a.experts, 0, a.experts
    for _ in range(a.experts):
        ex.gate_up.append(Linear.from_dense(torch.randn(2 * a.inter, a.hidden, device="cuda") * 0.05, fmt, segments=[a.inter, a.inter]))
        ex.down.append(Linear.from_dense(torch.randn(a.hidden, a.inter, device="cuda") * 0.05, fmt))
    x = torch.randn(a.tokens, a.hidden, device="cuda").bfloat16()
    logits = torch.randn(a.tokens, a.experts, device="cuda")
    wbytes = sum(l.nbytes() for l in ex.gate_up) + sum(l.nbytes() for l in ex.down)

    def run():
        w, ids = ops.router_topk(logits, a.topk, True, 0, a.experts)
        return ops.moe(x, w, ids, ex)
    res = {}
    for name, rows in (("narrow", 48), ("padded_128_row_tiles", 0)):
        ops.MOE_NARROW_ROWS = rows
        run()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            run()
        med, best = timeit(g.replay, a.iters, flush=True)
        res[name + "_us"] = med * 1e3
    pk = peaks()
    print(json.dumps({"kernel": f"moe layer {a.kind}", "tokens": a.tokens, "experts": a.experts, "topk": a.topk, "hidden": a.hidden,
                      "inter": a.inter, **res, "expert_weight_mb": wbytes / 1e6,
                      "weight_gbs_narrow": wbytes / res["narrow_us"] / 1e3,
                      "x_hbm_" + pk["src"]: wbytes / res["narrow_us"] / 1e3 / pk["hbm_gbs"], "status": ops.take_status()}))


def bench_gdn(a):
    """Gated DeltaNet layer core (conv + gated delta rule + gated norm) over prompts: the chunked tensor-core kernel against
    (preparation of all chunks in parallel + sequential scan, and the one fused kernel) against the token-by-token kernel
    on the same inputs."""
    from ..batch import SeqChunk, build_batch
    from ..config import named_config
    from ..kv import KVCache
    from ..ops import get_ops
    ops = get_ops("cuda")
    cfg = named_config("qwen3-next-80b-a3b")
    hk, hv, dk, dv = a.hk, a.hv, 128, 128
    cfg.linear_num_key_heads, cfg.linear_num_value_heads = hk, hv
    cfg.num_layers, cfg.layer_types = 1, ["linear_attention"]

    class G:
        pass
    gd = G()
    gd.k_heads, gd.v_heads = hk, hv
    C = 2 * hk * dk + hv * dv
    gd.conv_w = (torch.randn(C, 4, device="cuda") * 0.3).bfloat16()
    gd.A_log = torch.log(torch.linspace(1, 4, hv, device="cuda") * 0.1)
    gd.dt_bias = torch.randn(hv, device="cuda") * 0.1
    gd.norm_w = torch.ones(dv, device="cuda").bfloat16()

    class M:
        pass
    m = M()
    m.cfg = cfg
    kv = KVCache(cfg, 4, a.seqs, (a.tokens + 15) // 16 + 1, "bf16", "cuda", "logical")
    batch = build_batch([SeqChunk(b, [0] * a.tokens, 0) for b in range(a.seqs)], kv.block_table_host, "cuda")
    T = batch.num_rows
    mixed = torch.randn(T, C, device="cuda").bfloat16()
    z = torch.randn(T, hv * dv, device="cuda").bfloat16()
    bb = torch.randn(T, hv, device="cuda").bfloat16()
    aa = torch.randn(T, hv, device="cuda").bfloat16()
    res = {}
    for name, cm, split in (("chunked", 64, True), ("chunked_one_kernel", 64, False), ("token_by_token", 0, False)):
        ops.GDN_CHUNK_MIN, ops.GDN_SPLIT = cm, split
        med, best = timeit(lambda: ops.gdn(mixed, z, bb, aa, gd, m, batch, kv, 0), a.iters, flush=False)
        res[name + "_ms"] = med
    res["status"] = ops.take_status()
    print(json.dumps({"kernel": "gdn layer core", "seqs": a.seqs, "tokens": a.tokens, "k_heads": hk, "v_heads": hv, **res,
                      "speedup": res["token_by_token_ms"] / res["chunked_ms"],
                      "us_per_token_chunked": res["chunked_ms"] * 1e3 / a.tokens}))


def main(argv=None):
    ap = argparse.ArgumentParser(prog="blaze_b200.benchmarks.kernels")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("attention")
    p.add_argument("--batch", type=int, default=256)
    p.add_argument("--ctx", type=int, default=1024)
    p.add_argument("--qlen", type=int, default=1)
    p.add_argument("--hq", type=int, default=32)
    p.add_argument("--hkv", type=int, default=8)
    p.add_argument("--splits", type=int, default=0)
    p.add_argument("--prof", action="store_true", help="print per-role wait cycles of the decode kernel")
    p.add_argument("--iters", type=int, default=10)
    p = sub.add_parser("gemm")
    p.add_argument("--kind", default="nvfp4")
    p.add_argument("--m", type=int, default=256)
    p.add_argument("--n", type=int, default=6144)
    p.add_argument("--k", type=int, default=4096)
    p.add_argument("--bn", type=int, default=0)
    p.add_argument("--wide", default="auto", choices=["auto", "on", "off"])
    p.add_argument("--ksplit", type=int, default=0)
    p.add_argument("--sk", default="auto", help="cluster split-K kernel: auto | on | off | a K-slice count 1..8")
    p.add_argument("--f32", action="store_true")
    p.add_argument("--with-quant", action="store_true", help="fp8_block: time the 1x128 activation quantiser with the GEMM")
    p.add_argument("--iters", type=int, default=10)
    p = sub.add_parser("norm")
    p.add_argument("--rows", type=int, default=256)
    p.add_argument("--hidden", type=int, default=4096)
    p.add_argument("--iters", type=int, default=10)
    p = sub.add_parser("moe")
    p.add_argument("--kind", default="nvfp4")
    p.add_argument("--tokens", type=int, default=256)
    p.add_argument("--experts", type=int, default=128)
    p.add_argument("--topk", type=int, default=8)
    p.add_argument("--hidden", type=int, default=2048)
    p.add_argument("--inter", type=int, default=768)
    p.add_argument("--iters", type=int, default=5)
    p = sub.add_parser("gdn")
    p.add_argument("--seqs", type=int, default=1)
    p.add_argument("--tokens", type=int, default=4096)
    p.add_argument("--hk", type=int, default=16)
    p.add_argument("--hv", type=int, default=32)
    p.add_argument("--iters", type=int, default=5)
    a = ap.parse_args(argv)
    {"attention": bench_attention, "gemm": bench_gemm, "norm": bench_norm, "gdn": bench_gdn, "moe": bench_moe}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
