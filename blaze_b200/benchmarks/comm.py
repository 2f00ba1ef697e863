"""Collective micro-benchmarks, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29511 \
        -m blaze_b200.benchmarks.comm --rows 256 --hidden 4096

Times, inside a captured CUDA graph of ``--reps`` back-to-back calls (so that the host is not what is measured) and as
the maximum over ranks:  the NCCL all-reduce of a bf16 ``[rows, hidden]`` buffer, NCCL all-reduce + this library's
residual/RMSNorm/NVFP4 kernel (the unfused sequence), the in-kernel all-reduce over peer memory, the fused all-reduce +
residual + RMSNorm (+ NVFP4 quantisation) kernel, and the one-kernel GEMM + all-reduce.  Prints one JSON line on rank 0;
``x_link`` relates the fused kernels to the bytes that must cross NVLink per GPU at the measured 770 GB/s per direction.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=256)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=12288, help="K of the row-cut GEMM before the reduction (per model, not per rank)")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-multicast", action="store_true")
    ap.add_argument("--prof", action="store_true", help="also print where block 0 of the fused kernels spends its time")
    a = ap.parse_args(argv)
    from ..linear import Linear
    from ..ops import get_ops
    from ..parallel.symm import SymmAllReduce
    from ..parallel.tp import TPGroup
    from ..quant import Format

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    group = TPGroup.from_env(dev)
    if group is None:
        raise SystemExit("run under torch.distributed.run with at least 2 processes")
    rank, world = group.rank, group.world
    ops = get_ops(dev)
    T, H = a.rows, a.hidden
    fused = SymmAllReduce.create(group, dev, max_rows=max(T, 512), hidden=H, use_multicast=not a.no_multicast)
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    x = (torch.randn(T, H, generator=g, device=dev) * 0.1).bfloat16()
    w = torch.ones(H, dtype=torch.bfloat16, device=dev)
    K = a.inter // world
    lin = Linear.from_dense(torch.randn(H, K, generator=g, device=dev) * 0.02, Format.NVFP4)
    nxt = Linear.from_dense(torch.randn(256, H, generator=g, device=dev) * 0.02, Format.NVFP4)    # decides the quant format
    xk = ops.quantize_rows((torch.randn(T, K, generator=g, device=dev) * 0.1).bfloat16(), lin)
    res_full = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
    res_shard = fused.shard_rows(res_full)

    def nccl_ar():
        dist.all_reduce(x)

    def nccl_ar_norm():
        dist.all_reduce(x)
        ops.norm(x, res_full, w, 1e-6, False, quant_for=nxt)

    def fused_ar():
        fused.all_reduce(fused.next_input(T, H))

    def fused_rn():
        fused.reduce_norm(fused.next_input(T, H), res_shard, w, 1e-6, False, quant_for=nxt)

    def gemm_then_rn():
        ops.linear(lin, xk, out=fused.next_input(T, H))
        fused.reduce_norm(fused.next_input(T, H), res_shard, w, 1e-6, False, quant_for=nxt)

    qkv = Linear.from_dense(torch.randn(6144 // world, H, generator=g, device=dev) * 0.02, Format.NVFP4)

    def rn_then_gemm():
        qa = fused.reduce_norm(fused.next_input(T, H), res_shard, w, 1e-6, False, quant_for=qkv)
        ops.linear(qkv, qa)

    def rn_signal_then_gemm_waits():
        qa = fused.reduce_norm(fused.next_input(T, H), res_shard, w, 1e-6, False, quant_for=qkv, defer=True)
        ops.linear(qkv, qa)

    def gemm_only():
        ops.linear(lin, xk)

    def gemm_ar():
        y = fused.gemm_allreduce(ops, lin, xk, T)
        ops.norm(y, res_full, w, 1e-6, False, quant_for=nxt, zero_src=True)

    def gemm_push_then_rn():
        fused.reduce_norm(fused.gemm_push(ops, lin, xk, T), res_shard, w, 1e-6, False, quant_for=nxt)

    def gemm_push_rn_next_gemm():
        qa = fused.reduce_norm(fused.gemm_push(ops, lin, xk, T), res_shard, w, 1e-6, False, quant_for=qkv)
        ops.linear(qkv, qa)

    def gemm_rn_next_gemm():
        ops.linear(lin, xk, out=fused.next_input(T, H))
        qa = fused.reduce_norm(fused.next_input(T, H), res_shard, w, 1e-6, False, quant_for=qkv)
        ops.linear(qkv, qa)

    def gemm_push_only():
        fused.gemm_push(ops, lin, xk, T)

    import ctypes as _ct
    _loc = fused.arena.local.data_ptr()

    def gemm_push_local():
        # the same epilogue with every owner's slot buffer in local memory: what the push costs without NVLink
        b = fused.push_cur ^ 1
        fused.push_cur = b
        VPn = _ct.c_void_p
        slots = (VPn * world)(*[VPn(_loc + fused.off_slot[b])] * world)
        flags = (VPn * world)(*[VPn(_loc + fused.off_slot_flag + 2048 + 64 * b)] * world)
        fused.lib.blz_gemm_push_rs(slots, flags, VPn(fused.push_state.data_ptr() + 8), VPn(fused.push_state.data_ptr() + 12), rank, world,
                                   fused.rows_per(T))
        ops.linear(lin, xk, out=fused.arena.view(fused.off_in[0], T * H * 2).view(torch.bfloat16).view(T, H), wide=False, sk=False)

    cases = [("nccl_allreduce", nccl_ar), ("nccl_allreduce+norm_quant", nccl_ar_norm), ("fused_allreduce", fused_ar),
             ("fused_allreduce_norm_quant", fused_rn), ("gemm", gemm_only), ("gemm+fused_allreduce_norm_quant", gemm_then_rn),
             ("fused_allreduce_norm_quant+next_gemm", rn_then_gemm),
             ("fused_allreduce_norm_quant(signal only)+next_gemm(waits)", rn_signal_then_gemm_waits),
             ("gemm(push reduce-scatter) alone", gemm_push_only), ("gemm(push, local slots only)", gemm_push_local),
             ("gemm(push reduce-scatter)+slots_norm_quant", gemm_push_then_rn),
             ("gemm+fused_allreduce_norm_quant+next_gemm", gemm_rn_next_gemm),
             ("gemm(push reduce-scatter)+slots_norm_quant+next_gemm", gemm_push_rn_next_gemm)]
    if fused.use_mc:
        cases.append(("gemm_allreduce_one_kernel+norm_quant", gemm_ar))
    out = {}
    for name, fn in cases:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(a.reps):
                fn()
        times = []
        for _ in range(a.iters):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            gr.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / a.reps)
        times.sort()
        t = torch.tensor([times[len(times) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name] = float(t.item()) * 1e3
        del gr
    phases = {}
    if a.prof:
        # where block 0 of one kernel spends its time: wait for the peers, reduction (+ norm), stores, closing barrier
        import ctypes
        buf = torch.zeros(8, dtype=torch.int64, device=dev)
        fused.lib.blz_comm_set_prof.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        fused.lib.blz_comm_set_prof(fused.comm, ctypes.c_void_p(buf.data_ptr()))
        for name, fn in (("fused_allreduce", fused_ar), ("fused_allreduce_norm_quant", fused_rn),
                         ("gemm(push reduce-scatter)+slots_norm_quant", gemm_push_then_rn)):
            acc = torch.zeros(4, dtype=torch.float64)
            n = 0
            for _ in range(10):
                dist.barrier()
                torch.cuda.synchronize()
                buf.zero_()
                fn()
                torch.cuda.synchronize()
                b = buf.tolist()
                if b[4] and b[1]:
                    mid = b[2] if b[2] else b[1]
                    acc += torch.tensor([b[1] - b[0], mid - b[1], b[3] - mid, b[4] - b[3]], dtype=torch.float64)
                    n += 1
            if n:
                phases[name] = {k: float(v) / n / 1e3 for k, v in zip(("entry_barrier_us", "reduce_us", "norm_store_us", "exit_barrier_us"), acc)}
        fused.lib.blz_comm_set_prof(fused.comm, ctypes.c_void_p(0))
    status = ops.take_status()
    if rank == 0:
        # bytes each GPU must send (= receive) for a reduce-scatter + all-gather of the bf16 buffer
        link_bytes = 2.0 * (world - 1) / world * T * H * 2
        floor_us = link_bytes / 770e9 * 1e6
        print(json.dumps({"bench": "comm", "world": world, "rows": T, "hidden": H, "multicast": fused.use_mc, "us": out, "phases_block0": phases,
                          "nvlink_floor_us_bf16_allreduce": floor_us, "x_link_fused_allreduce": floor_us / out["fused_allreduce"],
                          "status": status}))
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


if __name__ == "__main__":
    main()
