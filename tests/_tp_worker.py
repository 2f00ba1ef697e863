"""Worker run under torch.distributed.run by test_multigpu.py (one process per GPU)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from blaze_b200 import quant  # noqa: E402
from blaze_b200.config import ModelConfig, RopeConfig  # noqa: E402
from blaze_b200.engine import Engine, EngineConfig  # noqa: E402
from blaze_b200.linear import Linear  # noqa: E402
from blaze_b200.models.qwen3 import Model, TPInfo  # noqa: E402
from blaze_b200.ops import ref  # noqa: E402
from blaze_b200.parallel.symm import SymmAllReduce  # noqa: E402
from blaze_b200.parallel.tp import TPGroup  # noqa: E402
from blaze_b200.quant import Format  # noqa: E402


def pipeline_case(dev):
    """Two pipeline stages on two GPUs (one rank each, NCCL hand-off of hidden rows in micro-batches): the tokens must be the
    single-process tokens; near-ties may flip where the stage split changes nothing but the launch shapes, so most must agree."""
    from blaze_b200.config import ModelConfig, RopeConfig
    from blaze_b200.llm import LLM
    from blaze_b200.parallel.pp import stage_layers
    from blaze_b200.parallel.worker import attach, follow
    from blaze_b200.sampler import SamplingParams
    pg = TPGroup.from_env(dev, pp=2)
    rank = pg.global_rank
    assert (pg.stages, pg.world) == (2, 1)
    cfg = ModelConfig(vocab_size=2048, hidden_size=512, num_layers=4, num_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, rope=RopeConfig(theta=1e6))
    cfg.layer_types = ["full_attention"] * 4
    prompts = torch.randint(0, 2048, (5, 70), generator=torch.Generator().manual_seed(3)).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    base = dict(weight_format="nvfp4", device=dev, max_seqs=8, max_model_len=256, use_graphs=False, seed=2,
                enable_prefix_caching=False, chunk=128)
    solo = [o.token_ids for o in LLM(cfg, **base).generate(prompts, sp)] if rank == 0 else None
    llm = LLM(cfg, stage_layers=stage_layers(cfg.num_layers, 2, pg.stage), **base)
    llm.group = pg
    lead = attach(llm, pg, pp_chunk=64)
    if rank == 0:
        got = [o.token_ids for o in llm.generate(prompts, sp)]
        lead.quit()
        same = sum(a == b for a, b in zip(sum(solo, []), sum(got, [])))
        total = len(sum(solo, []))
        print(f"[pp-gpu] tokens equal to the single-process run: {same}/{total}; {llm.pipeline.micro_batches} micro-batches in "
              f"{llm.sched.stats.steps} steps", flush=True)
        assert all(len(g) == 10 for g in got) and same >= 0.85 * total
        assert llm.pipeline.micro_batches > llm.sched.stats.steps
    else:
        assert follow(llm) == 0
    torch.cuda.synchronize()
    from blaze_b200.ops import get_ops
    assert get_ops(dev).take_status() == 0
    dist.barrier()
    if rank == 0:
        print("[worker] pipeline ok", flush=True)
    dist.destroy_process_group()


def main():
    case = sys.argv[1]
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    if case == "pipeline":
        return pipeline_case(dev)
    group = TPGroup.from_env(dev)
    rank, world = group.rank, group.world
    use_mc = os.environ.get("BLAZE_TEST_MULTICAST", "1") == "1"
    T, H = 200, 2048
    fused = SymmAllReduce.create(group, dev, max_rows=512, hidden=H, use_multicast=use_mc)
    if rank == 0:
        print(f"[worker] case={case} world={world} multicast={'on' if fused.use_mc else 'off'}", flush=True)
    g = torch.Generator(device=dev).manual_seed(100 + rank)

    if case == "allreduce":
        for it in range(3):
            x = torch.randn(T, H, generator=g, device=dev).bfloat16()
            want = x.float().clone()
            dist.all_reduce(want)
            buf = fused.next_input(T, H)
            buf.copy_(x)
            y = fused.all_reduce(buf)
            torch.cuda.synchronize()
            err = (y.float() - want).abs().max().item()
            assert err < 0.07, f"all-reduce mismatch {err}"
            # identical bits on every rank
            chk = y.float().sum().double()
            lst = [torch.zeros_like(chk) for _ in range(world)]
            dist.all_gather(lst, chk)
            assert all(float(v) == float(lst[0]) for v in lst), "ranks disagree"
    elif case == "gemm_allreduce":
        from blaze_b200.ops import get_ops
        ops = get_ops(dev)
        if not fused.use_mc:
            print("[worker] no multicast mapping: fused GEMM + all-reduce skipped", flush=True)
        else:
            for fmt, M, N, K in ((Format.DENSE, 200, 2048, 1024), (Format.NVFP4, 256, 2048, 2048), (Format.DENSE, 64, 2048, 512)):
                w = torch.randn(N, K, generator=g, device=dev) * 0.05
                lin = Linear.from_dense(w, fmt)
                x = torch.randn(M, K, generator=g, device=dev).bfloat16()
                local = ops.linear(lin, x).float()
                want = local.clone()
                dist.all_reduce(want)
                for rep in range(2):
                    y = fused.gemm_allreduce(ops, lin, x, M)
                    torch.cuda.synchronize()
                    err = (y.float() - want).abs().max().item()
                    ref_mag = want.abs().mean().item()
                    assert err < 0.05 * max(ref_mag, 1.0) + 0.05, f"fused GEMM+all-reduce mismatch {err} (mean |ref| {ref_mag})"
                    y.zero_()            # hand the accumulation buffer back zeroed, as the norm kernel does
                    torch.cuda.synchronize()
                    dist.barrier()
    elif case == "reduce_norm":
        w = (1 + 0.1 * torch.randn(H, generator=torch.Generator(device=dev).manual_seed(7), device=dev)).bfloat16()
        gfull = torch.Generator(device=dev).manual_seed(11)
        res_full = torch.randn(T, H, generator=gfull, device=dev).bfloat16()
        for mode, fmt in ((0, None), (1, Format.NVFP4), (2, Format.MXFP8), (3, None)):
            x = torch.randn(T, H, generator=g, device=dev).bfloat16()
            tot = x.float().clone()
            dist.all_reduce(tot)
            tot = tot.bfloat16()
            res = fused.shard_rows(res_full)
            lin = Linear.from_dense(torch.randn(64, H, device=dev) * 0.02, fmt) if fmt else None
            buf = fused.next_input(T, H)
            buf.copy_(x)
            out = fused.reduce_norm(buf, res, None if mode == 3 else w, 1e-6, False, lin)
            torch.cuda.synchronize()
            want_h, want_res = ref.rmsnorm(tot, w, 1e-6, res_full)
            per = fused.rows_per(T)
            lo, hi = rank * per, min(T, rank * per + per)
            assert (res[:hi - lo].float() - want_res[lo:hi].float()).abs().max().item() < 0.07, "residual shard"
            if mode == 0:
                assert (out.float() - want_h.float()).abs().max().item() < 0.1, "normed rows"
            elif mode == 3:
                assert (out.float() - want_res.float()).abs().max().item() < 0.07, "summed rows"
            elif mode == 1:
                sf = quant.unswizzle_sf_128x4(out.sf, T, H // 16).view(torch.float8_e4m3fn)
                xd = quant.nvfp4_dequantize(out.data, sf, out.row_scale)
                e = (xd - want_h.float()).abs().mean().item()
                assert e < 0.12, f"nvfp4 rows err {e}"
            else:
                sf = quant.unswizzle_sf_128x4(out.sf, T, H // 32)
                xd = quant.mxfp8_dequantize(out.data.view(torch.float8_e4m3fn), sf)
                e = (xd - want_h.float()).abs().mean().item()
                assert e < 0.04, f"mxfp8 rows err {e}"
    elif case == "push_reduce_norm":
        from blaze_b200.ops import get_ops
        ops = get_ops(dev)
        w = (1 + 0.1 * torch.randn(H, generator=torch.Generator(device=dev).manual_seed(7), device=dev)).bfloat16()
        res_full = torch.randn(512, H, generator=torch.Generator(device=dev).manual_seed(11), device=dev).bfloat16()
        for it, (fmt, M, K, qfmt) in enumerate(((Format.DENSE, 200, 1024, None), (Format.NVFP4, 256, 2048, Format.NVFP4),
                                                (Format.NVFP4, 77, 1024, Format.MXFP8), (Format.DENSE, 300, 512, None),
                                                (Format.NVFP4, 256, 2048, Format.NVFP4))):
            lin = Linear.from_dense(torch.randn(H, K, generator=g, device=dev) * 0.05, fmt)
            x = torch.randn(M, K, generator=g, device=dev).bfloat16()
            local = ops.linear(lin, x, wide=False, sk=False)                  # this rank's partial sums, bf16
            tot = local.float().clone()
            dist.all_reduce(tot)
            tot = tot.bfloat16()
            res = fused.shard_rows(res_full[:M])
            nxt = Linear.from_dense(torch.randn(64, H, device=dev) * 0.02, qfmt) if qfmt else None
            pushed = fused.gemm_push(ops, lin, x, M)
            out = fused.reduce_norm(pushed, res, w, 1e-6, False, nxt)
            torch.cuda.synchronize()
            want_h, want_res = ref.rmsnorm(tot, w, 1e-6, res_full[:M])
            per = fused.rows_per(M)
            lo, hi = rank * per, min(M, rank * per + per)
            tol = 0.07 * max(1.0, want_res.float().abs().max().item() / 4)
            assert (res[:hi - lo].float() - want_res[lo:hi].float()).abs().max().item() < tol, f"case {it}: residual shard"
            if qfmt is None:
                assert (out.float() - want_h.float()).abs().max().item() < 0.1, f"case {it}: normed rows"
            elif qfmt == Format.NVFP4:
                sf = quant.unswizzle_sf_128x4(out.sf, M, H // 16).view(torch.float8_e4m3fn)
                xd = quant.nvfp4_dequantize(out.data, sf, out.row_scale)
                e = (xd - want_h.float()).abs().mean().item()
                assert e < 0.12, f"case {it}: nvfp4 rows err {e}"
            else:
                sf = quant.unswizzle_sf_128x4(out.sf, M, H // 32)
                xd = quant.mxfp8_dequantize(out.data.view(torch.float8_e4m3fn), sf)
                e = (xd - want_h.float()).abs().mean().item()
                assert e < 0.04, f"case {it}: mxfp8 rows err {e}"
            dist.barrier()
    elif case == "model":
        cfg = ModelConfig(vocab_size=2048, hidden_size=512, num_layers=2, num_heads=8, num_kv_heads=2, head_dim=128,
                          intermediate_size=1024, rope=RopeConfig(theta=1e6))
        cfg.layer_types = ["full_attention"] * 2
        prompts = torch.randint(0, 2048, (3, 37), generator=torch.Generator().manual_seed(5)).tolist()

        def run(tp, fused_on):
            if tp.group is not None:
                tp.group.fused = SymmAllReduce.create(tp.group, dev, max_rows=256, hidden=512, use_multicast=use_mc) if fused_on else None
            m = Model.random_init(cfg, fmt=Format.DENSE, seed=3, device=dev, tp=tp)
            eng = Engine(m, EngineConfig(max_seqs=4, max_model_len=128, kv_dtype="fp8", kv_tokens=2048, use_graphs=False))
            seqs = [eng.open_from() for _ in prompts]
            toks = eng.forward(eng.plan([(s, p, 1) for s, p in zip(seqs, prompts)]), "greedy")
            outs = [toks.tolist()]
            for _ in range(6):
                toks = eng.forward(eng.plan([(s, [int(t)], 1) for s, t in zip(seqs, toks.tolist())]), "greedy")
                outs.append(toks.tolist())
            return outs

        solo = run(TPInfo(), False)
        nccl = run(TPInfo(rank, world, group), False)
        fus = run(TPInfo(rank, world, group), True)
        if rank == 0:
            print("[worker] fusion mode", group.fused.mode, flush=True)
        if rank == 0:
            print("[worker] tp1  ", solo[:3], "\n[worker] nccl ", nccl[:3], "\n[worker] fused", fus[:3], flush=True)
        agree = sum(a == b for a, b in zip(sum(solo, []), sum(fus, [])))
        total = len(sum(solo, []))
        assert nccl[0] == solo[0] or agree >= total * 0.8, "TP=2 (NCCL) diverges from TP=1"
        assert agree >= total * 0.8, f"fused TP path diverges from TP=1: {agree}/{total}"
    else:
        raise SystemExit(f"unknown case {case}")
    torch.cuda.synchronize()
    from blaze_b200.ops import get_ops
    st = get_ops(dev).take_status()
    assert st == 0, f"device status {st}"
    dist.barrier()
    if rank == 0:
        print(f"[worker] {case} ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
