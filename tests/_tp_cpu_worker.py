"""Worker for test_tp_cpu.py: two gloo ranks on the CPU (run under torch.distributed.run)."""
import datetime
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from blaze_b200.config import named_config  # noqa: E402
from blaze_b200.llm import LLM  # noqa: E402
from blaze_b200.models.qwen3 import TPInfo  # noqa: E402
from blaze_b200.parallel.tp import TPGroup  # noqa: E402
from blaze_b200.parallel.worker import Leader, follow  # noqa: E402
from blaze_b200.sampler import SamplingParams  # noqa: E402


def build(tp, **kw):
    cfg = named_config("tiny")
    base = dict(device="cpu", dtype=torch.float32, max_seqs=8, max_model_len=256, use_graphs=False, seed=0, tp=tp)
    base.update(kw)
    return LLM(cfg, **base)


def main():
    case = sys.argv[1]
    timeout = datetime.timedelta(seconds=20 if case == "rank_leaves" else 120)
    dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]), timeout=timeout)
    group = TPGroup.from_env("cpu")
    rank, world = group.rank, group.world
    prompts = torch.randint(0, 1024, (4, 21), generator=torch.Generator().manual_seed(3)).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=10)

    if case == "generate":
        # the same requests through one process and through two tensor-parallel ranks (rank 0 plans, rank 1 follows)
        solo = [o.token_ids for o in build(TPInfo()).generate(prompts, sp)] if rank == 0 else None
        llm = build(TPInfo(rank, world, group), chunk=16)
        if rank == 0:
            lead = Leader(llm.engine, group)
            got = [o.token_ids for o in llm.generate(prompts, sp)]
            lead.quit()
            same = sum(a == b for a, b in zip(sum(solo, []), sum(got, [])))
            total = len(sum(solo, []))
            print(f"[tp-cpu] tokens equal to the single-process run: {same}/{total}", flush=True)
            assert same >= 0.9 * total
            assert all(len(g) == 10 for g in got)
        else:
            assert follow(llm) == 0
    elif case == "expert_placement":
        # expert parallelism over two ranks with the experts spread by a routing profile: same tokens as one process with
        # the experts in checkpoint order, and the statistics collected under the placement stay in checkpoint numbering
        import numpy as np
        from blaze_b200.expert_heat import ExpertHeat
        cfg = named_config("tiny-hybrid")
        path = sys.argv[2]
        kw = dict(device="cpu", dtype=torch.float32, max_seqs=8, max_model_len=256, use_graphs=False, seed=0, chunk=16)
        if rank == 0:
            solo_llm = LLM(cfg, expert_heat=True, **kw)
            solo = [o.token_ids for o in solo_llm.generate(prompts, sp)]
            solo_llm.save_expert_heat()
            prof = ExpertHeat(cfg.num_layers, cfg.num_experts)
            load = np.ones(cfg.num_experts)
            load[:cfg.num_experts // 2] = 50.0          # the hot half is what rank 0 would hold in checkpoint order
            prof.longterm[:] = load
            prof.recent[:] = load
            prof.save(path)
        dist.barrier()
        llm = LLM(cfg, tp=TPInfo(rank, world, group, ep=True), expert_heat=path, expert_placement="heat", **kw)
        order = llm.model.tp.expert_order
        assert order is not None and sorted(order[0].tolist()) == list(range(cfg.num_experts))
        half = cfg.num_experts // 2
        hot_on_rank0 = sum(1 for e in order[0][:half] if e < half)
        assert hot_on_rank0 == half // 2, "the hot experts must be split evenly over the two ranks"
        if rank == 0:
            before = llm.heat.longterm.copy()
            lead = Leader(llm.engine, group)
            got = [o.token_ids for o in llm.generate(prompts, sp)]
            lead.quit()
            same = sum(a == b for a, b in zip(sum(solo, []), sum(got, [])))
            total = len(sum(solo, []))
            print(f"[tp-cpu] tokens equal to the single-process run: {same}/{total}", flush=True)
            assert same >= 0.9 * total
            llm.heat.fold()
            if same == total:
                assert np.array_equal(llm.heat.longterm - before, solo_llm.heat.longterm), "statistics must be in checkpoint numbering"
                print("[tp-cpu] routing statistics equal to the single-process run", flush=True)
        else:
            assert follow(llm) == 0
    elif case == "mtp":
        # a one-layer chain drafter cut over the two ranks like the target: its steps are mirrored on rank 1 (with the fused
        # input rows broadcast from rank 0), its head is the target's sharded head; the streams equal plain decoding
        from blaze_b200.parallel.worker import attach
        sp4 = SamplingParams(temperature=0.0, max_tokens=14)
        solo = [o.token_ids for o in build(TPInfo()).generate(prompts, sp4)] if rank == 0 else None
        llm = build(TPInfo(rank, world, group), chunk=16, spec_method="mtp", max_draft=4)
        assert llm.drafter is not None and llm.drafter.m.tp.world == 2
        lead = attach(llm, group)
        if rank == 0:
            assert llm.draft_leader is not None
            got = [o.token_ids for o in llm.generate(prompts, sp4)]
            lead.quit()
            same = sum(a == b for a, b in zip(sum(solo, []), sum(got, [])))
            total = len(sum(solo, []))
            st = llm.sched.stats
            print(f"[tp-cpu] MTP k=4 under TP 2: tokens equal to plain single-process decoding {same}/{total}; drafted "
                  f"{st.draft_tokens}, accepted {st.accepted_tokens}", flush=True)
            assert same >= 0.9 * total and st.draft_tokens > 0 and llm.drafter.proposed > 0
        else:
            assert follow(llm) == 0
    elif case == "pipeline":
        # two pipeline stages (one rank each): layers split in half, hidden rows handed over in micro-batches of 8 rows,
        # the last stage returns the tokens to rank 0; outputs must equal the single-process run exactly
        from blaze_b200.parallel.pp import stage_layers
        from blaze_b200.parallel.worker import attach
        pg = TPGroup.from_env("cpu", pp=2)
        assert (pg.stage, pg.stages, pg.world, pg.global_rank) == (rank, 2, 1, rank)
        cfg = named_config("tiny")
        solo = [o.token_ids for o in build(TPInfo()).generate(prompts, sp)] if rank == 0 else None
        llm = build(TPInfo(), chunk=16, stage_layers=stage_layers(cfg.num_layers, 2, pg.stage))
        llm.group = pg
        lead = attach(llm, pg, pp_chunk=8)
        if rank == 0:
            got = [o.token_ids for o in llm.generate(prompts, sp)]
            lead.quit()
            assert got == solo, (got, solo)
            assert llm.pipeline.micro_batches > llm.sched.stats.steps      # prompt steps were cut into several micro-batches
            print(f"[pp-cpu] two stages give the single-process tokens; {llm.pipeline.micro_batches} micro-batches in "
                  f"{llm.sched.stats.steps} steps", flush=True)
        else:
            assert follow(llm) == 0
    elif case == "rank_leaves":
        # rank 1 leaves between two steps; rank 0's next step must end with an error inside the group timeout, fail the
        # requests of that step and leave the scheduler able to answer again (here: with an error, since the group is gone)
        llm = build(TPInfo(rank, world, group))
        if rank == 0:
            Leader(llm.engine, group)
            finished = []
            from blaze_b200.sched import GenRequest
            llm.sched.submit(GenRequest("r0", prompts[0], SamplingParams(temperature=0.0, max_tokens=50),
                                        sink=lambda ev: finished.append(ev) if ev.finish is not None else None))
            llm.sched.start()
            import time
            t0 = time.monotonic()
            while not finished and time.monotonic() - t0 < 60:
                time.sleep(0.05)
            llm.sched.stop()
            assert finished, "the request never finished after the peer left"
            assert finished[0].finish.value == "error" and finished[0].error
            print(f"[tp-cpu] peer left: request failed after {time.monotonic() - t0:.1f}s with {finished[0].error[:60]!r}", flush=True)
            os._exit(0)
        else:
            # follow three steps, then leave with nothing in flight
            eng = llm.engine
            from blaze_b200.batch import SeqChunk
            from blaze_b200.engine import Seq
            for _ in range(3):
                msg = group.broadcast_object(None, 0)
                _, mode, raw, changed, gone, feedback = msg
                for row, pg in changed.items():
                    s = eng.seqs.setdefault(row, Seq(row=row))
                    eng.kv.set_pages(row, pg[len(s.pages):], len(s.pages))
                    s.pages = list(pg)
                eng.forward([SeqChunk(a, b, c, d) for a, b, c, d, _, _ in raw], mode, feedback=feedback)
            os._exit(0)
    else:
        raise SystemExit(f"unknown case {case}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
