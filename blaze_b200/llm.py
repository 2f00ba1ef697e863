"""Public offline API: ``LLM(...).generate(prompt_token_ids, params)``.

Builds the model (a local safetensors directory, or a named random-init shape), the engine and the
scheduler, and drives requests to completion.  The HTTP server uses the same three objects with the
scheduler running on its own thread.  Corresponds to the reference's ``Engine::load_with`` + ``Scheduler::start``
wiring in ``crates/blaze/src/main.rs:889-1078`` and its ``generate`` subcommand (:364-551).
"""
from __future__ import annotations

import os
import time
from typing import Dict, List, Optional, Sequence, Union

import torch

from . import log
from .config import ModelConfig, named_config
from .engine import Engine, EngineConfig
from .models.qwen3 import Model, TPInfo
from .quant import Format
from .sampler import SamplingParams
from .sched import Finish, GenEvent, GenRequest, SchedConfig, Scheduler


class RequestOutput:
    def __init__(self, request_id: str):
        self.request_id = request_id
        self.token_ids: List[int] = []
        self.logprobs: List[dict] = []
        self.finish_reason: Optional[str] = None
        self.error: Optional[str] = None
        self.prompt_tokens = 0
        self.cached_tokens = 0
        self.t_first = 0.0
        self.t_done = 0.0
        self.hidden = None


class LLM:
    def __init__(self, model: Union[str, ModelConfig, Model], *, weight_format: str = "dense", device: Optional[str] = None,
                 dtype=torch.bfloat16, tp=None, kv_cache_dtype: str = "auto", kv_tokens: int = 0, max_seqs: int = 256,
                 max_model_len: int = 4096, chunk: int = 2048, enable_prefix_caching: bool = True, cache_slots: int = 4,
                 use_graphs: bool = True, spec_method: str = "none", max_draft: int = 4, seed: int = 0,
                 eos_ids: Sequence[int] = (), drafter=None, max_step_tokens: int = 8192, warm_graphs: bool = False,
                 kv_host_tokens: int = 0, schedule: str = "interleave", kv_rotate: bool = False,
                 draft_tree_width: int = 1, draft_model: Optional[str] = None, draft_head_vocab: int = 0,
                 draft_tree_depth: int = 4, watchdog: bool = False, max_verify: int = 8, tune: bool = False,
                 stage_layers: Optional[tuple] = None, expert_heat: Union[str, bool, None] = None,
                 expert_placement: str = "contiguous", spec_fixed: bool = False):
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        tpi = tp if isinstance(tp, TPInfo) else TPInfo()
        fmt = {"dense": Format.DENSE, "bf16": Format.DENSE, "nvfp4": Format.NVFP4, "mxfp8": Format.MXFP8,
               "fp8_block": Format.FP8_BLOCK, "fp8": Format.FP8_CHANNEL}[weight_format]
        lo, hi = stage_layers if stage_layers is not None else (0, None)     # this rank's pipeline stage
        if expert_placement not in ("contiguous", "heat"):
            raise ValueError(f"unknown expert placement {expert_placement!r}")
        if expert_placement == "heat" and tpi.ep and tpi.world > 1 and tpi.expert_order is None and not isinstance(model, Model):
            # expert parallelism with the experts spread by the routing profile: every rank reads the same file
            from .expert_heat import ExpertHeat
            mc = model if isinstance(model, ModelConfig) else (ModelConfig.load(model) if os.path.isdir(model) else named_config(model))
            E = int(getattr(mc, "num_experts", 0) or 0)
            prof = ExpertHeat.load(expert_heat, mc.num_layers, E) if (E and isinstance(expert_heat, str)) else None
            if prof is not None and prof.longterm.sum() > 0 and E % tpi.world == 0:
                tpi.expert_order = ExpertHeat.order_for(prof.placement(tpi.world, recent=False))
                log.info("experts.placed", ranks=tpi.world, worst_before=float(prof.imbalance(tpi.world, recent=False).max()),
                         worst_after=float(prof.imbalance(tpi.world, prof.placement(tpi.world, recent=False), recent=False).max()))
            else:
                log.info("experts.placement_skipped", reason="no routing profile with observations for this model")
        with log.Stage("model"):
            if isinstance(model, Model):
                self.model = model
            elif isinstance(model, ModelConfig):
                self.model = Model.random_init(model, fmt, seed, self.device, dtype, tpi, first_layer=lo, last_layer=hi)
            elif os.path.isdir(model):
                self.model = Model.load(model, self.device, dtype, tpi, first_layer=lo, last_layer=hi)
            else:
                self.model = Model.random_init(named_config(model), fmt, seed, self.device, dtype, tpi, first_layer=lo, last_layer=hi)
        cfg = self.model.cfg
        self.heat = None
        if expert_heat:
            # routing statistics of a mixture-of-experts model: a path keeps the profile across restarts, True keeps it in memory
            from .expert_heat import attach as attach_heat
            self.heat = attach_heat(self.model, expert_heat if isinstance(expert_heat, str) else None)
            self._heat_writer = tpi.rank == 0          # the ranks of a stage see the same routing: one of them writes
        if tune and self.model.ops.is_cuda:
            # time the GEMM kernel variants of this model's layer shapes once per device (cached on disk) and route by the result
            from .tune import tune_model
            with log.Stage("tune"):
                tune_model(self.model, rows=sorted({min(max_seqs, 256), min(max_seqs, 64)}))
        if kv_cache_dtype == "auto":
            kv_cache_dtype = "fp8" if (self.device.type == "cuda" and self.model.ops.is_cuda) else \
                ("fp32" if dtype == torch.float32 else "bf16")
        if kv_cache_dtype.startswith("nvfp4") and self.model.ops.is_cuda:
            raise ValueError(f"kv_cache_dtype {kv_cache_dtype!r}: the attention kernels read FP8 pages; NVFP4 pages run on the oracle op set")
        with log.Stage("kv"):
            self.engine = Engine(self.model, EngineConfig(kv_tokens=kv_tokens, max_seqs=max_seqs, max_model_len=max_model_len,
                                                          kv_dtype=kv_cache_dtype, chunk=chunk, use_graphs=use_graphs,
                                                          kv_rotate=kv_rotate))
        eos = tuple(eos_ids) or tuple(cfg.eos_token_ids)
        if self.model.cfg.has_hc and (drafter is not None or spec_method in ("mtp", "eagle", "dflash")):
            # a drafter reads the target's hidden rows; a hyper-connection model hands out its streams instead
            raise ValueError("model drafters are not built for hyper-connection models: use --spec-method ngram or suffix")
        if drafter is None and spec_method in ("mtp", "eagle", "dflash"):
            from .models.drafter import build_drafter
            with log.Stage("drafter"):
                drafter = build_drafter(self.model, spec_method, model if isinstance(model, str) else None, draft_model,
                                        max_seqs, max_model_len, draft_head_vocab, seed + 7, draft_tree_width, draft_tree_depth)
        self.drafter = drafter
        if watchdog:
            self.engine.start_watchdog()
        self.sched = Scheduler(self.engine, SchedConfig(chunk=chunk, max_seqs=max_seqs, prefix_cache=enable_prefix_caching,
                                                        cache_slots=cache_slots, spec_method=spec_method, max_draft=max_draft,
                                                        draft_tree_width=draft_tree_width, max_verify=max_verify, spec_fixed=spec_fixed,
                                                        draft_tree_depth=draft_tree_depth,
                                                        eos_ids=eos, max_model_len=max_model_len,
                                                        max_step_tokens=max_step_tokens, kv_host_pages=kv_host_tokens // 16, schedule=schedule),
                               drafter=drafter)
        if self.heat is not None:
            # counters move to the host every 256 steps and the profile is written every 8192, on the scheduler's thread
            self.sched.housekeeping = ((256, self.heat.fold), (8192, self.save_expert_heat))
        if warm_graphs:
            with log.Stage("graphs"):
                self.engine.capture_decode_graphs()
        self._n = 0

    def save_expert_heat(self) -> None:
        """Fold the routing counters collected so far into the profile and write it back (no-op without ``expert_heat``)."""
        if self.heat is not None:
            if self.heat.path and self._heat_writer:
                self.heat.save()
            else:
                self.heat.fold()

    def generate(self, prompts: Sequence[Sequence[int]], params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 on_event=None) -> List[RequestOutput]:
        """Run ``prompts`` (lists of token ids) to completion; returns outputs in input order."""
        outs: Dict[str, RequestOutput] = {}
        order: List[str] = []

        def sink(ev: GenEvent):
            o = outs[ev.request_id]
            if ev.tokens:
                if not o.token_ids:
                    o.t_first = time.monotonic()
                o.token_ids.extend(ev.tokens)
            if ev.logprobs:
                o.logprobs.extend(ev.logprobs)
            if ev.hidden is not None:
                o.hidden = ev.hidden
            if ev.finish is not None:
                o.finish_reason, o.error, o.t_done = ev.finish.value, ev.error, time.monotonic()
            o.prompt_tokens, o.cached_tokens = ev.prompt_tokens, ev.cached_tokens
            if on_event:
                on_event(ev)

        for i, p in enumerate(prompts):
            sp = params[i] if isinstance(params, (list, tuple)) else (params or SamplingParams())
            rid = f"gen-{self._n}"
            self._n += 1
            outs[rid] = RequestOutput(rid)
            order.append(rid)
            self.sched.submit(GenRequest(rid, list(p), sp, sink=sink))
        self.sched.run_until_idle()
        return [outs[r] for r in order]

    def embed(self, prompts: Sequence[Sequence[int]]) -> List[torch.Tensor]:
        outs: Dict[str, RequestOutput] = {}
        order = []

        def sink(ev):
            if ev.hidden is not None:
                outs[ev.request_id].hidden = ev.hidden

        for p in prompts:
            rid = f"emb-{self._n}"
            self._n += 1
            outs[rid] = RequestOutput(rid)
            order.append(rid)
            self.sched.submit(GenRequest(rid, list(p), SamplingParams(max_tokens=1), embed_only=True, sink=sink))
        self.sched.run_until_idle()
        return [outs[r].hidden for r in order]
