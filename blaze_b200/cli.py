"""Command line: engine flags, service flags, ``--config`` files and presets, and the sub-commands.

Mirrors the reference's ``crates/blaze/src/main.rs`` (``EngineArgs`` :24-176, subcommands :364-551: serve, generate,
inspect, score, self-spec, stage-worker, vision-check) and ``crates/blaze/src/cli.rs`` (flat JSON ``--config`` where
explicit flags win and unknown keys fail :76; presets fast / balanced / quality :42-49).

    python -m blaze_b200 serve --model /path/to/checkpoint --tp 8 --kv-cache-dtype fp8 --spec-method mtp
    python -m blaze_b200 generate --model qwen3-8b --weights nvfp4 --prompt-ids 1,2,3 --max-tokens 16
    python -m blaze_b200 inspect --model /path/to/checkpoint
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Any, Dict, List, Optional, Sequence

PRESETS: Dict[str, Dict[str, Any]] = {
    # favour latency: shallow speculation, small prefill chunks
    "fast": {"chunk": 1024, "max_verify": 4, "draft_tree_depth": 3, "prompt_cache_slots": 2},
    "balanced": {"chunk": 2048, "max_verify": 8, "draft_tree_depth": 4, "prompt_cache_slots": 4},
    # favour throughput and cache reuse
    "quality": {"chunk": 4096, "max_verify": 8, "draft_tree_depth": 6, "prompt_cache_slots": 8, "kv_cache_dtype": "bf16"},
}


def engine_parser(p: argparse.ArgumentParser) -> None:
    g = p.add_argument_group("engine")
    g.add_argument("--model", required=False, help="checkpoint directory, or a named shape (tiny, qwen3-8b, …) for random init")
    g.add_argument("--weights", default=None, help="format for random-init shapes: dense | nvfp4 | mxfp8 | fp8_block | fp8")
    g.add_argument("--config", default=None, help="flat JSON file of flag values (explicit flags win; unknown keys fail)")
    g.add_argument("--preset", default=None, choices=sorted(PRESETS))
    g.add_argument("--max-model-len", type=int, default=None)
    g.add_argument("--kv-tokens", default="auto", help="KV capacity in tokens, or 'auto' (size from free memory)")
    g.add_argument("--schedule", default="interleave", choices=["interleave", "prefill_first"],
                   help="interleave: decode rows + one prefill chunk per step; prefill_first: prompts first, decode rows join "
                        "at most every 0.25 s while prompts are waiting")
    g.add_argument("--kv-host-tokens", type=int, default=0,
                   help="pinned host memory behind the prefix cache, in tokens: evicted snapshots wait there (0 = off)")
    g.add_argument("--expert-heat", default=None, metavar="PATH",
                   help="mixture-of-experts models: keep per-expert routing statistics in this profile file (loaded at start, "
                        "written back periodically and at exit; shown by the info route and `inspect --expert-heat`)")
    g.add_argument("--expert-placement", default="contiguous", choices=["contiguous", "heat"],
                   help="with --ep: which experts a rank holds.  contiguous: experts r*E/ranks ..; heat: spread by the routing "
                        "profile of --expert-heat (heaviest first onto the least loaded rank)")
    g.add_argument("--kv-cache-dtype", default=None, choices=["fp8", "bf16", "fp32", "nvfp4", "nvfp4_4over6", "auto"])
    g.add_argument("--kv-host", action="store_true", help="keep cold KV pages in pinned host memory")
    g.add_argument("--kv-rotate", action="store_true", help="randomised Hadamard rotation of q and k rows before the KV write")
    g.add_argument("--chunk", type=int, default=None, help="prefill tokens per iteration")
    g.add_argument("--vram-reserve", type=float, default=2.0, help="GiB kept free when sizing the KV pool")
    g.add_argument("--max-seqs", type=int, default=None)
    g.add_argument("--disable-prefix-caching", action="store_true")
    g.add_argument("--prompt-cache-slots", type=int, default=None)
    g.add_argument("--tp", type=int, default=1, help="tensor-parallel ranks (one process per GPU)")
    g.add_argument("--pp", type=int, default=1, help="pipeline stages")
    g.add_argument("--pp-chunk", type=int, default=512)
    g.add_argument("--ep", action="store_true", help="shard MoE experts across the tensor-parallel ranks")
    g.add_argument("--yarn-factor", type=float, default=None)
    g.add_argument("--draft-model", default=None, help="EAGLE / DFlash drafter checkpoint")
    g.add_argument("--mtp-model", default=None, help="checkpoint holding the MTP drafter's `mtp.*` tensors (default: the target's own)")
    # Flags of the reference engine whose job is done differently here.  Their neutral values are accepted so that launch
    # scripts carry over; any other value is refused with the reason (``check_compat``).
    c = p.add_argument_group("accepted for compatibility")
    c.add_argument("--gemm", default="auto", help="auto | nvfp4: the weight format decides the kernel here; bf16 (widened weights through a library GEMM) is not offered")
    c.add_argument("--attn-f16-acc", default="auto", help="auto | off: attention accumulates in fp32 in tensor memory")
    c.add_argument("--prefill-attention", default="auto", help="auto: one prefill attention kernel")
    c.add_argument("--verify-attention", default="auto", help="auto: verify rows go through the decode / row-block kernels")
    c.add_argument("--prefill-a16", default="none", help="none: activations follow the weight format on prefill as on decode")
    c.add_argument("--l2-prefetch-mib", type=float, default=None, help="0: there is no L2 weight prefetch between kernels")
    c.add_argument("--draft-head-vram", default="auto", help="auto | on: a drafter's LM head is always in device memory")
    c.add_argument("--pp-remote", default=None, help="not offered: pipeline stages are ranks of one torch.distributed job")
    c.add_argument("--ple-threads", type=int, default=None, help="accepted and unused: the n-gram embedding tables (PLE) live in device memory, no host threads read them")
    c.add_argument("--ple-cache-gib", type=float, default=None, help="accepted and unused: the PLE tables live in device memory, there is no host row cache")
    g.add_argument("--spec-method", default=None, choices=["none", "ngram", "suffix", "mtp", "eagle", "dflash"])
    g.add_argument("--max-verify", type=int, default=None)
    g.add_argument("--suffix-assist", action="store_true")
    g.add_argument("--mtp-window", type=int, default=8192)
    g.add_argument("--mtp-head-vocab", type=int, default=0)
    g.add_argument("--mtp-head-cands", type=int, default=32768)
    g.add_argument("--draft-tree-width", type=int, default=1)
    g.add_argument("--draft-tree-depth", type=int, default=None)
    g.add_argument("--no-graphs", action="store_true")
    g.add_argument("--tune", action="store_true",
                   help="time the GEMM kernel variants for this model's layer shapes at start-up (cached per device under "
                        "~/.cache/blaze_b200) and route each linear layer to the measured winner")
    g.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--device", default=None)


def service_parser(p: argparse.ArgumentParser) -> None:
    g = p.add_argument_group("service")
    g.add_argument("--host", default="127.0.0.1")
    g.add_argument("--port", type=int, default=8000)
    g.add_argument("--api-key", action="append", default=None)
    g.add_argument("--served-model-name", default=None)
    g.add_argument("--print-config", action="store_true", help="print the effective configuration (API keys redacted) and exit "
                                                               "without loading a model")
    g.add_argument("--api-key-file", default=None, help="file with one API key per line (blank lines ignored)")
    g.add_argument("--max-queue", "--max-queued-requests", dest="max_queue", type=int, default=1024,
                   help="most accepted generations, queued ones included; beyond it requests get 429")
    g.add_argument("--max-concurrency", "--max-concurrent-requests", dest="max_concurrency", type=int, default=512,
                   help="most HTTP requests in flight, their streaming bodies included")
    g.add_argument("--request-timeout", type=float, default=600.0)
    g.add_argument("--shutdown-timeout", type=float, default=10.0, help="longest graceful drain after SIGINT / SIGTERM, seconds")
    g.add_argument("--max-request-body-mib", type=int, default=64)
    g.add_argument("--allowed-origins", default="*", help="allowed CORS origins, comma separated; '*' allows all, 'none' disables CORS")
    g.add_argument("--log-color", default="auto", choices=["auto", "always", "never"])
    g.add_argument("--disable-log-requests", action="store_true", help="no per-request lifecycle log lines (metrics continue)")
    g.add_argument("--log-inputs", action="store_true", help="log bounded previews of request payloads")
    g.add_argument("--log-outputs", action="store_true", help="log bounded previews of response payloads")
    g.add_argument("--max-log-len", type=int, default=400, help="most characters of a payload preview")
    g.add_argument("--log-stats-interval", type=float, default=5.0, help="seconds between scheduler summaries; 0 disables them")
    g.add_argument("--override-generation-config", default=None, metavar="JSON",
                   help="sampling defaults over --generation-config (explicit flags and request parameters win)")
    g.add_argument("--instruct-sampling", default=None, metavar="JSON",
                   help="sampling defaults of chat requests with thinking off, over the defaults above, e.g. "
                        "'{\"temperature\":0.7,\"top_p\":0.8,\"presence_penalty\":1.5}'")
    g.add_argument("--frequency-penalty", type=float, default=None)
    g.add_argument("--repetition-penalty", type=float, default=None)
    g.add_argument("--min-tokens", type=int, default=None)
    g.add_argument("--default-max-tokens", type=int, default=512)
    g.add_argument("--log-level", default="info")
    g.add_argument("--log-format", default="text", choices=["text", "json"])
    g.add_argument("--profile-prefill", action="store_true")
    g.add_argument("--generation-config", default=None)
    g.add_argument("--samplers", default=None, help="default sampler stage order, e.g. penalties,temperature,top_k,top_p")
    g.add_argument("--top-nsigma", type=float, default=None)
    g.add_argument("--top-h", type=float, default=None)
    g.add_argument("--tool-call-parser", default="hermes")
    g.add_argument("--reasoning-parser", default="qwen3")
    g.add_argument("--chat-family", default=None, choices=["chatml", "deepseek", "glm", "kimi"])
    g.add_argument("--temperature", type=float, default=None, help="default sampling of requests that do not set it (also --top-p, "
                                                                     "--top-k, --min-p, --presence-penalty)")
    g.add_argument("--top-p", type=float, default=None)
    g.add_argument("--top-k", type=int, default=None)
    g.add_argument("--min-p", type=float, default=None)
    g.add_argument("--presence-penalty", type=float, default=None)
    g.add_argument("--max-tokens", type=int, default=None, help="default max_tokens of chat requests (same as --default-max-tokens)")
    g.add_argument("--step-tokens", "--max-num-batched-tokens", dest="step_tokens", type=int, default=None,
                   help="tokens of one step (decode tokens + the prefill chunk)")
    g.add_argument("--spec-ngram", type=int, default=None, help="draft tokens per verify of the n-gram / suffix drafts, 0 off")
    g.add_argument("--spec-fixed", action="store_true", help="always verify the whole draft (by default drafts are cut or skipped "
                                                             "by the measured verify cost)")
    g.add_argument("--thinking-budget", type=int, default=None,
                   help="default thinking budget in tokens of chat requests (requests override it with thinking_token_budget)")
    g.add_argument("--vision", default="auto", choices=["auto", "gpu", "cpu", "off"], help="where the vision tower runs; off: no image input")
    g.add_argument("--vision-threads", type=int, default=None, help="CPU threads of a vision tower that runs on the CPU")
    g.add_argument("--mm-encoder-batch", type=int, default=None,
                   help="most images in one pass of the vision tower: 0 (the reference's auto) or 1; images are encoded one at a time here")
    g.add_argument("--mm-encoder-patches", type=int, default=None,
                   help="patch budget of one pass of the vision tower: accepted and unused, a pass encodes one image whatever its size")
    g.add_argument("--mm-processor-kwargs", default=None, metavar="JSON",
                   help="image processor settings over the checkpoint's (min_pixels, max_pixels, size.shortest_edge / longest_edge); "
                        "requests override them with mm_processor_kwargs")
    g.add_argument("--limit-mm-per-prompt", default="", help="most images per request, as JSON ({\"image\": 4}) or image=4")
    g.add_argument("--mm-low-detail-pixels", type=int, default=512 * 512,
                   help="image_url.detail \"low\": cap of the image's pixels; 0 ignores detail")
    g.add_argument("--image-fetch-timeout", type=float, default=5.0, help="seconds the http(s) image downloads of one request may take")
    g.add_argument("--image-fetch-max-mib", type=int, default=64, help="largest image fetched from an http(s) URL, MiB")
    g.add_argument("--allowed-media-domains", default="", help="hosts http(s) image URLs may name, comma separated (default: any)")
    g.add_argument("--grammar-whitespace", type=int, default=64,
                   help="longest white-space run between JSON tokens of structured outputs, characters (0: unbounded; requests "
                        "override it with whitespace_pattern or disable_any_whitespace)")
    g.add_argument("--chat-template", default=None, metavar="FILE",
                   help="Jinja chat template to use instead of the checkpoint's (a file path)")
    g.add_argument("--chat-template-kwargs", default=None, metavar="JSON",
                   help="default template arguments (e.g. '{\"thinking\": true}'); a request's chat_template_kwargs override them")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="blaze_b200")
    sub = ap.add_subparsers(dest="command", required=True)
    s = sub.add_parser("serve", help="start the HTTP server")
    engine_parser(s)
    service_parser(s)
    g = sub.add_parser("generate", help="generate from token ids or text and print the result")
    engine_parser(g)
    g.add_argument("--prompt", default=None)
    g.add_argument("--prompt-ids", default=None, help="comma-separated token ids")
    g.add_argument("--max-tokens", type=int, default=32)
    g.add_argument("--temperature", type=float, default=0.0)
    i = sub.add_parser("inspect", help="list checkpoint tensors and their formats; with --expert-heat, report a routing profile")
    i.add_argument("--model", required=True, help="checkpoint directory (or a named shape with --expert-heat)")
    i.add_argument("--expert-heat", default=None, metavar="PATH", help="routing profile written by a run with --expert-heat")
    i.add_argument("--ranks", type=int, default=8, help="expert-parallel ranks the placement report is computed for")
    sc = sub.add_parser("score", help="per-token log-probabilities of a token sequence")
    engine_parser(sc)
    sc.add_argument("--prompt-ids", required=True)
    ss = sub.add_parser("self-spec", help="test of the verify / commit path: greedy decode, then the same continuation through "
                                          "verify rounds whose drafts are that decode with a wrong token every few positions")
    engine_parser(ss)
    ss.add_argument("--prompt", default=None)
    ss.add_argument("--prompt-ids", default=None, help="comma-separated token ids")
    ss.add_argument("--max-tokens", type=int, default=96)
    ss.add_argument("--draft", type=int, default=7, help="draft tokens per round")
    et = sub.add_parser("eagle-test", help="drafter test (needs --spec-method mtp / eagle / dflash or --draft-model): greedy decode, "
                                           "then the same prompt through draft + verify rounds; prints accepted tokens per round, "
                                           "the speed of both and where the outputs part")
    engine_parser(et)
    et.add_argument("--prompt", default=None)
    et.add_argument("--prompt-ids", default=None, help="comma-separated token ids")
    et.add_argument("--max-tokens", type=int, default=200)
    et.add_argument("--draft", type=int, default=6, help="draft tokens per round")
    w = sub.add_parser("stage-worker", help="serve one pipeline stage for a remote coordinator")
    engine_parser(w)
    w.add_argument("--listen", default="127.0.0.1:7000")
    w.add_argument("--stage", type=int, default=1)
    v = sub.add_parser("vision-check", help="compare the CUDA vision tower with the CPU tower on an image")
    v.add_argument("--model", required=True)
    v.add_argument("--image", required=True)
    return ap


def resolve(argv: Sequence[str]) -> argparse.Namespace:
    """Parse ``argv``; layer preset < config file < explicit flags (``cli.rs:76``)."""
    ap = build_parser()
    ns = ap.parse_args(list(argv))
    explicit = set()
    for a in argv:
        if a.startswith("--"):
            explicit.add(a[2:].split("=")[0].replace("-", "_"))
    layered: Dict[str, Any] = {}
    if getattr(ns, "preset", None):
        layered.update(PRESETS[ns.preset])
    if getattr(ns, "config", None):
        with open(ns.config) as f:
            cfg = json.load(f)
        if not isinstance(cfg, dict):
            raise SystemExit("--config must hold a JSON object")
        for k, v in cfg.items():
            key = k.replace("-", "_")
            if not hasattr(ns, key):
                raise SystemExit(f"--config: unknown key {k!r}")
            layered[key] = v
    for k, v in layered.items():
        if k not in explicit and hasattr(ns, k):
            setattr(ns, k, v)
    return ns


_COMPAT = {
    # flag attribute: (accepted values, why anything else is refused)
    "gemm": (("auto", "nvfp4"), "the GEMM kernel follows the weight format; there is no widened-weight library path"),
    "attn_f16_acc": (("auto", "off"), "attention accumulates in fp32 (tensor memory); there is no fp16 accumulation mode"),
    "prefill_attention": (("auto",), "there is one prefill attention kernel"),
    "verify_attention": (("auto",), "verify rows use the decode / row-block attention kernels; there are no alternatives to pick"),
    "prefill_a16": (("none",), "prefill quantises activations like decode does; 16-bit prefill inputs are not built"),
    "l2_prefetch_mib": ((None, 0, 0.0), "there is no L2 weight prefetch between kernels"),
    "draft_head_vram": (("auto", "on"), "a drafter's LM head always lives in device memory"),
    "mm_encoder_batch": ((None, 0, 1), "the vision tower encodes one image per pass; passes over several images are not built"),
    "pp_remote": ((None,), "pipeline stages are ranks of one torch.distributed job: launch every stage with torch.distributed.run "
                           "(--nnodes / --node-rank for several machines) and --pp"),
}


def check_compat(ns: argparse.Namespace) -> None:
    """Refuse, with the reason, a reference-engine flag set to something this engine cannot honour."""
    for attr, (ok, why) in _COMPAT.items():
        v = getattr(ns, attr, ok[0])
        if v not in ok:
            raise SystemExit(f"--{attr.replace('_', '-')} {v}: {why}")
    if getattr(ns, "mtp_model", None):
        if getattr(ns, "spec_method", None) not in (None, "mtp"):
            raise SystemExit("--mtp-model goes with --spec-method mtp")
        if getattr(ns, "draft_model", None) and ns.draft_model != ns.mtp_model:
            raise SystemExit("--mtp-model and --draft-model name different checkpoints")
        ns.spec_method, ns.draft_model = "mtp", ns.mtp_model


def spec_defaults(ns: argparse.Namespace) -> None:
    """``--spec-method mtp`` implies its window / candidate settings; PP with a drafter is refused (``main.rs:203-254``)."""
    if getattr(ns, "spec_method", None) in (None, "none") and getattr(ns, "draft_model", None):
        ns.spec_method = "eagle"
    if getattr(ns, "spec_method", None) in ("mtp", "eagle", "dflash") and getattr(ns, "pp", 1) > 1:
        raise SystemExit("pipeline parallelism cannot be combined with a drafter")
    if getattr(ns, "max_verify", None) is None:
        ns.max_verify = 8
    if getattr(ns, "draft_tree_depth", None) is None:
        ns.draft_tree_depth = 4


def build_llm(ns: argparse.Namespace):
    import torch
    from .llm import LLM
    from .models.qwen3 import TPInfo
    from .parallel.tp import TPGroup
    check_compat(ns)
    spec_defaults(ns)
    device = ns.device or ("cuda" if torch.cuda.is_available() else "cpu")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if ns.tp > 1 and world != ns.tp * max(getattr(ns, "pp", 1), 1):
        raise SystemExit(f"--tp {ns.tp}: launch one process per GPU, e.g. python -m torch.distributed.run "
                         f"--nproc-per-node {ns.tp} --master-addr 127.0.0.1 -m blaze_b200 …")
    group = None
    pp = max(int(getattr(ns, "pp", 1) or 1), 1)
    if world > 1:
        local = int(os.environ.get("LOCAL_RANK", "0"))
        if device.startswith("cuda"):
            torch.cuda.set_device(local)
            device = f"cuda:{local}"
        group = TPGroup.from_env(device, pp=pp)
    tp = TPInfo(group.rank, group.world, group if group.world > 1 else None, ep=ns.ep) if group else TPInfo()
    kv = ns.kv_cache_dtype or "auto"
    if kv.startswith("nvfp4") and device.startswith("cuda"):
        raise SystemExit(f"--kv-cache-dtype {kv}: the attention kernels read FP8 pages; NVFP4 pages (plain or 4-over-6 scales) are "
                         "written and read by the oracle op set only (--device cpu).  Use fp8 (the compact format here), bf16 or fp32")
    if getattr(ns, "kv_host", False):
        raise SystemExit("--kv-host (live sequences in pinned host memory) is not built; --kv-host-tokens N gives the prefix "
                         "cache a pinned-host tier of N tokens")
    if getattr(ns, "pp", 1) > 1 and world != ns.pp * max(ns.tp, 1):
        raise SystemExit(f"--pp {ns.pp} --tp {ns.tp}: launch {ns.pp * max(ns.tp, 1)} processes (one per GPU), e.g. python -m "
                         f"torch.distributed.run --nproc-per-node {ns.pp * max(ns.tp, 1)} --master-addr 127.0.0.1 -m blaze_b200 …")
    kv_tokens = 0 if str(ns.kv_tokens) == "auto" else int(ns.kv_tokens)
    spec_ngram = getattr(ns, "spec_ngram", None)           # draft tokens per verify; 0 switches speculation off
    stage_range = None
    if group is not None and group.stages > 1:
        from .config import ModelConfig, named_config
        from .parallel.pp import stage_layers
        mcfg = ModelConfig.load(ns.model) if (ns.model and os.path.isdir(ns.model)) else named_config(ns.model or "tiny")
        stage_range = stage_layers(mcfg.num_layers, group.stages, group.stage)
    llm = LLM(ns.model or "tiny", weight_format=ns.weights or "dense", device=device, tp=tp, kv_cache_dtype=kv,
              stage_layers=stage_range,
              kv_tokens=kv_tokens, max_seqs=ns.max_seqs or 256, max_model_len=ns.max_model_len or 4096,
              chunk=ns.chunk or 2048, enable_prefix_caching=not ns.disable_prefix_caching,
              cache_slots=ns.prompt_cache_slots or 4, use_graphs=not ns.no_graphs,
              spec_method=("none" if spec_ngram == 0 else ns.spec_method or "none"),
              max_draft=min(ns.max_verify - 1, 8) if not spec_ngram else max(1, min(int(spec_ngram), ns.max_verify - 1)), seed=ns.seed,
              spec_fixed=bool(getattr(ns, "spec_fixed", False)),
              **({"max_step_tokens": int(ns.step_tokens)} if getattr(ns, "step_tokens", None) else {}),
              kv_host_tokens=getattr(ns, "kv_host_tokens", 0) or 0, schedule=getattr(ns, "schedule", "interleave"), kv_rotate=bool(getattr(ns, "kv_rotate", False)),
              draft_tree_width=int(getattr(ns, "draft_tree_width", 1) or 1),
              tune=bool(getattr(ns, "tune", False)), draft_model=getattr(ns, "draft_model", None), draft_head_vocab=int(getattr(ns, "mtp_head_vocab", 0) or 0),
              draft_tree_depth=int(ns.draft_tree_depth or 4), max_verify=int(ns.max_verify or 8),
              expert_heat=getattr(ns, "expert_heat", None), expert_placement=getattr(ns, "expert_placement", "contiguous"))
    llm.group = group
    if group is not None:
        from .parallel.worker import attach
        attach(llm, group, int(getattr(ns, "pp_chunk", 512) or 512))
    if group is not None and group.world > 1 and ns.comm == "fused" and device.startswith("cuda"):
        from .parallel.symm import SymmAllReduce
        group.fused = SymmAllReduce.create(group, device, max_rows=(ns.chunk or 2048) + (ns.max_seqs or 256) + 64,
                                           hidden=llm.model.cfg.hidden_size)
    return llm


def main(argv: Optional[Sequence[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    ns = resolve(argv)
    from . import log
    if hasattr(ns, "log_level"):
        color = {"always": True, "never": False}.get(getattr(ns, "log_color", "auto"))      # auto: a terminal decides
        log.configure(level=ns.log_level, fmt=ns.log_format, color=color)
    if ns.command == "inspect":
        if getattr(ns, "expert_heat", None):
            from .inspect import inspect_expert_heat
            return inspect_expert_heat(ns.model, ns.expert_heat, ns.ranks)
        from .inspect import inspect_checkpoint
        return inspect_checkpoint(ns.model)
    if ns.command == "serve":
        from .server.run import serve
        return serve(ns)
    if ns.command == "eagle-test":
        ns.max_draft = ns.draft
        if getattr(ns, "spec_method", "none") in (None, "none") and not getattr(ns, "draft_model", None):
            print("eagle-test needs --spec-method mtp / eagle / dflash or --draft-model", file=sys.stderr)
            return 2
    if ns.command in ("generate", "score", "self-spec", "eagle-test"):
        llm = build_llm(ns)
        grp = getattr(llm, "group", None)
        if grp is not None and grp.global_rank != 0:
            from .parallel.worker import follow
            return follow(llm)            # the other ranks execute the steps that rank 0 plans
        try:
            return _run_offline(ns, llm)
        finally:
            if getattr(llm, "leader", None) is not None:
                llm.leader.quit()
    if ns.command == "stage-worker":
        from .remote import serve_stage
        return serve_stage(ns)
    if ns.command == "vision-check":
        from .models.vision import check_reference
        return check_reference(ns.model, ns.image)
    return 2


def _run_offline(ns, llm) -> int:
    if ns.command == "generate":
        from .sampler import SamplingParams
        from .text import load_tokenizer
        tok = load_tokenizer(ns.model if ns.model and os.path.isdir(ns.model) else None, llm.model.cfg.vocab_size)
        ids = [int(x) for x in ns.prompt_ids.split(",")] if ns.prompt_ids else tok.encode(ns.prompt or "hello")
        out = llm.generate([ids], SamplingParams(temperature=ns.temperature, max_tokens=ns.max_tokens))[0]
        print(json.dumps({"token_ids": out.token_ids, "text": tok.decode(out.token_ids), "finish_reason": out.finish_reason}))
        return 0
    if ns.command in ("self-spec", "eagle-test"):
        from .text import load_tokenizer
        tok = load_tokenizer(ns.model if ns.model and os.path.isdir(ns.model) else None, llm.model.cfg.vocab_size)
        ids = [int(x) for x in ns.prompt_ids.split(",")] if ns.prompt_ids else tok.encode(ns.prompt or "hello")
        return self_spec(llm, ids, ns.max_tokens, ns.draft) if ns.command == "self-spec" else eagle_test(llm, ids, ns.max_tokens)
    if ns.command == "score":
        import torch
        ids = [int(x) for x in ns.prompt_ids.split(",")]
        s = llm.engine.open_from()
        logits = llm.engine.forward(llm.engine.plan([(s, ids, len(ids))]), "logits")
        lp = torch.log_softmax(logits.float(), -1)
        scores = [float(lp[i, ids[i + 1]]) for i in range(len(ids) - 1)]
        print(json.dumps({"logprobs": scores, "sum": sum(scores)}))
        return 0
    return 2


def self_spec(llm, ids, max_tokens: int, draft: int) -> int:
    """Greedy reference decode through the engine, then the same continuation through verify rounds whose drafts are the
    reference with a wrong token at pseudo-random places; accepted rows are committed, rejected ones truncated.  Prints how
    many tokens match (reference: ``Command::SelfSpec``, crates/blaze/src/main.rs:831-880)."""
    import time
    eng = llm.engine
    vocab = llm.model.cfg.vocab_size

    def prefill():
        s = eng.open_from()
        return s, int(eng.forward(eng.plan([(s, ids, 1)]), "greedy")[0])
    s, first = prefill()
    reference = [first]
    t0 = time.perf_counter()
    while len(reference) < max_tokens:
        reference.append(int(eng.forward(eng.plan([(s, [reference[-1]], 1)]), "greedy")[0]))
    plain = (max_tokens - 1) / max(time.perf_counter() - t0, 1e-9)
    eng.close(s)
    s, first = prefill()
    out, rounds, lcg = [first], 0, 12345
    t0 = time.perf_counter()
    while len(out) < max_tokens:
        pos = len(out)
        drafts = [reference[pos + j] if pos + j < len(reference) else 0 for j in range(draft)]
        lcg = (lcg * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        wrong = (lcg >> 33) % (draft + 3)
        if wrong < draft:
            drafts[wrong] = (drafts[wrong] + 1) % min(vocab, 1000)
        rows = [out[-1]] + drafts
        base = s.length
        picks = eng.forward(eng.plan([(s, rows, len(rows))], defer_state=True), "greedy").tolist()
        acc = 0
        while acc < draft and picks[acc] == drafts[acc]:
            acc += 1
        out.extend(int(t) for t in picks[:acc + 1])
        if eng.kv.gdn_layers:
            eng.commit_state([(s, acc + 1)])
        eng.truncate(s, base + acc + 1)
        rounds += 1
    dt = max(time.perf_counter() - t0, 1e-9)
    out = out[:max_tokens]
    same = next((i for i, (a, b) in enumerate(zip(out, reference)) if a != b), min(len(out), len(reference)))
    eng.close(s)
    print(f"{same}/{max_tokens} tokens match the reference; {rounds} rounds ({len(out) / max(rounds, 1):.2f} tokens per round, "
          f"{len(out) / dt:.1f} tok/s; plain decode {plain:.1f} tok/s)")
    return 0 if same == max_tokens else 1


def eagle_test(llm, ids, max_tokens: int) -> int:
    """Greedy decode without the drafter, then the same prompt through the scheduler's draft + verify rounds; prints the
    accepted tokens per round, both speeds and the first position where the outputs part (near-ties may flip between step
    shapes).  Reference: ``Command::EagleTest``, crates/blaze/src/main.rs:692-830."""
    import time
    from .sampler import SamplingParams
    sp = SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)
    sched = llm.sched
    drafter, method = sched.drafter, sched.cfg.spec_method
    sched.drafter, sched.cfg.spec_method = None, "none"
    t0 = time.perf_counter()
    plain = llm.generate([ids], sp)[0].token_ids
    t_plain = time.perf_counter() - t0
    sched.drafter, sched.cfg.spec_method = drafter, method
    sched.cache.clear()
    d0, a0, s0 = sched.stats.draft_tokens, sched.stats.accepted_tokens, sched.stats.steps
    t0 = time.perf_counter()
    spec = llm.generate([ids], sp)[0].token_ids
    t_spec = time.perf_counter() - t0
    drafted, accepted, rounds = sched.stats.draft_tokens - d0, sched.stats.accepted_tokens - a0, sched.stats.steps - s0
    same = next((i for i, (a, b) in enumerate(zip(spec, plain)) if a != b), min(len(spec), len(plain)))
    print(json.dumps({"tokens": len(spec), "match_until": same, "rounds": rounds, "drafted": drafted, "accepted": accepted,
                      "accepted_per_round": accepted / max(rounds, 1), "plain_tok_s": len(plain) / max(t_plain, 1e-9),
                      "spec_tok_s": len(spec) / max(t_spec, 1e-9), "drafter": method}))
    return 0
