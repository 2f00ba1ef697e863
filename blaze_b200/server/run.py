"""``serve``: bind the port first (503 ``model_loading`` with the load stage while the model loads), load the model on a
worker thread, then attach it; graceful shutdown on SIGINT / SIGTERM (reference: ``crates/blaze/src/main.rs:889-1078``,
``server.rs:177-245`` early listener, ``server.rs:340-351`` shutdown)."""
from __future__ import annotations

import os
import threading

from .. import log
from ..service import ServiceArgs
from .app import ServerState, create_app


def service_args_of(ns) -> ServiceArgs:
    from .media import parse_limit
    try:
        limit = parse_limit(getattr(ns, "limit_mm_per_prompt", ""))
    except ValueError as e:
        raise SystemExit(str(e))
    svc = _service_args(ns)
    svc.limit_mm_per_prompt = limit
    svc.thinking_budget = getattr(ns, "thinking_budget", None)
    svc.vision, svc.vision_threads = getattr(ns, "vision", "auto"), getattr(ns, "vision_threads", None)
    svc.mm_processor_kwargs = _json_object(getattr(ns, "mm_processor_kwargs", None), "--mm-processor-kwargs")
    svc.mm_low_detail_pixels = int(getattr(ns, "mm_low_detail_pixels", 512 * 512))
    svc.image_fetch_timeout = float(getattr(ns, "image_fetch_timeout", 5.0))
    svc.image_fetch_max_mib = int(getattr(ns, "image_fetch_max_mib", 64))
    svc.allowed_media_domains = tuple(d.strip().lower() for d in (getattr(ns, "allowed_media_domains", "") or "").split(",") if d.strip())
    if getattr(ns, "max_tokens", None):
        svc.default_max_tokens = int(ns.max_tokens)
    from ..service import merge_sampling
    try:
        # order of precedence, lowest first: generation_config.json, --override-generation-config, explicit flags
        gc = getattr(ns, "generation_config", None)
        if gc in (None, "auto") and getattr(ns, "model", None) and os.path.isdir(ns.model):
            auto = os.path.join(ns.model, "generation_config.json")
            if os.path.isfile(auto):
                svc.read_generation_config(auto)
        merge_sampling(svc.defaults, _json_object(getattr(ns, "override_generation_config", None), "--override-generation-config"),
                       "--override-generation-config")
        merge_sampling(svc.instruct_sampling, _json_object(getattr(ns, "instruct_sampling", None), "--instruct-sampling"),
                       "--instruct-sampling")
    except ValueError as e:
        raise SystemExit(str(e))
    for flag in ("temperature", "top_p", "top_k", "min_p", "presence_penalty", "frequency_penalty", "repetition_penalty", "min_tokens"):
        v = getattr(ns, flag, None)
        if v is not None:
            svc.defaults[flag] = v
    keys = list(svc.api_keys)
    if getattr(ns, "api_key_file", None):
        with open(ns.api_key_file) as f:
            keys += [ln.strip() for ln in f if ln.strip()]
    svc.api_keys = tuple(keys)
    origins = (getattr(ns, "allowed_origins", "*") or "*").strip()
    svc.cors_origins = () if origins == "none" else tuple(o.strip() for o in origins.split(",") if o.strip())
    svc.shutdown_timeout = float(getattr(ns, "shutdown_timeout", 10.0))
    svc.max_request_body_mib = int(getattr(ns, "max_request_body_mib", 64))
    svc.log_requests = not getattr(ns, "disable_log_requests", False)
    svc.log_inputs, svc.log_outputs = bool(getattr(ns, "log_inputs", False)), bool(getattr(ns, "log_outputs", False))
    svc.max_log_len = int(getattr(ns, "max_log_len", 400))
    svc.log_stats_interval = float(getattr(ns, "log_stats_interval", 5.0))
    return svc


def _service_args(ns) -> ServiceArgs:
    return ServiceArgs(host=ns.host, port=ns.port, api_keys=tuple(ns.api_key or ()), served_model_name=ns.served_model_name,
                       max_queue=ns.max_queue, max_concurrency=ns.max_concurrency, request_timeout_s=ns.request_timeout,
                       default_max_tokens=ns.default_max_tokens, log_level=ns.log_level, log_format=ns.log_format,
                       profile_prefill=ns.profile_prefill, generation_config=ns.generation_config, samplers=ns.samplers,
                       top_nsigma=ns.top_nsigma, top_h=ns.top_h, tool_call_parser=ns.tool_call_parser,
                       reasoning_parser=ns.reasoning_parser or None,
                       chat_family=getattr(ns, "chat_family", None), grammar_whitespace=int(getattr(ns, "grammar_whitespace", 64)),
                       chat_template_kwargs=_json_object(getattr(ns, "chat_template_kwargs", None), "--chat-template-kwargs"))


def _json_object(text, flag):
    if not text:
        return {}
    import json
    try:
        v = json.loads(text)
    except ValueError as e:
        raise SystemExit(f"{flag}: not JSON ({e})")
    if not isinstance(v, dict):
        raise SystemExit(f"{flag}: expected a JSON object")
    return v


def serve(ns) -> int:
    import uvicorn
    from ..cli import build_llm
    from ..text import load_tokenizer
    svc = service_args_of(ns)
    if getattr(ns, "print_config", False):
        import json
        engine = {k: v for k, v in sorted(vars(ns).items()) if not k.startswith("_") and k not in ("api_key", "command")}
        print(json.dumps({"service": svc.public_config(), "flags": engine}, indent=1, default=str))
        return 0
    name = os.path.basename(os.path.normpath(ns.model)) if ns.model else "blaze"
    st = ServerState(svc, name)
    app = create_app(st)
    rank = int(os.environ.get("RANK", "0"))

    def load():
        try:
            llm = build_llm(ns)
            st.leader = getattr(llm, "leader", None)       # build_llm attached the step protocol when there are other ranks
            tok = load_tokenizer(ns.model if ns.model and os.path.isdir(ns.model) else None, llm.model.cfg.vocab_size)
            if getattr(ns, "chat_template", None):
                with open(ns.chat_template, encoding="utf-8") as f:
                    tok.chat_template = f.read()
            vision = None
            if llm.model.cfg.vision_config and ns.model and os.path.isdir(ns.model) and svc.vision != "off":
                from ..models.vision import Vision
                with log.Stage("vision"):
                    if svc.vision == "cpu" and svc.vision_threads:
                        import torch
                        torch.set_num_threads(int(svc.vision_threads))
                    vision = Vision.load(ns.model, "cpu" if svc.vision == "cpu" else llm.device)
            st.attach(llm, tok, vision)
            log.info("server.ready", model=st.model_name, port=svc.port)
        except Exception as e:
            log.error("server.load_failed", error=repr(e))
            os._exit(101)

    if rank != 0:
        # non-zero ranks execute the step plans that rank 0 broadcasts
        llm = build_llm(ns)
        from ..parallel.worker import follow
        return follow(llm)
    threading.Thread(target=load, name="blaze-load", daemon=True).start()
    config = uvicorn.Config(app, host=svc.host, port=svc.port, log_level="warning", timeout_graceful_shutdown=max(int(svc.shutdown_timeout), 1))
    server = uvicorn.Server(config)

    @app.on_event("shutdown")
    async def _shutdown():
        st.shutting_down = True
        if st.llm is not None:
            st.llm.sched.stop()
            st.llm.save_expert_heat()
    server.run()
    return 0
