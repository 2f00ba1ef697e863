"""OpenAI-compatible HTTP API (FastAPI): chat/completions, completions, embeddings, Responses, Anthropic Messages,
tokenize / detokenize, models, health, metrics, server info.

Route list and behaviour follow the reference's ``crates/blaze/src/server.rs:282-301`` and ``server/*.rs``:
early 503 ``model_loading`` body with the current load stage while the model loads (:177-245), auth by Bearer or
``x-api-key`` (``server/control.rs:44``), request id / CORS / semaphore admission / deadline middleware (:100), SSE
streaming with ``[DONE]``, usage accounting, Prometheus text at ``/metrics`` (:360-406), an in-memory store of the
last 256 Responses objects (``server/responses.rs``).
"""
from __future__ import annotations

import asyncio
import contextvars
import base64
import hmac
import json
import struct
import time
import uuid
from collections import OrderedDict
from typing import Any, AsyncIterator, Dict, List, Optional

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from .. import __version__, log
from ..chat import ChatFormatter, ChatResponseProcessor, get_think_parser, get_tool_parser
from ..sampler import SamplingParams
from ..sched import Finish, GenEvent, GenRequest, ThinkBudget
from . import messages as anth
from . import responses as rsp
from ..service import (MAX_COMPLETIONS_PER_REQUEST, RequestError, ServiceArgs, sampling_of, stop_strings_of,
                       thinking_budget_of)
from ..structured import forced_call_grammar, ConstraintError, Grammars, grammar_of
from ..telemetry import Histogram

RESPONSES_KEPT = 256
THINK_CLOSING = "\n\nConsidering the limited time, I have to give the solution based on the thinking directly now.\n</think>\n\n"


# the HTTP request being served (set by the middleware): generations poll it to notice a client that went away
_current_request: "contextvars.ContextVar[Optional[Request]]" = contextvars.ContextVar("blaze_current_request", default=None)


def _err(status: int, message: str, typ: str = "invalid_request_error", param=None, code=None) -> JSONResponse:
    """An error in the OpenAI shape; on the Messages routes in Anthropic's (``server/messages.rs:13``)."""
    req = _current_request.get()
    if req is not None and req.url.path.startswith("/v1/messages"):
        return JSONResponse(anth.error_body(status, message), status_code=status)
    return JSONResponse({"error": {"message": message, "type": typ, "param": param, "code": code}}, status_code=status)


class Totals:
    def __init__(self):
        self.requests = self.errors = self.prompt_tokens = self.cached_tokens = self.output_tokens = 0
        self.e2e = Histogram.latency()
        self.inflight = 0
        self.cancelled = 0


class ServerState:
    """Everything the handlers need.  ``llm`` is None while the model is loading."""

    def __init__(self, svc: ServiceArgs, model_name: str = "blaze"):
        self.svc, self.model_name = svc, svc.served_model_name or model_name
        self.llm = None
        self.tokenizer = None
        self.formatter: Optional[ChatFormatter] = None
        self.grammars: Optional[Grammars] = None
        self.vision = None
        self.totals = Totals()
        self.started = time.time()
        self.responses: "OrderedDict[str, Dict[str, Any]]" = OrderedDict()
        self.sem = asyncio.Semaphore(svc.max_concurrency)
        self.waiting = 0
        self.shutting_down = False
        self.developer_as_system = False

    def attach(self, llm, tokenizer, vision=None) -> None:
        from .media import MediaPolicy
        svc = self.svc
        self.media_policy = MediaPolicy(limit_images=svc.limit_mm_per_prompt, low_detail_pixels=svc.mm_low_detail_pixels,
                                        fetch_timeout_s=svc.image_fetch_timeout, fetch_max_bytes=svc.image_fetch_max_mib << 20,
                                        allowed_domains=tuple(svc.allowed_media_domains), processor=dict(svc.mm_processor_kwargs),
                                        enabled=svc.vision != "off")
        if svc.vision == "off":
            vision = None
        llm.sched.health.TICK_S = float(svc.log_stats_interval)          # --log-stats-interval
        self.tokenizer = tokenizer
        cfg = llm.model.cfg
        tpl = getattr(tokenizer, "chat_template", None) or ""
        # family encoders place developer turns themselves; a Jinja template that never names the role would reject them
        self.developer_as_system = bool(tpl) and "developer" not in tpl
        self.formatter = ChatFormatter.for_checkpoint(
            self.model_name, {"model_type": cfg.model_type, "architectures": [cfg.architecture]},
            getattr(tokenizer, "chat_template", None), self.svc.chat_family or None)
        eos = tuple(llm.sched.cfg.eos_ids) or tuple(getattr(tokenizer, "eos_ids", ()))
        llm.sched.cfg.eos_ids = eos
        self.grammars = Grammars.load(tokenizer, cfg.vocab_size, eos)
        self.vision = vision
        self.llm = llm
        llm.engine.start_watchdog()
        if llm.sched._thread is None:
            llm.sched.start()

    @property
    def ready(self) -> bool:
        return self.llm is not None

    @property
    def vocab(self) -> int:
        return self.llm.model.cfg.vocab_size

    @property
    def max_len(self) -> int:
        return self.llm.sched.cfg.max_model_len


class Gen:
    """One generation in flight: submits to the scheduler and yields events on the asyncio side (``server.rs:794``)."""

    def __init__(self, st: ServerState, prompt: List[int], params: SamplingParams, **kw):
        self.st = st
        self.q: "asyncio.Queue[GenEvent]" = asyncio.Queue()
        self.loop = asyncio.get_running_loop()
        self.rid = "req-" + uuid.uuid4().hex[:16]
        self.req = GenRequest(self.rid, prompt, params, sink=self._sink, **kw)
        self.prompt_tokens = len(prompt)
        self.cached = 0
        self.finish: Optional[Finish] = None
        self.error: Optional[str] = None
        self.n_out = 0
        self.http_request = _current_request.get()
        st.llm.sched.submit(self.req)

    def _sink(self, ev: GenEvent) -> None:
        try:
            self.loop.call_soon_threadsafe(self.q.put_nowait, ev)
        except RuntimeError:       # the client's event loop is gone
            pass

    async def events(self) -> AsyncIterator[GenEvent]:
        deadline = time.monotonic() + self.st.svc.request_timeout_s
        last_probe = time.monotonic()

        async def client_gone() -> bool:
            """A client that closed its connection (streaming or not) ends the generation; probed twice a second."""
            nonlocal last_probe
            last_probe = time.monotonic()
            req = self.http_request
            try:
                return req is not None and await req.is_disconnected()
            except Exception:
                return False
        while True:
            try:
                ev = await asyncio.wait_for(self.q.get(), timeout=min(max(deadline - time.monotonic(), 0.01), 0.5))
            except asyncio.TimeoutError:
                if time.monotonic() >= deadline:
                    self.st.llm.sched.abort(self.rid)
                    self.finish, self.error = Finish.ABORT, "request deadline exceeded"
                    return
                ev = None
            if (ev is None or time.monotonic() - last_probe > 0.5) and await client_gone():
                self.abort(cancelled=True)
                self.finish, self.error = Finish.ABORT, "client disconnected"
                return
            if ev is None:
                continue
            self.cached = ev.cached_tokens
            self.n_out += len(ev.tokens)
            if ev.tokens or ev.hidden is not None:
                yield ev
            if ev.finish is not None:
                self.finish, self.error = ev.finish, ev.error
                return

    def abort(self, cancelled: bool = True) -> None:
        """End the request early.  ``cancelled``: the client went away (counted as such); False: a stop string matched."""
        if cancelled and not getattr(self, "_counted_cancel", False):
            self._counted_cancel = True
            self.st.totals.cancelled += 1
        self.st.llm.sched.abort(self.rid)


def shown(ev: GenEvent, include_stop: bool = False):
    """(tokens, logprobs) of an event as the answer shows them: the end-of-sequence or stop token that ended the generation
    is not part of the text unless the request asked for it (``include_stop_str_in_output``)."""
    if ev.stopped_on is None or include_stop or not ev.tokens:
        return ev.tokens, ev.logprobs
    return ev.tokens[:-1], (ev.logprobs[:-1] if ev.logprobs else ev.logprobs)


def finish_reason(f: Optional[Finish], tool_calls: bool = False, stopped_by_string: bool = False) -> str:
    if tool_calls:
        return "tool_calls"
    if stopped_by_string or f == Finish.STOP:
        return "stop"
    if f == Finish.LENGTH:
        return "length"
    return "stop" if f is None else f.value


def _usage(prompt: int, out: int, cached: int = 0) -> Dict[str, Any]:
    return {"prompt_tokens": prompt, "completion_tokens": out, "total_tokens": prompt + out,
            "prompt_tokens_details": {"cached_tokens": cached}}


def _lp_entry(tok, lp: dict) -> Dict[str, Any]:
    def one(tid, v):
        b = tok.token_bytes(tid)
        return {"token": b.decode("utf-8", errors="replace"), "logprob": max(v, -9999.0), "bytes": list(b)}
    e = one(lp["token"], lp["logprob"])
    e["top_logprobs"] = [one(t, v) for t, v in lp.get("top", [])]
    return e


def _preview(text: str, limit: int) -> str:
    """A bounded, single-line preview of a payload for the log (control characters escaped)."""
    text = text if len(text) <= limit else text[:limit] + f"... ({len(text)} characters)"
    return text.encode("unicode_escape").decode("ascii") if any(ord(c) < 32 for c in text) else text


def create_app(st: ServerState) -> FastAPI:
    app = FastAPI(title="blaze_b200", version=__version__)

    # ------------------------------------------------------------------ middleware: request id, CORS, auth, loading, admission
    @app.middleware("http")
    async def control(request: Request, call_next):
        rid = request.headers.get("x-request-id") or ""
        if not rid or len(rid) > 128 or not all(c.isalnum() or c in "-_.:" for c in rid):
            rid = uuid.uuid4().hex          # absent or not a plain token: the server names the request
        path = request.url.path
        _current_request.set(request)
        cors = {"x-request-id": rid}
        if st.svc.cors_origins:
            origin = request.headers.get("origin")
            allowed = "*" if "*" in st.svc.cors_origins else (origin if origin in st.svc.cors_origins else st.svc.cors_origins[0])
            cors.update({"access-control-allow-origin": allowed, "access-control-allow-headers": "*",
                         "access-control-allow-methods": "GET,POST,DELETE,OPTIONS"})
        if request.method == "OPTIONS":
            return PlainTextResponse("", headers=cors)
        open_paths = ("/health", "/ping", "/version", "/metrics")
        if st.svc.api_keys and path not in open_paths:
            key = request.headers.get("x-api-key")
            auth = request.headers.get("authorization", "")
            if auth.lower().startswith("bearer "):
                key = auth[7:].strip()
            if not key or not any(hmac.compare_digest(key, k) for k in st.svc.api_keys):
                r = _err(401, "invalid or missing API key", "authentication_error", code="invalid_api_key")
                r.headers.update(cors)
                return r
        if not st.ready and path not in ("/ping", "/version", "/metrics"):
            body = {"error": {"message": "model is loading", "type": "service_unavailable", "code": "model_loading"},
                    "status": "loading", **log.Stage.status()}
            return JSONResponse(body, status_code=503, headers={**cors, "retry-after": "5"})
        heavy = request.method == "POST" and path.startswith("/v1/") and path not in ("/v1/messages/count_tokens",)
        if heavy:
            if st.shutting_down:
                return _err(503, "server is shutting down", "service_unavailable")
            if st.waiting >= st.svc.max_queue:
                st.totals.errors += 1
                return _err(429, "too many requests queued", "rate_limit_error", code="queue_full")
            st.waiting += 1
            try:
                await st.sem.acquire()
            finally:
                st.waiting -= 1
            st.totals.inflight += 1
        t0 = time.monotonic()
        released = False

        def release():
            nonlocal released
            if heavy and not released:
                released = True
                st.sem.release()
                st.totals.inflight -= 1
                st.totals.e2e.observe(time.monotonic() - t0)
        _current_request.set(request)
        try:
            resp = await call_next(request)
        except Exception:
            release()
            raise
        resp.headers.update(cors)
        if isinstance(resp, StreamingResponse) or hasattr(resp, "body_iterator"):
            inner = resp.body_iterator

            async def wrapped():
                try:
                    async for chunk in inner:
                        yield chunk
                finally:
                    release()
            resp.body_iterator = wrapped()
        else:
            release()
        return resp

    async def _body(request: Request) -> Dict[str, Any]:
        limit = st.svc.max_request_body_mib << 20
        declared = request.headers.get("content-length")
        if declared and declared.isdigit() and int(declared) > limit:
            raise RequestError(f"request body is larger than {st.svc.max_request_body_mib} MiB", None, "request_too_large", 413)
        raw = await request.body()
        if len(raw) > limit:
            raise RequestError(f"request body is larger than {st.svc.max_request_body_mib} MiB", None, "request_too_large", 413)
        if st.svc.log_inputs:
            log.info("request.input", path=request.url.path, body=_preview(raw.decode("utf-8", "replace"), st.svc.max_log_len))
        try:
            b = json.loads(raw)
        except Exception:
            raise RequestError("request body must be JSON")
        if not isinstance(b, dict):
            raise RequestError("request body must be a JSON object")
        return b

    @app.exception_handler(RequestError)
    async def on_request_error(request: Request, e: RequestError):
        st.totals.errors += 1
        return _err(e.status, e.message, "invalid_request_error" if e.status < 500 else "server_error", e.param,
                    code=None if e.code == "invalid_request_error" else e.code)

    from starlette.exceptions import HTTPException as _HTTPException

    @app.exception_handler(_HTTPException)
    async def on_http_error(request: Request, e: _HTTPException):
        # unknown routes and wrong methods answer with the OpenAI error object too
        what = {404: f"no route {request.method} {request.url.path}", 405: f"method {request.method} is not allowed on {request.url.path}"}.get(
            e.status_code, str(e.detail))
        return _err(e.status_code, what, "invalid_request_error", code={404: "not_found", 405: "method_not_allowed"}.get(e.status_code))

    @app.exception_handler(ConstraintError)
    async def on_constraint_error(request: Request, e: ConstraintError):
        st.totals.errors += 1
        return _err(400, str(e), param="response_format")

    # ------------------------------------------------------------------ control plane
    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.get("/ping")
    async def ping():
        return PlainTextResponse("pong")

    @app.get("/version")
    async def version():
        return {"version": __version__}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [_model_card()]}

    @app.get("/v1/models/{model_id:path}")
    async def model(model_id: str):
        if model_id != st.model_name:
            return _err(404, f"model {model_id!r} not found", code="model_not_found")
        return _model_card()

    def _model_card():
        return {"id": st.model_name, "object": "model", "created": int(st.started), "owned_by": "blaze_b200",
                "max_model_len": st.max_len}

    @app.get("/server_info")
    @app.get("/get_server_info")
    async def server_info():
        llm = st.llm
        s = llm.sched.stats
        return {"version": __version__, "model": st.model_name, "uptime_s": round(time.time() - st.started, 1),
                "max_model_len": st.max_len, "tp": llm.model.tp.world, "kv_dtype": llm.engine.ecfg.kv_dtype,
                "kv_pages": llm.engine.num_pages, "kv_pages_free": llm.engine.pages.free_count,
                "active": len(llm.sched.active), "waiting": len(llm.sched.waiting), "preempted": len(llm.sched.preempted),
                "stats": vars(s), "prefix_cache": {"entries": len(llm.sched.cache.entries), "hits": llm.sched.cache.hits,
                                                   "lookups": llm.sched.cache.lookups},
                "weights": llm.model.weight_format.value, "kernels": llm.model.ops.name,
                "sampling_defaults": dict(st.svc.defaults), "default_max_tokens": st.svc.default_max_tokens,
                "scheduler": {"schedule": llm.sched.cfg.schedule, "chunk": llm.sched.cfg.chunk, "max_seqs": llm.sched.cfg.max_seqs,
                              "max_step_tokens": llm.sched.cfg.max_step_tokens, "spec_method": llm.sched.cfg.spec_method,
                              "max_draft": llm.sched.cfg.max_draft, "prefix_cache": llm.sched.cfg.prefix_cache},
                "config": {k: ("[REDACTED]" if "key" in k else v) for k, v in st.svc.public_config().items()},
                **({"expert_heat": llm.heat.report(max(llm.model.tp.world, 8))} if getattr(llm, "heat", None) is not None else {})}

    @app.get("/metrics")
    async def metrics():
        t = st.totals
        lines = []

        def counter(name, v, help_):
            lines.append(f"# HELP {name} {help_}\n# TYPE {name} counter\n{name} {v}\n")

        def gauge(name, v, help_):
            lines.append(f"# HELP {name} {help_}\n# TYPE {name} gauge\n{name} {v}\n")
        counter("blaze_requests_total", t.requests, "Requests accepted")
        counter("blaze_request_errors_total", t.errors, "Requests rejected or failed")
        counter("blaze_prompt_tokens_total", t.prompt_tokens, "Prompt tokens processed")
        counter("blaze_cached_prompt_tokens_total", t.cached_tokens, "Prompt tokens served from the prefix cache")
        counter("blaze_generation_tokens_total", t.output_tokens, "Tokens generated")
        gauge("blaze_requests_in_flight", t.inflight, "Requests being served")
        gauge("blaze_requests_running", t.inflight, "Requests being served (same as blaze_requests_in_flight)")
        counter("blaze_requests_cancelled_total", t.cancelled, "Requests whose client went away before the end")
        counter("blaze_prefill_tokens_total", t.prompt_tokens - t.cached_tokens, "Prompt tokens computed (not served from the prefix cache)")
        gauge("blaze_requests_waiting", st.waiting, "Requests waiting for admission")
        if st.ready:
            sc = st.llm.sched
            gauge("blaze_sequences_active", len(sc.active), "Sequences in the running batch")
            gauge("blaze_kv_pages_free", st.llm.engine.pages.free_count, "Free KV pages")
            counter("blaze_preemptions_total", sc.stats.preemptions, "Recompute preemptions")
            counter("blaze_draft_tokens_total", sc.stats.draft_tokens, "Speculative tokens proposed")
            counter("blaze_accepted_draft_tokens_total", sc.stats.accepted_tokens, "Speculative tokens accepted")
            counter("blaze_prefix_cache_lookups_total", sc.cache.lookups, "Prefix-cache lookups")
            counter("blaze_prefix_cache_hits_total", sc.cache.hits, "Prefix-cache hits")
            gauge("blaze_prefix_cache_entries", len(sc.cache.entries), "Snapshots held on the device")
            if sc.cache.host is not None:
                gauge("blaze_kv_host_entries", len(sc.cache.host_entries), "Snapshots parked in the host KV tier")
                gauge("blaze_kv_host_pages_free", sc.cache.host.free_pages, "Free pages of the host KV tier")
                counter("blaze_kv_host_hits_total", sc.cache.host_hits, "Prefix-cache hits served from the host KV tier")
                counter("blaze_kv_host_spilled_pages_total", sc.cache.host.spilled_pages, "Pages copied to the host KV tier")
            eng = st.llm.engine
            counter("blaze_failed_steps_total", sc.stats.failed, "Engine steps that failed (their requests ended with an error)")
            counter("blaze_device_status_errors_total", eng.status_errors, "Steps in which a kernel reported an error through the device status word")
            counter("blaze_engine_hangs_total", eng.hangs, "Steps the watchdog reported as hung")
            counter("blaze_slow_steps_total", sc.health.outliers, "Steps flagged as latency outliers")
            gauge("blaze_mean_step_seconds", round(sc.health.mean_s, 6), "Running mean of the engine step time")
            lines.append(sc.ttft.render("blaze_time_to_first_token_seconds", "Time to first token"))
            lines.append(sc.tpot.render("blaze_time_per_output_token_seconds", "Time per output token"))
            lines.append(sc.step_ms.render("blaze_step_seconds", "Engine step time"))
        lines.append(t.e2e.render("blaze_request_seconds", "End-to-end request time"))
        return PlainTextResponse("".join(lines), media_type="text/plain; version=0.0.4")

    # ------------------------------------------------------------------ tokenisation
    @app.post("/tokenize")
    async def tokenize(request: Request):
        b = await _body(request)
        if "messages" in b:
            # what a chat request with the same body would use as its prompt (tools, tool_choice, template arguments)
            _check_continuation(b, b["messages"] if isinstance(b["messages"], list) else [])
            text, prefix, _ = _render_chat(b)
            ids = st.tokenizer.encode(text, add_special_tokens=bool(b.get("add_special_tokens", False)))
            if prefix:                        # a continued turn is tokenised on its own, after the prompt
                ids = ids + st.tokenizer.encode(prefix, add_special_tokens=False)
        else:
            text = b.get("prompt", b.get("text"))
            if not isinstance(text, str):
                raise RequestError("prompt must be a string", "prompt")
            ids = st.tokenizer.encode(text, add_special_tokens=bool(b.get("add_special_tokens", False)))
        out = {"tokens": ids, "count": len(ids), "max_model_len": st.max_len}
        if b.get("return_token_strs"):
            out["token_strs"] = [st.tokenizer.decode([t], skip_special_tokens=False) for t in ids]
        return out

    @app.post("/detokenize")
    async def detokenize(request: Request):
        b = await _body(request)
        ids = b.get("tokens")
        if not isinstance(ids, list) or any(isinstance(t, bool) or not isinstance(t, int) or not 0 <= t < st.vocab for t in ids):
            raise RequestError("tokens must be a list of token ids of this model's vocabulary", "tokens")
        return {"prompt": st.tokenizer.decode(ids, skip_special_tokens=bool(b.get("skip_special_tokens", False)))}

    # ------------------------------------------------------------------ helpers shared by the generation routes
    def _check_model(b):
        m = b.get("model")
        if m is not None and m != st.model_name and m != "default":
            raise RequestError(f"model {m!r} is not served here (serving {st.model_name!r})", "model", "model_not_found", 404)

    def _check_len(n_prompt: int, params: SamplingParams):
        if n_prompt == 0:
            raise RequestError("prompt is empty", "prompt")
        if n_prompt + 1 > st.max_len:
            raise RequestError(f"prompt has {n_prompt} tokens; the context limit is {st.max_len}", "prompt",
                               "context_length_exceeded")
        params.max_tokens = max(1, min(params.max_tokens, st.max_len - n_prompt - 1))

    def _think(b, enable_thinking) -> Optional[ThinkBudget]:
        budget = thinking_budget_of(b, st.svc.thinking_budget)
        if budget is None:
            return None
        o, c = st.tokenizer.token_id("<think>"), st.tokenizer.token_id("</think>")
        if o is None or c is None:
            return None
        return ThinkBudget(budget, o, c, st.tokenizer.encode(THINK_CLOSING))

    def _think_parser(st, in_think: Optional[bool] = None):
        """Reasoning splitter of the configured family (None when reasoning parsing is off).  ``in_think``: the prompt
        ended inside the reasoning channel (None: the family's default)."""
        return get_think_parser(st.svc.reasoning_parser, starts_in_think=in_think) if st.svc.reasoning_parser else None

    def _cache_point(prompt_ids: List[int]) -> Optional[int]:
        """Prefix-cache boundary: the last ``<|im_start|>`` (``server.rs:926-933``)."""
        ims = st.tokenizer.token_id("<|im_start|>")
        if ims is None:
            return None
        for i in range(len(prompt_ids) - 1, 0, -1):
            if prompt_ids[i] == ims:
                return i
        return None

    def _account(g: Gen):
        t = st.totals
        t.requests += 1
        t.prompt_tokens += g.prompt_tokens
        t.cached_tokens += g.cached
        t.output_tokens += g.n_out
        if g.finish == Finish.ERROR:
            t.errors += 1

    def _sse(obj) -> bytes:
        return ("data: " + json.dumps(obj, ensure_ascii=False, separators=(",", ":")) + "\n\n").encode()

    def _check_tool_choice(tools, choice) -> Optional[List[str]]:
        """Validate ``tool_choice`` against ``tools``; returns the tool names a forced call may use (``required``: all of
        them, a named function: that one), or None when nothing is forced."""
        names = [(t.get("function") or {}).get("name") for t in tools or [] if isinstance(t, dict)]
        if isinstance(choice, str):
            if choice not in ("auto", "none", "required"):
                raise RequestError('tool_choice must be "auto", "none", "required" or a named function', "tool_choice")
            if choice == "required":
                if not names:
                    raise RequestError('tool_choice is "required" but tools is empty', "tool_choice")
                return names
            return None
        if isinstance(choice, dict):
            name = (choice.get("function") or {}).get("name")
            if name not in names:
                raise RequestError(f'tool named "{name}" in tool_choice is not present in tools', "tool_choice")
            return [name]
        if choice is not None:
            raise RequestError('tool_choice must be "auto", "none", "required" or a named function', "tool_choice")
        return None

    def _check_continuation(b, msgs) -> None:
        cont = b.get("continue_final_message")
        if cont in (None, False, 0):
            return
        if b.get("add_generation_prompt") is True:
            raise RequestError("continue_final_message and add_generation_prompt cannot both be true", "continue_final_message")
        last = msgs[-1] if msgs else {}
        if not isinstance(last, dict) or str(last.get("role", "")).lower() != "assistant":
            raise RequestError("continue_final_message needs the last message to be an assistant message", "continue_final_message")

    def _render_chat(b: Dict[str, Any]):
        """(prompt text, continuation prefix, thinking) of a chat request body; request errors of the family encoders
        become 400s."""
        msgs = b.get("messages")
        if isinstance(msgs, list) and any(isinstance(m, dict) and "reasoning" in m and "reasoning_content" not in m for m in msgs):
            # agent frameworks replay an assistant turn's reasoning under either name
            b = {**b, "messages": [({**m, "reasoning_content": m["reasoning"]} if isinstance(m, dict) and isinstance(m.get("reasoning"), str)
                                    and "reasoning_content" not in m else m) for m in msgs]}
        if isinstance(msgs, list) and st.developer_as_system and any(isinstance(m, dict) and str(m.get("role", "")).lower() == "developer" for m in msgs):
            # new OpenAI SDKs send system prompts as developer messages; a template that does not know the role gets them as system
            b = {**b, "messages": [({**m, "role": "system"} if isinstance(m, dict) and str(m.get("role", "")).lower() == "developer" else m)
                                   for m in b["messages"]]}
        try:
            return st.formatter.render_request(b, st.svc.chat_template_kwargs)
        except (ValueError, TypeError, IndexError, KeyError) as e:
            raise RequestError(f"cannot render the chat prompt: {e}", "messages")

    # ------------------------------------------------------------------ /v1/chat/completions
    async def _prepare_chat(b: Dict[str, Any]):
        _check_model(b)
        msgs = b.get("messages")
        if not isinstance(msgs, list) or not msgs:
            raise RequestError("messages must be a non-empty list", "messages")
        tools = b.get("tools")
        tool_choice = b.get("tool_choice", "auto" if tools else "none")
        forced = _check_tool_choice(tools, tool_choice)
        _check_continuation(b, msgs)
        if st.vision is None:
            for m in msgs:
                for part in (m.get("content") if isinstance(m, dict) and isinstance(m.get("content"), list) else []):
                    kind = part.get("type") if isinstance(part, dict) else None
                    if kind in ("image_url", "image", "input_image", "video_url", "video", "audio_url", "input_audio"):
                        raise RequestError(f"this model only takes text input; received a content part of type {kind!r}", "messages")
        if tool_choice == "none":
            tools_for_prompt = None
        else:
            tools_for_prompt = tools
        text, prefix, enable_thinking = _render_chat(b)
        ids = st.tokenizer.encode(text)
        if prefix:
            ids = ids + st.tokenizer.encode(prefix, add_special_tokens=False)      # the continued turn is tokenised on its own
        mm = None
        if st.vision is not None:
            from .media import collect_images
            mm = await collect_images(msgs, st.vision, st.svc.allow_remote_images, st.media_policy, b.get("mm_processor_kwargs"))
        # a reasoning model's prompt with thinking switched off takes the instruct sampling defaults
        instruct = st.svc.reasoning_parser is not None and (enable_thinking is False or text.rstrip("\n").endswith("</think>"))
        params = sampling_of(b, st.svc, st.vocab, instruct=instruct)
        _check_len(len(ids), params)
        spec = grammar_of(b, st.svc.grammar_whitespace)
        in_think = text.rstrip("\n").endswith(("<think>", "<|open|>think<|sep|>")) and not prefix
        if forced and spec is None and not in_think and not prefix and st.grammars.ll_tok is not None:
            # tool_choice forces a call: the answer must be calls to the named tools in the parser's syntax.  Where the
            # syntax is not known, or the prompt leaves the model inside its reasoning, the model is only asked.
            g = forced_call_grammar(st.svc.tool_call_parser, forced, b.get("parallel_tool_calls") is False)
            if g is not None:
                spec = {"kind": "grammar", "grammar": g}
        return ids, params, tools_for_prompt, enable_thinking, spec, mm, in_think

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        b = await _body(request)
        ids, params, tools, enable_thinking, spec, mm, in_think = await _prepare_chat(b)
        stops = stop_strings_of(b)
        include_stop = bool(b.get("include_stop_str_in_output", b.get("no_stop_trim", False)))
        skip_special = bool(b.get("skip_special_tokens", True))
        n = params.n
        stream = bool(b.get("stream", False))
        reasoning = st.svc.reasoning_parser is not None and enable_thinking is not False and b.get("separate_reasoning") is not False
        created, cid = int(time.time()), "chatcmpl-" + uuid.uuid4().hex[:24]
        want_lp = params.logprobs is not None

        def make(i):
            p = SamplingParams(**{**vars(params), "seed": None if params.seed is None else params.seed + i, "n": 1})
            cons = st.grammars.constraint(spec) if spec else None
            g = Gen(st, ids, p, cache_point=_cache_point(ids), constraint=cons, think=_think(b, enable_thinking), mm=mm)
            proc = ChatResponseProcessor(st.tokenizer, stops, include_stop, skip_special, reasoning=reasoning,
                                         tool_parser=get_tool_parser(st.svc.tool_call_parser, tools) if tools else None,
                                         think_parser=_think_parser(st, in_think))
            return g, proc
        gens = [make(i) for i in range(n)]

        if not stream:
            choices = []
            for i, (g, proc) in enumerate(gens):
                lps = []
                async for ev in g.events():
                    toks, elp = shown(ev, include_stop)
                    d = proc.push(toks)
                    if elp:
                        lps.extend(elp)
                    if d.stopped:
                        g.abort(cancelled=False)
                        break
                proc.finish()
                _account(g)
                if g.finish == Finish.ERROR:
                    return _err(500, g.error or "generation failed", "server_error")
                msg: Dict[str, Any] = {"role": "assistant", "content": proc.text or (None if proc.tool_calls else "")}
                if proc.reasoning_text and b.get("include_reasoning") is not False:
                    msg["reasoning_content"] = proc.reasoning_text
                if proc.tool_calls:
                    calls = proc.tool_calls[:1] if b.get("parallel_tool_calls") is False else proc.tool_calls
                    msg["tool_calls"] = [{k: v for k, v in c.to_openai(j).items() if k != "index"} for j, c in enumerate(calls)]
                ch = {"index": i, "message": msg, "finish_reason": finish_reason(g.finish, bool(proc.tool_calls), proc.stopped),
                      "stop_reason": proc.stop_matched}
                if want_lp:
                    ch["logprobs"] = {"content": [_lp_entry(st.tokenizer, l) for l in lps]}
                choices.append(ch)
            usage = _usage(len(ids), sum(g.n_out for g, _ in gens), gens[0][0].cached)
            if st.svc.log_outputs:
                log.info("request.output", id=cid, text=_preview(choices[0]["message"].get("content") or "", st.svc.max_log_len),
                         finish=choices[0]["finish_reason"])
            return {"id": cid, "object": "chat.completion", "created": created, "model": st.model_name, "choices": choices,
                    "usage": usage}

        include_usage = bool((b.get("stream_options") or {}).get("include_usage", False))

        async def gen_stream():
            base = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": st.model_name}
            try:
                for i, (g, proc) in enumerate(gens):
                    yield _sse({**base, "choices": [{"index": i, "delta": {"role": "assistant", "content": ""}, "finish_reason": None}]})
                    n_tools = 0

                    def chunks_of(d, lps=None):
                        nonlocal n_tools
                        out = []
                        delta: Dict[str, Any] = {}
                        if d.reasoning:
                            delta["reasoning_content"] = d.reasoning
                        if d.content:
                            delta["content"] = d.content
                        if d.tool_calls:
                            delta["tool_calls"] = [c.to_openai(n_tools + j) for j, c in enumerate(d.tool_calls)]
                            n_tools += len(d.tool_calls)
                        if delta:
                            ch = {"index": i, "delta": delta, "finish_reason": None}
                            if lps:
                                ch["logprobs"] = {"content": [_lp_entry(st.tokenizer, l) for l in lps]}
                            out.append(_sse({**base, "choices": [ch]}))
                        return out
                    async for ev in g.events():
                        toks, elp = shown(ev, include_stop)
                        d = proc.push(toks)
                        for c in chunks_of(d, elp if want_lp else None):
                            yield c
                        if d.stopped:
                            g.abort(cancelled=False)
                            break
                    for c in chunks_of(proc.finish()):
                        yield c
                    _account(g)
                    if g.finish == Finish.ERROR:
                        yield _sse({"error": {"message": g.error or "generation failed", "type": "server_error"}})
                    yield _sse({**base, "choices": [{"index": i, "delta": {}, "stop_reason": proc.stop_matched, "finish_reason":
                                                     finish_reason(g.finish, bool(proc.tool_calls), proc.stopped)}]})
                if include_usage:
                    yield _sse({**base, "choices": [], "usage": _usage(len(ids), sum(g.n_out for g, _ in gens), gens[0][0].cached)})
                yield b"data: [DONE]\n\n"
            finally:
                for g, _ in gens:
                    if g.finish is None:
                        g.abort()
        return StreamingResponse(gen_stream(), media_type="text/event-stream")

    # ------------------------------------------------------------------ /v1/completions
    def _prompts_of(b) -> List[List[int]]:
        p = b.get("prompt")
        if isinstance(p, str):
            return [st.tokenizer.encode(p)]
        if isinstance(p, list) and p and all(isinstance(x, int) for x in p):
            return [list(p)]
        if isinstance(p, list) and p and all(isinstance(x, str) for x in p):
            return [st.tokenizer.encode(x) for x in p]
        if isinstance(p, list) and p and all(isinstance(x, list) and all(isinstance(t, int) for t in x) for x in p):
            return [list(x) for x in p]
        raise RequestError("prompt must be a string, a list of strings, a list of token ids or a list of those", "prompt")

    @app.post("/v1/completions")
    async def completions(request: Request):
        b = await _body(request)
        _check_model(b)
        prompts = _prompts_of(b)
        params = sampling_of(b, st.svc, st.vocab)
        if len(prompts) * params.n > MAX_COMPLETIONS_PER_REQUEST:
            raise RequestError(f"at most {MAX_COMPLETIONS_PER_REQUEST} generations per request", "n")
        keep = b.get("truncate_prompt_tokens")
        if keep is not None:
            if isinstance(keep, bool) or not isinstance(keep, int) or keep < 1:
                raise RequestError("truncate_prompt_tokens must be a positive integer", "truncate_prompt_tokens")
            prompts = [p[-keep:] for p in prompts]          # the tail of an over-long prompt is what is kept
        for p in prompts:
            if any(t < 0 or t >= st.vocab for t in p):
                raise RequestError("prompt token id outside the vocabulary", "prompt")
            _check_len(len(p), params)
        stops = stop_strings_of(b)
        include_stop = bool(b.get("include_stop_str_in_output", False))
        echo = bool(b.get("echo", False))
        if echo and params.logprobs is not None:
            raise RequestError("echo with logprobs is not supported (prompt log-probabilities are not computed)", "echo")
        stream = bool(b.get("stream", False))
        spec = grammar_of(b, st.svc.grammar_whitespace)
        created, cid = int(time.time()), "cmpl-" + uuid.uuid4().hex[:24]
        gens = []
        for pi, p in enumerate(prompts):
            for j in range(params.n):
                sp = SamplingParams(**{**vars(params), "seed": None if params.seed is None else params.seed + j, "n": 1})
                cons = st.grammars.constraint(spec) if spec else None
                gens.append((Gen(st, p, sp, constraint=cons), ChatResponseProcessor(
                    st.tokenizer, stops, include_stop, bool(b.get("skip_special_tokens", True))), p))

        def lp_obj(lps, offset0=0):
            toks = [st.tokenizer.token_bytes(l["token"]).decode("utf-8", errors="replace") for l in lps]
            offs, o = [], offset0
            for t in toks:
                offs.append(o)
                o += len(t)
            return {"tokens": toks, "token_logprobs": [max(l["logprob"], -9999.0) for l in lps],
                    "top_logprobs": [{st.tokenizer.token_bytes(t).decode("utf-8", errors="replace"): max(v, -9999.0)
                                      for t, v in l.get("top", [])} for l in lps], "text_offset": offs}

        if not stream:
            choices = []
            for i, (g, proc, p) in enumerate(gens):
                lps = []
                async for ev in g.events():
                    toks, elp = shown(ev, include_stop)
                    d = proc.push(toks)
                    if elp:
                        lps.extend(elp)
                    if d.stopped:
                        g.abort(cancelled=False)
                        break
                proc.finish()
                _account(g)
                if g.finish == Finish.ERROR:
                    return _err(500, g.error or "generation failed", "server_error")
                text = (st.tokenizer.decode(p) if echo else "") + proc.text
                ch = {"index": i, "text": text, "finish_reason": finish_reason(g.finish, False, proc.stopped), "logprobs": None,
                      "stop_reason": proc.stop_matched}
                if params.logprobs is not None:
                    ch["logprobs"] = lp_obj(lps)
                choices.append(ch)
            if st.svc.log_outputs:
                log.info("request.output", id=cid, text=_preview(choices[0]["text"], st.svc.max_log_len), finish=choices[0]["finish_reason"])
            return {"id": cid, "object": "text_completion", "created": created, "model": st.model_name, "choices": choices,
                    "usage": _usage(sum(len(p) for _, _, p in gens), sum(g.n_out for g, _, _ in gens), 0)}

        include_usage = bool((b.get("stream_options") or {}).get("include_usage", False))

        async def gen_stream():
            base = {"id": cid, "object": "text_completion", "created": created, "model": st.model_name}
            try:
                for i, (g, proc, p) in enumerate(gens):
                    if echo:
                        yield _sse({**base, "choices": [{"index": i, "text": st.tokenizer.decode(p), "finish_reason": None}]})
                    sent = 0                     # characters of this choice's text already sent (text_offset of the next token)
                    pend_lp = []
                    async for ev in g.events():
                        toks, elp = shown(ev, include_stop)
                        d = proc.push(toks)
                        if elp and params.logprobs is not None:
                            pend_lp.extend(elp)
                        if d.content or pend_lp:
                            ch = {"index": i, "text": d.content or "", "finish_reason": None}
                            if params.logprobs is not None:
                                ch["logprobs"] = lp_obj(pend_lp, sent)
                                pend_lp = []
                            sent += len(d.content or "")
                            yield _sse({**base, "choices": [ch]})
                        if d.stopped:
                            g.abort(cancelled=False)
                            break
                    d = proc.finish()
                    _account(g)
                    ch = {"index": i, "text": d.content, "finish_reason": finish_reason(g.finish, False, proc.stopped)}
                    if params.logprobs is not None:
                        ch["logprobs"] = lp_obj(pend_lp, sent)
                    yield _sse({**base, "choices": [ch]})
                if include_usage:
                    yield _sse({**base, "choices": [], "usage": _usage(sum(len(p) for _, _, p in gens), sum(g.n_out for g, _, _ in gens))})
                yield b"data: [DONE]\n\n"
            finally:
                for g, _, _ in gens:
                    if g.finish is None:
                        g.abort()
        return StreamingResponse(gen_stream(), media_type="text/event-stream")

    # ------------------------------------------------------------------ /v1/embeddings
    @app.post("/v1/embeddings")
    async def embeddings(request: Request):
        b = await _body(request)
        _check_model(b)
        inp = b.get("input")
        if isinstance(inp, str):
            items = [st.tokenizer.encode(inp)]
        elif isinstance(inp, list) and inp and all(isinstance(x, str) for x in inp):
            items = [st.tokenizer.encode(x) for x in inp]
        elif isinstance(inp, list) and inp and all(isinstance(x, int) for x in inp):
            items = [inp]
        elif isinstance(inp, list) and inp and all(isinstance(x, list) for x in inp):
            items = inp
        else:
            raise RequestError("input must be a string, a list of strings or token ids", "input")
        dims = b.get("dimensions")
        if dims is not None and (not isinstance(dims, int) or dims < 1 or dims > st.llm.model.cfg.hidden_size):
            raise RequestError("dimensions must be between 1 and the hidden size", "dimensions")
        fmt = b.get("encoding_format", "float")
        if fmt not in ("float", "base64"):
            raise RequestError("encoding_format must be float or base64", "encoding_format")
        data, total = [], 0
        for i, ids in enumerate(items):
            if not ids or len(ids) + 1 > st.max_len:
                raise RequestError("input is empty or longer than the context limit", "input")
            g = Gen(st, list(ids), SamplingParams(max_tokens=1), embed_only=True)
            vec = None
            async for ev in g.events():
                if ev.hidden is not None:
                    vec = ev.hidden
            _account(g)
            if vec is None:
                return _err(500, g.error or "embedding failed", "server_error")
            if dims:
                vec = vec[:dims]
            vec = vec / vec.norm().clamp_min(1e-12)
            vals = vec.tolist()
            emb = base64.b64encode(struct.pack(f"<{len(vals)}f", *vals)).decode() if fmt == "base64" else vals
            data.append({"object": "embedding", "index": i, "embedding": emb})
            total += len(ids)
        return {"object": "list", "data": data, "model": st.model_name, "usage": {"prompt_tokens": total, "total_tokens": total}}

    # ------------------------------------------------------------------ /v1/responses (OpenAI Responses API adapter)
    @app.post("/v1/responses")
    async def responses(request: Request):
        b = await _body(request)
        _check_model(b)
        kept = None
        prev = b.get("previous_response_id")
        if prev:
            old = st.responses.get(prev)
            if old is None:
                raise RequestError(f"no response with id {prev!r} is kept", "previous_response_id", "not_found", 404)
            kept = old["_messages"]
        cb, msgs, custom = rsp.chat_request(b, kept)
        ids, params, tools_p, enable_thinking, spec, mm, in_think = await _prepare_chat(cb)
        rid = rsp.new_id("resp")
        cons = st.grammars.constraint(spec) if spec else None
        g = Gen(st, ids, params, cache_point=_cache_point(ids), constraint=cons, mm=mm)
        proc = ChatResponseProcessor(st.tokenizer, stop_strings_of(cb),
                                     reasoning=st.svc.reasoning_parser is not None and enable_thinking is not False,
                                     tool_parser=get_tool_parser(st.svc.tool_call_parser, tools_p) if tools_p else None,
                                     think_parser=_think_parser(st, in_think))
        single = cb.get("parallel_tool_calls") is False

        def calls():
            return proc.tool_calls[:1] if single else proc.tool_calls

        def use():
            return rsp.usage(len(ids), g.n_out, g.cached)

        def remember(obj, reasoning, text):
            if b.get("store", True):
                st.responses[rid] = {**obj, "_messages": rsp.kept_messages(msgs, reasoning, text, calls())}
                while len(st.responses) > RESPONSES_KEPT:
                    st.responses.popitem(last=False)

        if not cb.get("stream"):
            async for ev in g.events():
                if proc.push(shown(ev)[0]).stopped:
                    g.abort(cancelled=False)
                    break
            proc.finish()
            _account(g)
            if g.finish == Finish.ERROR:
                return _err(500, g.error or "generation failed", "server_error")
            length = g.finish == Finish.LENGTH and not proc.stopped
            reasoning, text = rsp.settle(proc.reasoning_text, proc.text, len(calls()), not length)
            obj = rsp.shell(b, rid, st.model_name, "incomplete" if length else "completed")
            obj["output"] = rsp.output_items(reasoning, text, calls(), custom)
            obj["output_text"] = text
            obj["usage"] = use()
            if length:
                obj["incomplete_details"] = {"reason": "max_output_tokens"}
            remember(obj, reasoning, text)
            return obj

        async def gen_stream():
            es = rsp.EventStream(b, rid, st.model_name, custom)
            sent = 0

            def wire(pairs):
                return b"".join((f"event: {k}\n" + "data: " + json.dumps(v, ensure_ascii=False) + "\n\n").encode() for k, v in pairs)

            def route(d):
                nonlocal sent
                pairs = es.on_reasoning(d.reasoning) + es.on_text(d.content)
                for c in d.tool_calls:
                    if not (single and sent):
                        pairs += es.on_call(c)
                    sent += 1
                return pairs
            yield wire(es.start())
            try:
                async for ev in g.events():
                    d = proc.push(shown(ev)[0])
                    pairs = route(d)
                    if pairs:
                        yield wire(pairs)
                    if d.stopped:
                        g.abort(cancelled=False)
                        break
                pairs = route(proc.finish())
                _account(g)
                if g.finish == Finish.ERROR:
                    yield wire(pairs + es.failed(g.error or "generation failed"))
                    return
                length = g.finish == Finish.LENGTH and not proc.stopped
                pairs += es.finish(length, not length, len(calls()), use())
                remember(es.resp, es.reasoning, es.text)
                yield wire(pairs)
            finally:
                if g.finish is None:
                    g.abort()
        return StreamingResponse(gen_stream(), media_type="text/event-stream")

    @app.get("/v1/responses/{rid}")
    async def get_response(rid: str):
        obj = st.responses.get(rid)
        if obj is None:
            return _err(404, f"response {rid!r} not found", code="not_found")
        return {k: v for k, v in obj.items() if not k.startswith("_")}

    @app.delete("/v1/responses/{rid}")
    async def delete_response(rid: str):
        if st.responses.pop(rid, None) is None:
            return _err(404, f"response {rid!r} not found", code="not_found")
        return {"id": rid, "object": "response.deleted", "deleted": True}

    # ------------------------------------------------------------------ /v1/messages (Anthropic Messages adapter)
    @app.post("/v1/messages/count_tokens")
    async def count_tokens(request: Request):
        b = await _body(request)
        text, prefix, _ = _render_chat(anth.chat_request(b))
        return {"input_tokens": len(st.tokenizer.encode(text)) + (len(st.tokenizer.encode(prefix, add_special_tokens=False)) if prefix else 0)}

    @app.post("/v1/messages")
    async def messages(request: Request):
        b = await _body(request)
        if not isinstance(b.get("max_tokens"), int) or isinstance(b.get("max_tokens"), bool):
            raise RequestError("max_tokens is required", "max_tokens")
        _check_model(b)
        cb = anth.chat_request(b)
        ids, params, tools_p, enable_thinking, spec, mm, in_think = await _prepare_chat(cb)
        mid = anth.new_id("msg")
        cons = st.grammars.constraint(spec) if spec else None
        g = Gen(st, ids, params, cache_point=_cache_point(ids), constraint=cons, mm=mm)
        proc = ChatResponseProcessor(st.tokenizer, stop_strings_of(cb),
                                     reasoning=st.svc.reasoning_parser is not None and enable_thinking is not False,
                                     tool_parser=get_tool_parser(st.svc.tool_call_parser, tools_p) if tools_p else None,
                                     think_parser=_think_parser(st, in_think))
        single = cb.get("parallel_tool_calls") is False

        if not cb.get("stream"):
            async for ev in g.events():
                if proc.push(shown(ev)[0]).stopped:
                    g.abort(cancelled=False)
                    break
            proc.finish()
            _account(g)
            if g.finish == Finish.ERROR:
                return JSONResponse({"type": "error", "error": {"type": "api_error", "message": g.error or "generation failed"}}, status_code=500)
            calls = proc.tool_calls[:1] if single else proc.tool_calls
            length = g.finish == Finish.LENGTH and not proc.stopped
            reasoning, text = rsp.settle(proc.reasoning_text, proc.text, len(calls), not length)
            reason, sequence = anth.stop_reason(length, bool(calls), proc.stop_matched)
            return {"id": mid, "type": "message", "role": "assistant", "model": b.get("model") or st.model_name,
                    "content": anth.blocks(reasoning, text, calls), "stop_reason": reason, "stop_sequence": sequence,
                    "usage": anth.usage(len(ids), g.n_out, g.cached)}

        async def gen_stream():
            bs = anth.BlockStream(mid, b.get("model") or st.model_name, len(ids))

            def wire(events):
                return b"".join((f"event: {e['type']}\n" + "data: " + json.dumps(e, ensure_ascii=False) + "\n\n").encode() for e in events)

            def route(d):
                out = bs.on_reasoning(d.reasoning) + bs.on_text(d.content)
                for c in d.tool_calls:
                    if not (single and bs.calls):
                        out += bs.on_call(c)
                return out
            yield wire(bs.start())
            try:
                async for ev in g.events():
                    d = proc.push(shown(ev)[0])
                    out = route(d)
                    if out:
                        yield wire(out)
                    if d.stopped:
                        g.abort(cancelled=False)
                        break
                out = route(proc.finish())
                _account(g)
                if g.finish == Finish.ERROR:
                    yield wire(out + bs.error(g.error or "generation failed"))
                    return
                length = g.finish == Finish.LENGTH and not proc.stopped
                yield wire(out + bs.finish(length, proc.stop_matched, g.n_out, g.cached))
            finally:
                if g.finish is None:
                    g.abort()
        return StreamingResponse(gen_stream(), media_type="text/event-stream")

    return app
