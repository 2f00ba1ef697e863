"""Service policy: API keys, admission limits, timeouts, default sampling, request-field validation.

Reference: ``crates/blaze/src/service.rs`` (``ServiceArgs`` :9-90, defaults :167-168, ``validate_sampling`` :271,
``validate_pipeline_fields`` :307) and the limits in ``crates/blaze/src/server.rs:39-48`` / ``check_ranges`` :430.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

from .sampler import DEFAULT_PIPELINE, SamplingParams, Stage, parse_pipeline

MAX_N = 64
MAX_STOP_STRINGS = 64
MAX_STOP_BYTES = 1024
MAX_STOP_IDS = 1024
MAX_COMPLETIONS_PER_REQUEST = 256
MAX_TOP_LOGPROBS = 20


class RequestError(ValueError):
    """A 4xx-class validation error (``code`` is the OpenAI-style error code)."""

    def __init__(self, message: str, param: Optional[str] = None, code: str = "invalid_request_error", status: int = 400):
        super().__init__(message)
        self.message, self.param, self.code, self.status = message, param, code, status


@dataclass
class ServiceArgs:
    host: str = "127.0.0.1"
    port: int = 8000
    api_keys: Tuple[str, ...] = ()
    served_model_name: Optional[str] = None
    max_queue: int = 1024              # requests waiting for admission
    max_concurrency: int = 512         # requests in flight
    request_timeout_s: float = 600.0
    default_max_tokens: int = 512
    log_level: str = "info"
    log_format: str = "text"
    log_requests: bool = False
    profile_prefill: bool = False
    generation_config: Optional[str] = None      # JSON file with default sampling values
    samplers: Optional[str] = None               # default stage order
    top_nsigma: Optional[float] = None
    top_h: Optional[float] = None
    tool_call_parser: str = "hermes"
    reasoning_parser: Optional[str] = "qwen3"
    chat_family: Optional[str] = None            # built-in renderer + message normalisation: chatml, deepseek, glm, kimi
    chat_template_kwargs: Dict[str, Any] = field(default_factory=dict)    # template arguments a request may override
    grammar_whitespace: int = 64                 # longest white-space run between JSON tokens of structured outputs (0: unbounded)
    thinking_budget: Optional[int] = None        # default thinking budget in tokens (requests override it with thinking_token_budget)
    vision: str = "auto"                         # where the vision tower runs: auto | gpu | cpu | off
    vision_threads: Optional[int] = None
    mm_processor_kwargs: Dict[str, Any] = field(default_factory=dict)
    limit_mm_per_prompt: int = 999
    mm_low_detail_pixels: int = 512 * 512
    image_fetch_timeout: float = 5.0
    image_fetch_max_mib: int = 64
    allowed_media_domains: Tuple[str, ...] = ()
    allow_remote_images: bool = True
    shutdown_timeout: float = 10.0               # longest graceful drain after SIGINT / SIGTERM, seconds
    max_request_body_mib: int = 64               # larger request bodies are refused with 413
    log_inputs: bool = False                     # bounded previews of request payloads in the request log
    log_outputs: bool = False                    # bounded previews of response payloads
    max_log_len: int = 400                       # characters of a payload preview
    log_stats_interval: float = 5.0              # seconds between scheduler summaries (0: none)
    instruct_sampling: Dict[str, Any] = field(default_factory=dict)   # defaults of chat requests with thinking off, over `defaults`
    cors_origins: Tuple[str, ...] = ("*",)
    defaults: Dict[str, Any] = field(default_factory=dict)

    def public_config(self) -> Dict[str, Any]:
        """The service flags as the info route may show them (flag spelling; keys are never shown)."""
        out: Dict[str, Any] = {}
        for k, v in vars(self).items():
            if k == "api_keys":
                if v:
                    out["api-key"] = "[REDACTED]"
                continue
            out[k.replace("_", "-")] = list(v) if isinstance(v, tuple) else v
        return out

    def __post_init__(self):
        env = os.environ.get("BLAZE_API_KEY")
        if env and not self.api_keys:
            self.api_keys = tuple(k for k in env.split(",") if k)
        if self.generation_config and self.generation_config not in ("auto", "none"):
            self.read_generation_config(self.generation_config)
        if self.samplers:
            self.defaults.setdefault("samplers", self.samplers)
        if self.top_nsigma is not None:
            self.defaults.setdefault("top_nsigma", self.top_nsigma)
        if self.top_h is not None:
            self.defaults.setdefault("top_h", self.top_h)


SAMPLING_KEYS = ("temperature", "top_p", "top_k", "min_p", "repetition_penalty", "presence_penalty", "frequency_penalty",
                 "top_nsigma", "top_h", "seed", "min_tokens", "samplers")


def merge_sampling(into: Dict[str, Any], src: Dict[str, Any], what: str, override: bool = True) -> None:
    """Merge a JSON object of sampling defaults; unknown keys are an error (a misspelt key must not be ignored)."""
    if not isinstance(src, dict):
        raise ValueError(f"{what} must be a JSON object")
    for k, v in src.items():
        if k not in SAMPLING_KEYS:
            raise ValueError(f"{what}: unknown sampling parameter {k!r}")
        if v is not None and (override or k not in into):
            into[k] = v


def _read_generation_config(self, path: str) -> None:
    with open(path) as f:
        g = json.load(f)
    for k in ("temperature", "top_p", "top_k", "min_p", "repetition_penalty", "presence_penalty", "frequency_penalty"):
        if k in g and g[k] is not None:
            self.defaults.setdefault(k, g[k])


ServiceArgs.read_generation_config = _read_generation_config


def _num(body, key, default, lo=None, hi=None, lo_open=False, integer=False):
    v = body.get(key)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise RequestError(f"{key} must be a number", key)
    if integer and int(v) != v:
        raise RequestError(f"{key} must be an integer", key)
    if lo is not None and (v <= lo if lo_open else v < lo):
        raise RequestError(f"{key} must be {'>' if lo_open else '>='} {lo}", key)
    if hi is not None and v > hi:
        raise RequestError(f"{key} must be <= {hi}", key)
    return int(v) if integer else float(v)


def validate_pipeline_fields(body: Dict[str, Any], pipeline: Sequence[Stage]) -> None:
    """A stage's parameter given without the stage in the chain is an error (``service.rs:307``)."""
    need = {"top_nsigma": Stage.TOP_NSIGMA, "top_h": Stage.TOP_H}
    for key, st in need.items():
        if body.get(key) is not None and st not in pipeline:
            raise RequestError(f"{key} is set but the sampler chain has no {key} stage; add it to `samplers`", key)


def sampling_of(body: Dict[str, Any], svc: ServiceArgs, vocab_size: int, max_tokens_key: str = "max_tokens",
                instruct: bool = False) -> SamplingParams:
    """Build and range-check sampling parameters from a request body (``server.rs:430-504``, :512).  ``instruct``: a chat
    request whose prompt switches thinking off takes the ``instruct_sampling`` defaults over the general ones."""
    b = dict(svc.defaults)
    if instruct:
        b.update(svc.instruct_sampling)
    b.update({k: v for k, v in body.items() if v is not None})
    try:
        pipeline = parse_pipeline(b.get("samplers"))
    except ValueError as e:
        raise RequestError(str(e), "samplers")
    validate_pipeline_fields(body, pipeline)
    mt = b.get(max_tokens_key, b.get("max_completion_tokens", b.get("max_output_tokens")))
    max_tokens = svc.default_max_tokens if mt is None else _num({"m": mt}, "m", 0, lo=1, integer=True)
    min_tokens = _num(b, "min_tokens", 0, lo=0, integer=True)
    if min_tokens > max_tokens:
        raise RequestError("min_tokens must be <= max_tokens", "min_tokens")
    lb_raw = b.get("logit_bias") or {}
    if not isinstance(lb_raw, dict):
        raise RequestError("logit_bias must be an object", "logit_bias")
    lb: Dict[int, float] = {}
    for k, v in lb_raw.items():
        try:
            tid = int(k)
        except (TypeError, ValueError):
            raise RequestError("logit_bias keys must be token ids", "logit_bias")
        if not 0 <= tid < vocab_size:
            raise RequestError(f"logit_bias token id {tid} is outside the vocabulary", "logit_bias")
        if isinstance(v, bool) or not isinstance(v, (int, float)) or not -100 <= v <= 100:
            raise RequestError("logit_bias values must be in [-100, 100]", "logit_bias")
        lb[tid] = float(v)
    stop_ids = b.get("stop_token_ids") or []
    if not isinstance(stop_ids, list) or len(stop_ids) > MAX_STOP_IDS or any(
            isinstance(t, bool) or not isinstance(t, int) or not 0 <= t < vocab_size for t in stop_ids):
        raise RequestError(f"stop_token_ids must be a list of at most {MAX_STOP_IDS} token ids of the vocabulary", "stop_token_ids")
    bad = b.get("bad_words_ids") or []
    if not isinstance(bad, list) or len(bad) > MAX_STOP_IDS:
        raise RequestError(f"bad_words_ids must be a list of at most {MAX_STOP_IDS} id lists", "bad_words_ids")
    lp = b.get("top_logprobs")
    logprobs = b.get("logprobs")
    want_lp: Optional[int] = None
    if isinstance(logprobs, bool):
        if logprobs:
            want_lp = _num({"t": lp}, "t", 0, lo=0, hi=MAX_TOP_LOGPROBS, integer=True) if lp is not None else 0
    elif logprobs is not None:
        want_lp = _num(b, "logprobs", 0, lo=0, hi=MAX_TOP_LOGPROBS, integer=True)
    seed = b.get("seed")
    if seed is not None and (isinstance(seed, bool) or not isinstance(seed, int) or not 0 <= seed < 2 ** 64):
        raise RequestError("seed must be a non-negative integer", "seed")
    if lp is not None and (isinstance(lp, bool) or not isinstance(lp, int)):
        raise RequestError("top_logprobs must be an integer", "top_logprobs")
    if "stream" in body and body["stream"] is not None and not isinstance(body["stream"], bool):
        raise RequestError("stream must be a boolean", "stream")
    return SamplingParams(
        temperature=_num(b, "temperature", 1.0, lo=0.0),
        top_p=_num(b, "top_p", 1.0, lo=0.0, hi=1.0, lo_open=True),
        top_k=_num(b, "top_k", -1, integer=True),
        min_p=_num(b, "min_p", 0.0, lo=0.0, hi=1.0),
        top_nsigma=_num(b, "top_nsigma", 1.0, lo=0.0),
        top_h=_num(b, "top_h", 0.4, lo=0.0, hi=1.0),
        repetition_penalty=_num(b, "repetition_penalty", 1.0, lo=0.0, lo_open=True),
        presence_penalty=_num(b, "presence_penalty", 0.0, lo=-2.0, hi=2.0),
        frequency_penalty=_num(b, "frequency_penalty", 0.0, lo=-2.0, hi=2.0),
        logit_bias=lb, pipeline=tuple(pipeline), seed=seed, max_tokens=max_tokens, min_tokens=min_tokens,
        stop_token_ids=tuple(stop_ids), bad_words=tuple(tuple(w) for w in bad), ignore_eos=bool(b.get("ignore_eos", False)),
        logprobs=want_lp, n=_num(b, "n", 1, lo=1, hi=MAX_N, integer=True))


def stop_strings_of(body: Dict[str, Any]) -> List[str]:
    stop = body.get("stop")
    if stop is None:
        return []
    if isinstance(stop, str):
        stop = [stop]
    if not isinstance(stop, list) or len(stop) > MAX_STOP_STRINGS or any(not isinstance(s, str) for s in stop):
        raise RequestError(f"stop must be a string or a list of at most {MAX_STOP_STRINGS} strings", "stop")
    for s in stop:
        if len(s.encode("utf-8")) > MAX_STOP_BYTES:
            raise RequestError(f"stop strings may be at most {MAX_STOP_BYTES} bytes", "stop")
    return [s for s in stop if s]


def thinking_budget_of(body: Dict[str, Any], default: Optional[int] = None) -> Optional[int]:
    v = body.get("thinking_token_budget", body.get("thinking_budget", default))
    if v is None:
        return None
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise RequestError("thinking_token_budget must be a non-negative integer", "thinking_token_budget")
    return v
