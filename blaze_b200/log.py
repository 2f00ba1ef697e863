"""Structured logging: levelled events as text or JSON lines, load stages with progress, request traces.

Same surface as the reference's ``crates/blaze/src/logging.rs`` (``event`` :559, ``block`` :580, load
``Stage`` with progress feeding the ``/health`` 503 body :908, per-request ``RequestTrace`` :1001-1024).
The native runtime's log callback (``kernels/src/runtime/log.cpp``) is bridged into the same sink.
"""
from __future__ import annotations

import contextvars
import json
import os
import sys
import threading
import time
from typing import Any, Dict, Optional

LEVELS = {"trace": 0, "debug": 1, "info": 2, "warn": 3, "error": 4, "off": 5}
_cfg = {"level": LEVELS.get(os.environ.get("BLAZE_LOG", "info"), 2), "format": os.environ.get("BLAZE_LOG_FORMAT", "text"),
        "color": sys.stderr.isatty(), "stream": sys.stderr}
_lock = threading.Lock()
_sinks = []
_request: contextvars.ContextVar[Optional["RequestTrace"]] = contextvars.ContextVar("blaze_request", default=None)
_COLORS = {"trace": "\x1b[90m", "debug": "\x1b[36m", "info": "\x1b[32m", "warn": "\x1b[33m", "error": "\x1b[31m"}


def configure(level: Optional[str] = None, fmt: Optional[str] = None, color: Optional[bool] = None, stream=None):
    if level is not None:
        if level not in LEVELS:
            raise ValueError(f"unknown log level {level!r}")
        _cfg["level"] = LEVELS[level]
    if fmt is not None:
        if fmt not in ("text", "json"):
            raise ValueError(f"unknown log format {fmt!r}")
        _cfg["format"] = fmt
    if color is not None:
        _cfg["color"] = color
    if stream is not None:
        _cfg["stream"] = stream


def add_sink(fn) -> None:
    """``fn(record: dict)`` receives every emitted event (tests, metrics)."""
    _sinks.append(fn)


def remove_sink(fn) -> None:
    if fn in _sinks:
        _sinks.remove(fn)


def enabled(level: str) -> bool:
    return LEVELS[level] >= _cfg["level"]


def render(rec: Dict[str, Any]) -> str:
    if _cfg["format"] == "json":
        return json.dumps(rec, separators=(",", ":"), default=str)
    ts = time.strftime("%H:%M:%S", time.localtime(rec["ts"])) + f".{int(rec['ts'] * 1000) % 1000:03d}"
    lvl = rec["level"]
    head = f"{lvl.upper():5s}"
    if _cfg["color"]:
        head = f"{_COLORS.get(lvl, '')}{head}\x1b[0m"
    fields = " ".join(f"{k}={_fmt(v)}" for k, v in rec.items() if k not in ("ts", "level", "event"))
    return f"{ts} {head} {rec['event']}" + (f" {fields}" if fields else "")


def _fmt(v) -> str:
    if isinstance(v, float):
        return f"{v:.4g}"
    s = str(v)
    return json.dumps(s) if (" " in s or "=" in s or not s) else s


def event(level: str, name: str, **fields) -> None:
    if not enabled(level):
        return
    rec = {"ts": time.time(), "level": level, "event": name}
    tr = _request.get()
    if tr is not None:
        rec["request_id"] = tr.request_id
    rec.update(fields)
    with _lock:
        for s in list(_sinks):
            s(rec)
        try:
            _cfg["stream"].write(render(rec) + "\n")
            _cfg["stream"].flush()
        except (ValueError, OSError):
            pass


def info(name, **f): event("info", name, **f)
def warn(name, **f): event("warn", name, **f)
def error(name, **f): event("error", name, **f)
def debug(name, **f): event("debug", name, **f)


def block(level: str, title: str, lines) -> None:
    """A titled multi-line block (kernel tables, tuning summaries)."""
    if not enabled(level):
        return
    if _cfg["format"] == "json":
        event(level, title, lines=list(lines))
        return
    with _lock:
        _cfg["stream"].write(f"---- {title}\n" + "".join(f"     {l}\n" for l in lines))
        _cfg["stream"].flush()


class Stage:
    """A load stage with progress; the newest one is what ``/health`` reports while loading."""
    current: Optional["Stage"] = None
    history = []

    def __init__(self, name: str, total: int = 0):
        self.name, self.total, self.done, self.t0 = name, total, 0, time.monotonic()
        Stage.current = self
        event("info", "load.stage", stage=name, total=total)

    def progress(self, done: int) -> None:
        self.done = done

    def end(self) -> None:
        dt = time.monotonic() - self.t0
        Stage.history.append((self.name, dt))
        event("info", "load.stage_done", stage=self.name, seconds=round(dt, 3))
        if Stage.current is self:
            Stage.current = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.end()

    @classmethod
    def status(cls) -> Dict[str, Any]:
        s = cls.current
        if s is None:
            return {"stage": "ready"}
        out = {"stage": s.name, "elapsed_s": round(time.monotonic() - s.t0, 2)}
        if s.total:
            out["progress"] = round(s.done / s.total, 4)
        return out


class RequestTrace:
    """Per-request timeline: admitted → first token → finished; emits ``request.*`` events."""

    def __init__(self, request_id: str):
        self.request_id = request_id
        self.t_start = time.monotonic()
        self.t_admitted = self.t_first = self.t_end = 0.0
        self.prompt_tokens = self.cached_tokens = self.output_tokens = 0

    def __enter__(self):
        self._tok = _request.set(self)
        return self

    def __exit__(self, *a):
        _request.reset(self._tok)

    def admitted(self, prompt_tokens: int, cached: int) -> None:
        self.t_admitted = time.monotonic()
        self.prompt_tokens, self.cached_tokens = prompt_tokens, cached
        event("debug", "request.admitted", request_id=self.request_id, prompt_tokens=prompt_tokens, cached=cached,
              queue_ms=round((self.t_admitted - self.t_start) * 1e3, 2))

    def first_token(self) -> None:
        if not self.t_first:
            self.t_first = time.monotonic()
            event("debug", "request.first_token", request_id=self.request_id,
                  ttft_ms=round((self.t_first - self.t_start) * 1e3, 2))

    def finished(self, reason: str, output_tokens: int) -> None:
        self.t_end = time.monotonic()
        self.output_tokens = output_tokens
        dec = self.t_end - (self.t_first or self.t_end)
        event("info", "request.finished", request_id=self.request_id, reason=reason, prompt_tokens=self.prompt_tokens,
              cached=self.cached_tokens, output_tokens=output_tokens,
              total_ms=round((self.t_end - self.t_start) * 1e3, 2),
              tpot_ms=round(dec * 1e3 / max(output_tokens - 1, 1), 3))


def current_request() -> Optional[RequestTrace]:
    return _request.get()
