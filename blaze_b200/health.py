"""Engine health: step-latency outlier detection and a periodic ``engine.stats`` event
(reference: ``crates/blaze/src/health.rs`` — outlier = 30x the running mean and > 5 s; stats every 5 s, :119)."""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Optional

from . import log


@dataclass
class StepShape:
    rows: int = 0
    seqs: int = 0


class Health:
    OUTLIER_FACTOR = 30.0
    OUTLIER_MIN_S = 5.0
    TICK_S = 5.0

    def __init__(self):
        self.mean_s = 0.0
        self.steps = 0
        self.outliers = 0
        self.errors = 0                 # steps that failed (device status, sampler, model exception)
        self.last_tick = time.monotonic()
        self.tokens_since_tick = 0
        self.steps_since_tick = 0
        self.last_outlier: Optional[str] = None

    def step(self, seconds: float, shape: StepShape) -> bool:
        """Record one step; returns True when it is a latency outlier."""
        self.steps += 1
        self.steps_since_tick += 1
        self.tokens_since_tick += shape.rows
        out = self.steps > 8 and seconds > self.OUTLIER_MIN_S and seconds > self.OUTLIER_FACTOR * self.mean_s
        if out:
            self.outliers += 1
            self.last_outlier = f"step took {seconds:.2f}s (mean {self.mean_s * 1e3:.1f} ms) rows={shape.rows} seqs={shape.seqs}"
            log.warn("engine.slow_step", seconds=round(seconds, 3), mean_ms=round(self.mean_s * 1e3, 2), rows=shape.rows)
        else:
            self.mean_s = seconds if self.steps == 1 else 0.95 * self.mean_s + 0.05 * seconds
        return out

    def tick(self, **extra) -> bool:
        now = time.monotonic()
        dt = now - self.last_tick
        if self.TICK_S <= 0 or dt < self.TICK_S:          # an interval of 0 switches the periodic summary off
            return False
        log.info("engine.stats", steps_per_s=round(self.steps_since_tick / dt, 2),
                 rows_per_s=round(self.tokens_since_tick / dt, 1), mean_step_ms=round(self.mean_s * 1e3, 3), **extra)
        self.last_tick, self.tokens_since_tick, self.steps_since_tick = now, 0, 0
        return True
