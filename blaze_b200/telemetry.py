"""Fixed-bucket histograms with Prometheus text rendering (reference: ``crates/blaze/src/telemetry.rs``, 16 buckets)."""
from __future__ import annotations

import threading
from typing import List, Sequence

LATENCY_BUCKETS = (0.001, 0.0025, 0.005, 0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1.0, 2.5, 5.0, 10.0, 30.0, 60.0, 120.0)


class Histogram:
    def __init__(self, bounds: Sequence[float]):
        self.bounds = tuple(bounds)
        self.counts = [0] * (len(self.bounds) + 1)
        self.total = 0.0
        self.n = 0
        self._lock = threading.Lock()

    @classmethod
    def latency(cls) -> "Histogram":
        return cls(LATENCY_BUCKETS)

    def observe(self, v: float) -> None:
        with self._lock:
            i = 0
            while i < len(self.bounds) and v > self.bounds[i]:
                i += 1
            self.counts[i] += 1
            self.total += v
            self.n += 1

    def quantile(self, q: float) -> float:
        """Upper bound of the bucket holding quantile ``q`` (0 when empty)."""
        with self._lock:
            if self.n == 0:
                return 0.0
            target, c = q * self.n, 0
            for i, k in enumerate(self.counts):
                c += k
                if c >= target:
                    return self.bounds[i] if i < len(self.bounds) else float("inf")
        return float("inf")

    def mean(self) -> float:
        return self.total / self.n if self.n else 0.0

    def render(self, name: str, help_text: str = "") -> str:
        lines: List[str] = []
        if help_text:
            lines.append(f"# HELP {name} {help_text}")
        lines.append(f"# TYPE {name} histogram")
        with self._lock:
            c = 0
            for b, k in zip(self.bounds, self.counts):
                c += k
                lines.append(f'{name}_bucket{{le="{b}"}} {c}')
            lines.append(f'{name}_bucket{{le="+Inf"}} {self.n}')
            lines.append(f"{name}_sum {self.total}")
            lines.append(f"{name}_count {self.n}")
        return "\n".join(lines) + "\n"
