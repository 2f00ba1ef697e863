"""Kernel autotuner: times candidate configurations per row-count bucket and keeps the winners in a JSON cache.

Reference: ``crates/blaze/src/tune.rs`` (row ``BUCKETS`` :13, candidates split x tiles :129, cache file
``~/.cache/blaze/tune-sm*.json`` :182, ``tune`` :243) and ``attn_tune.rs`` (attention split cache per GPU / rank).
Here the tunables are the GEMM N-tile (128 / 256) and CTA cap per (kind, N, K, row bucket), and the kv-split count of
the decode attention kernel per (batch bucket, context bucket).
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Iterable, Optional, Tuple

BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192)


def bucket(rows: int) -> int:
    for b in BUCKETS:
        if rows <= b:
            return b
    return BUCKETS[-1]


def cache_path(sm: int = 100, sms: int = 148, rank: int = 0) -> str:
    root = os.environ.get("BLAZE_CACHE_DIR", os.path.join(os.path.expanduser("~"), ".cache", "blaze_b200"))
    return os.path.join(root, f"tune-sm{sm}-{sms}sm-r{rank}.json")


class Tuning:
    def __init__(self, path: Optional[str] = None):
        self.path = path or cache_path()
        self.table: Dict[str, Dict] = {}
        self.dirty = False
        try:
            with open(self.path) as f:
                self.table = json.load(f)
        except (OSError, ValueError):
            self.table = {}

    @staticmethod
    def key(kind: str, *shape) -> str:
        return kind + ":" + "x".join(str(s) for s in shape)

    def get(self, kind: str, *shape) -> Optional[Dict]:
        return self.table.get(self.key(kind, *shape))

    def put(self, kind: str, shape: Tuple, cfg: Dict, ms: float) -> None:
        self.table[self.key(kind, *shape)] = {**cfg, "ms": round(ms, 5)}
        self.dirty = True

    def save(self) -> None:
        if not self.dirty:
            return
        os.makedirs(os.path.dirname(self.path), exist_ok=True)
        tmp = self.path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(self.table, f, indent=1, sort_keys=True)
        os.replace(tmp, self.path)
        self.dirty = False

    def tune(self, kind: str, shape: Tuple, candidates: Iterable[Dict], run: Callable[[Dict], float]) -> Dict:
        """Time every candidate with ``run(cfg) -> ms`` (the caller does warm-up and event timing) and keep the best."""
        hit = self.get(kind, *shape)
        if hit is not None:
            return hit
        best, best_ms = None, float("inf")
        for c in candidates:
            try:
                ms = run(c)
            except Exception:
                continue
            if ms < best_ms:
                best, best_ms = c, ms
        if best is None:
            raise RuntimeError(f"no candidate ran for {kind} {shape}")
        self.put(kind, shape, best, best_ms)
        return self.table[self.key(kind, *shape)]


def gemm_candidates(kind: int, N: int, K: int, rows: int):
    """Kernel variants worth timing for one linear layer at ``rows`` rows: the one-CTA-per-tile kernel with 128- or
    256-column tiles, and for decode-sized steps the cluster split-K kernel with its K-slice counts."""
    out = [{"kernel": "tc", "bn": 128}]
    if N % 256 == 0 and rows > 128:
        out.append({"kernel": "tc", "bn": 256})
    if rows <= 512:
        bk = {0: 64, 1: 256}.get(kind, 128)
        for ks in (1, 2, 3, 4, 6, 8):
            if ks <= (K + bk - 1) // bk:
                out.append({"kernel": "sk", "ks": ks})
    return out


def tune_linear(ops, lin, rows: int, tuning: Tuning, iters: int = 5) -> Dict:
    """Pick the N-tile for ``lin`` at ``rows`` rows on the current device."""
    import torch
    pk = ops.pack(lin)
    x = torch.randn(rows, lin.K, device=ops.device).bfloat16()
    xin = ops.quantize_rows(x, lin) if ops._qmode(lin) else x

    out = torch.empty(rows, lin.N, dtype=torch.bfloat16, device=ops.device)

    def call(cfg):
        if cfg["kernel"] == "sk":
            ops.linear(lin, xin, out=out, sk=cfg["ks"])
        else:
            ops.linear(lin, xin, out=out, bn=cfg["bn"], wide=False, sk=False)

    def run(cfg):
        # a captured graph of back-to-back calls: a single small launch timed from the host measures the host
        call(cfg)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                call(cfg)
        g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters
    return tuning.tune(f"gemm{pk['kind']}", (lin.N, lin.K, bucket(rows)), gemm_candidates(pk["kind"], lin.N, lin.K, rows), run)


def tune_model(model, rows: Iterable[int] = (256,), tuning: Optional[Tuning] = None, save: bool = True) -> Tuning:
    """Time the kernel variants of every distinct linear shape of ``model`` at the given row counts and install the table
    on its op set (``ops.tuning``), so that ``CudaOps.linear`` picks the measured winner per (format, N, K, row bucket).
    The table is kept in the JSON cache of this device, so later runs only load it (reference: the start-up GEMV tuning of
    ``crates/blaze/src/model.rs:1568-1590`` and ``tune.rs:243``)."""
    ops = model.ops
    if not getattr(ops, "is_cuda", False):
        return tuning or Tuning()
    import torch
    props = torch.cuda.get_device_properties(ops.device)
    t = tuning or Tuning(cache_path(props.major * 10 + props.minor, props.multi_processor_count, model.tp.rank))
    seen = set()
    for L in model.layers:
        lins = []
        if L.attn is not None:
            lins += [L.attn.qkv, L.attn.o]
        if L.gdn is not None:
            lins += [L.gdn.in_proj, L.gdn.out_proj]
        mlp = L.mlp
        if hasattr(mlp, "down") and hasattr(mlp, "gate_up") and not hasattr(mlp, "experts"):
            lins += [mlp.down]          # gate_up runs with the SwiGLU epilogue, which has one variant
        for lin in lins:
            for r in rows:
                key = (int(lin.fmt.value if hasattr(lin.fmt, "value") and isinstance(lin.fmt.value, int) else hash(lin.fmt) & 0xff),
                       lin.N, lin.K, bucket(r))
                if key in seen:
                    continue
                seen.add(key)
                tune_linear(ops, lin, r, t)
    if save:
        t.save()
    ops.tuning = t
    return t
