"""``inspect``: list a checkpoint's linear modules with their storage format, shapes and byte sizes
(reference: ``crates/blaze/src/inspect.rs``)."""
from __future__ import annotations

import collections

from .quant import resolve_format
from .weights import Checkpoint


def inspect_checkpoint(model_dir: str, out=print) -> int:
    ck = Checkpoint.open(model_dir)
    meta = ck.meta()
    mods = sorted({n.rsplit(".", 1)[0] for n in meta if n.endswith((".weight", ".weight_packed"))})
    by_fmt = collections.Counter()
    out(f"{model_dir}: {len(meta)} tensors, {ck.total_bytes() / 2**30:.2f} GiB, text prefix {ck.text_prefix()!r}")
    for m in mods:
        try:
            fmt = resolve_format(meta, m).value
        except KeyError:
            fmt = "?"
        w = meta.get(f"{m}.weight") or meta.get(f"{m}.weight_packed")
        by_fmt[fmt] += 1
        out(f"  {m:70s} {fmt:12s} {w[0]:8s} {tuple(w[1])}")
    out("formats: " + ", ".join(f"{k}={v}" for k, v in sorted(by_fmt.items())))
    return 0


def inspect_expert_heat(model: str, path: str, ranks: int = 8, out=print) -> int:
    """Report a routing profile (``expert_heat.ExpertHeat``): observed rows, the hottest experts, and the load imbalance
    over ``ranks`` expert-parallel ranks under the contiguous placement and under the heat-aware one."""
    import json
    import os

    import numpy as np

    from .config import ModelConfig, named_config
    from .expert_heat import ExpertHeat
    cfg = ModelConfig.load(model) if os.path.isdir(model) else named_config(model)
    E = int(getattr(cfg, "num_experts", 0) or 0)
    if E <= 0:
        out(f"{model}: not a mixture-of-experts model")
        return 1
    h = ExpertHeat.load(path, cfg.num_layers, E)
    if h is None:
        out(f"{path}: no routing profile of {E} experts")
        return 1
    rep = h.report(ranks)
    out(json.dumps(rep, indent=1))
    if ranks > 1 and E % ranks == 0:
        cont, bal = h.imbalance(ranks, recent=False), h.imbalance(ranks, h.placement(ranks, recent=False), recent=False)
        seen = np.nonzero(h.longterm.sum(axis=1) > 0)[0]
        out(f"layer: busiest-rank load over mean, {ranks} ranks (contiguous -> heat-aware)")
        for l in seen:
            out(f"  {int(l):3d}: {cont[l]:.3f} -> {bal[l]:.3f}")
    return 0


def compare_dumps(dir_a: str, dir_b: str) -> int:
    """Compare two ``BLAZE_DUMP`` directories file by file (the counterpart of the reference's ``scripts/cmp_dumps.py``):
    prints the largest and mean absolute difference of every tensor present in both, returns the number of files."""
    import os

    import torch
    names = sorted(set(os.listdir(dir_a)) & set(os.listdir(dir_b)))
    for n in names:
        a, b = torch.load(os.path.join(dir_a, n)), torch.load(os.path.join(dir_b, n))
        if a.shape != b.shape:
            print(f"{n}: shapes differ {tuple(a.shape)} vs {tuple(b.shape)}")
            continue
        d = (a - b).abs()
        print(f"{n}: max {d.max().item():.4g} mean {d.mean().item():.4g} (mean |a| {a.abs().mean().item():.4g})")
    return len(names)
