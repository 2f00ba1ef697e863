"""Decoder model: Qwen3 dense, Qwen3-MoE and the Qwen3-Next style hybrid (Gated DeltaNet + gated
attention + shared expert), loaded from safetensors or random-initialised, with tensor-parallel cuts.

Mirrors the structure of the reference's ``crates/blaze/src/model.rs`` (``load`` :1031-1661 for the
tensor names and TP cuts :1110-1282, ``forward`` :2330-2551, ``attention`` :2897, ``gdn`` :3513,
``mlp`` :3594) while adding what it refuses: plain Qwen3 attention (no gate), MoE without a shared
expert, and MoE under tensor / expert parallelism (``model.rs:1077-1080``).
"""
from __future__ import annotations

import os

import math
from typing import Dict, List, Optional

import torch

from ..batch import StepBatch
from ..config import ModelConfig, inv_freq
from ..kv import KVCache
from ..linear import Cut, Linear, part
from ..quant import Format


class Attn:
    index = None         # qwen4.Indexer of a sparse-attention model (class default: none)

    def __init__(self):
        self.qkv: Linear = None
        self.o: Linear = None
        self.q_norm: Optional[torch.Tensor] = None
        self.k_norm: Optional[torch.Tensor] = None
        self.heads = 0
        self.kv_heads = 0


class Gdn:
    def __init__(self):
        self.in_proj: Linear = None      # rows [q | k | v | z | b | a]
        self.out_proj: Linear = None
        self.conv_w: torch.Tensor = None  # [conv_dim, k]
        self.A_log: torch.Tensor = None
        self.dt_bias: torch.Tensor = None
        self.norm_w: torch.Tensor = None
        self.k_heads = 0
        self.v_heads = 0


class DenseMlp:
    def __init__(self):
        self.gate_up: Linear = None
        self.down: Linear = None


class Experts:
    """Routed experts of one layer (this rank's share under expert parallelism)."""

    def __init__(self):
        self.gate_up: List[Linear] = []
        self.down: List[Linear] = []
        self.num_experts = 0             # global expert count
        self.first = 0                   # first global expert id held locally
        self.count = 0                   # number held locally
        self.cuda_pack = None

    def forward_one(self, e: int, x: torch.Tensor) -> torch.Tensor:
        from ..ops import ref
        le = e - self.first
        return self.down[le].ref(ref.silu_mul(self.gate_up[le].ref(x)))


class MoeMlp:
    def __init__(self):
        self.router: Linear = None
        self.experts: Experts = None
        self.shared: Optional[DenseMlp] = None
        self.shared_gate: Optional[Linear] = None
        self.top_k = 0
        self.renorm = True


class Layer:
    def __init__(self):
        self.kind = "full_attention"
        self.input_norm: torch.Tensor = None
        self.post_norm: torch.Tensor = None
        self.attn: Optional[Attn] = None
        self.gdn: Optional[Gdn] = None
        self.mlp = None
        # Qwen4-Exp: hyper-connections around the two blocks (in place of the norms above) and an n-gram embedding
        self.hc_attn = self.hc_mlp = None
        self.ple = None


_PROFILE_PHASES = os.environ.get("BLAZE_PROFILE_PHASES", "0") == "1"
_FUSED_HEAD = os.environ.get("BLAZE_FUSED_HEAD", "1") != "0"
_DUMP_DIR = os.environ.get("BLAZE_DUMP", "")       # directory for per-layer tensor dumps (``model.rs:2087`` ``BLAZE_DUMP``)
_dump_step = [0]


def _dump(name: str, t) -> None:
    """Save a tensor of the current forward pass as fp32 for offline comparison (``inspect.compare_dumps``)."""
    os.makedirs(_DUMP_DIR, exist_ok=True)
    if hasattr(t, "dense") and getattr(t, "dense") is not None:
        t = t.dense
    if isinstance(t, torch.Tensor):
        torch.save(t.detach().float().cpu(), os.path.join(_DUMP_DIR, f"step{_dump_step[0]:04d}_{name}.pt"))


class _PhaseTimer:
    """CUDA-event timers around the phases of a forward pass (collective + norm, attention / GDN mixer, MLP), summed over
    the layers and logged as one ``model.phases`` event per step — the counterpart of the reference's ``--profile-prefill``
    (``model.rs:2233-2252``).  Enabled by ``BLAZE_PROFILE_PHASES=1``; never active inside a graph capture."""

    def __init__(self, device):
        self.on = torch.device(device).type == "cuda"
        self.marks = []
        self.nvtx = self.on and os.environ.get("BLAZE_NVTX", "0") == "1"      # also open an NVTX range per phase
        self._open = False

    def mark(self, name: str) -> None:
        if self.on:
            if self.nvtx:
                if self._open:
                    torch.cuda.nvtx.range_pop()
                torch.cuda.nvtx.range_push(name)
                self._open = True
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.marks.append((name, ev))

    def finish(self, **fields) -> None:
        if self.nvtx and self._open:
            torch.cuda.nvtx.range_pop()
            self._open = False
        if not self.on or not self.marks:
            return
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        end.synchronize()
        tot = {}
        for (name, ev), nxt in zip(self.marks, [e for _, e in self.marks[1:]] + [end]):
            tot[name] = tot.get(name, 0.0) + ev.elapsed_time(nxt)
        from .. import log
        log.event("info", "model.phases", **{k.replace("+", "_"): round(v, 3) for k, v in tot.items()}, **fields)


class TPInfo:
    """Rank layout.  ``group`` does the collectives (None on one rank)."""

    def __init__(self, rank: int = 0, world: int = 1, group=None, ep: bool = False, expert_order=None):
        self.rank, self.world, self.group, self.ep = rank, world, group, ep
        # [layers, experts]: slot j of a layer holds checkpoint expert expert_order[layer][j].  The router's rows and the
        # experts are stored in slot order, so expert parallelism (contiguous slots per rank) realises any placement
        # without a change to routing or kernels (expert_heat.ExpertHeat.order_for turns a placement into this table).
        self.expert_order = expert_order


class Model:
    def __init__(self, cfg: ModelConfig, device="cpu", dtype=torch.bfloat16, tp: Optional[TPInfo] = None, ops=None,
                 first_layer: int = 0, last_layer: Optional[int] = None):
        from ..ops import get_ops
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.tp = tp or TPInfo()
        self.ops = ops or get_ops(device)
        self.layers: List[Layer] = []
        self.embed: torch.Tensor = None
        self.final_norm: torch.Tensor = None
        self.lm_head: Linear = None
        self.first_layer = first_layer                        # pipeline stage range [first, last)
        self.last_layer = cfg.num_layers if last_layer is None else last_layer
        self.inv_freq = torch.tensor(inv_freq(cfg), dtype=torch.float32, device=device)
        self.rope_scale = cfg.rope.rope_scale()
        self.attn_scale = cfg.head_dim ** -0.5
        self.gdn_chunked = False
        self.capture_layers: List[int] = []                   # hidden states kept for drafters
        self.captured: Dict[int, torch.Tensor] = {}
        self.gdn_records: Dict[int, tuple] = {}               # per GDN layer: inputs of the last step that deferred state
        self.ple_records: Dict = {}                           # per n-gram embedding layer: the same for its convolution
        self.hc_final = None                                  # hyper-connection that reads the streams out (last stage)
        if cfg.has_hc and (self.tp.world > 1 or first_layer != 0 or self.last_layer != cfg.num_layers):
            # as in the reference (crates/blaze/src/model.rs:1077): the streams are not cut over ranks or stages
            raise ValueError("hyper-connection models run on one rank (no tensor or pipeline parallelism)")
        if cfg.indexer_heads and (self.tp.world > 1 or first_layer != 0 or self.last_layer != cfg.num_layers):
            raise ValueError("sparse-attention (indexer) models run on one rank (no tensor or pipeline parallelism)")
        if cfg.ple_layers and not cfg.has_hc:
            raise ValueError("per-layer n-gram embeddings are defined on hyper-connection streams (hc_count > 1)")
        self.weight_format = Format.DENSE

    @property
    def is_first_stage(self) -> bool:
        return self.first_layer == 0

    @property
    def is_last_stage(self) -> bool:
        return self.last_layer == self.cfg.num_layers

    # ================================================================== construction
    @classmethod
    def random_init(cls, cfg: ModelConfig, fmt: Format = Format.DENSE, seed: int = 0, device="cpu",
                    dtype=torch.bfloat16, tp: Optional[TPInfo] = None, std: float = 0.02, ops=None,
                    first_layer: int = 0, last_layer: Optional[int] = None, lm_head_fmt: Format = Format.DENSE,
                    router_std: Optional[float] = None) -> "Model":
        """N(0, std) weights from ``seed`` (norm weights 1, or 0 when zero-centred), quantised to ``fmt``.

        Full tensors are generated and quantised first and cut afterwards, so a TP=n model is an
        exact cut of the TP=1 model with the same seed.
        """
        m = cls(cfg, device, dtype, tp, ops, first_layer, last_layer)
        m.weight_format = fmt
        tpw, tpr = m.tp.world, m.tp.rank
        gen = torch.Generator(device=device)
        D, H = cfg.head_dim, cfg.hidden_size

        def rnd(n, k, tag, s=std):
            gen.manual_seed((seed * 1000003 + tag) & 0x7FFFFFFF)
            return torch.randn(n, k, generator=gen, device=device, dtype=torch.float32) * s

        def ones(n):
            return (torch.zeros if cfg.zero_centered_norm else torch.ones)(n, dtype=dtype, device=device)

        def lin(w, cut, f=fmt, segments=None, unit=1):
            if cut == Cut.COLS and tpw > 1:
                a, b = part(w.shape[1], tpr, tpw)
                w = w[:, a:b]
                return _tag(Linear.from_dense(w, f, dtype=dtype, segments=segments), Cut.COLS)
            if cut == Cut.ROWS and tpw > 1 and segments:
                pieces, r = [], 0
                for n in segments:
                    a, b = part(n // unit, tpr, tpw)
                    pieces.append(w[r + a * unit:r + b * unit])
                    r += n
                segs = [p.shape[0] for p in pieces]
                return _tag(Linear.from_dense(torch.cat(pieces), f, dtype=dtype, segments=segs), Cut.ROWS)
            if cut == Cut.ROWS and tpw > 1:
                a, b = part(w.shape[0] // unit, tpr, tpw)
                w = w[a * unit:b * unit]
            return _tag(Linear.from_dense(w, f, dtype=dtype, segments=segments), cut)

        def _tag(l, cut):
            l.cut = cut
            return l

        if m.is_first_stage or cfg.tie_word_embeddings:
            m.embed = rnd(cfg.vocab_size, H, 1).to(dtype)
        for i in range(m.first_layer, m.last_layer):
            L = Layer()
            L.kind = cfg.layer_type(i)
            base = 100 + i * 50
            L.input_norm, L.post_norm = ones(H), ones(H)
            if cfg.has_hc:
                from . import qwen4
                L.hc_attn = qwen4.random_hc(rnd, H, cfg.hc_count, cfg.hc_lowrank, 7000 + i * 20, dtype)
                L.hc_mlp = qwen4.random_hc(rnd, H, cfg.hc_count, cfg.hc_lowrank, 7000 + i * 20 + 5, dtype)
                if i in cfg.ple_layers:
                    L.ple = qwen4.random_ple(rnd, cfg, 7000 + i * 20 + 10, dtype, device,
                                             lambda w: _tag(Linear.from_dense(w, Format.DENSE, dtype=dtype), Cut.ALL))
            if L.kind == "full_attention":
                A = Attn()
                A.heads, A.kv_heads = cfg.num_heads // tpw, max(cfg.num_kv_heads // tpw, 1)
                qrows = cfg.num_heads * D * (2 if cfg.attn_output_gate else 1)
                qunit = D * (2 if cfg.attn_output_gate else 1)
                wq, wk, wv = rnd(qrows, H, base + 1), rnd(cfg.num_kv_heads * D, H, base + 2), rnd(cfg.num_kv_heads * D, H, base + 3)
                if tpw > 1:
                    qa, qb = part(cfg.num_heads, tpr, tpw)
                    wq = wq[qa * qunit:qb * qunit]
                    if cfg.num_kv_heads >= tpw:
                        ka, kb = part(cfg.num_kv_heads, tpr, tpw)
                    else:   # replicate KV heads: rank r uses head r * kv_heads // world
                        ka = tpr * cfg.num_kv_heads // tpw
                        kb = ka + 1
                    wk, wv = wk[ka * D:kb * D], wv[ka * D:kb * D]
                A.qkv = _tag(Linear.from_dense(torch.cat([wq, wk, wv]), fmt, dtype=dtype,
                                               segments=[wq.shape[0], wk.shape[0], wv.shape[0]]), Cut.ROWS)
                A.o = lin(rnd(H, cfg.num_heads * D, base + 4), Cut.COLS)
                if cfg.qk_norm:
                    A.q_norm, A.k_norm = ones(D), ones(D)
                if cfg.indexer_heads:
                    from . import qwen4
                    A.index = qwen4.Indexer()
                    A.index.proj = _tag(Linear.from_dense(rnd((cfg.indexer_heads + 1) * cfg.indexer_head_dim, H, base + 6, 0.1),
                                                          Format.DENSE, dtype=dtype), Cut.ALL)
                    A.index.q_norm = torch.zeros(cfg.indexer_head_dim, dtype=dtype, device=device)
                    A.index.k_norm = torch.zeros(cfg.indexer_head_dim, dtype=dtype, device=device)
                L.attn = A
            else:
                G = Gdn()
                hk, hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
                dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
                G.k_heads, G.v_heads = hk // tpw, hv // tpw
                segs_full = [hk * dk, hk * dk, hv * dv, hv * dv, hv, hv]
                units = [dk, dk, dv, dv, 1, 1]
                ws = [rnd(n, H, base + 10 + j) for j, n in enumerate(segs_full)]
                if tpw > 1:
                    ws = [w[part(w.shape[0] // u, tpr, tpw)[0] * u:part(w.shape[0] // u, tpr, tpw)[1] * u]
                          for w, u in zip(ws, units)]
                # the small b / a projections stay dense: their outputs feed gates
                G.in_proj = _tag(Linear.from_dense(torch.cat(ws), fmt, dtype=dtype, segments=[w.shape[0] for w in ws]), Cut.ROWS)
                G.out_proj = lin(rnd(H, hv * dv, base + 17), Cut.COLS)
                conv_dim = 2 * hk * dk + hv * dv
                cw = rnd(conv_dim, cfg.linear_conv_kernel_dim, base + 18, 0.2)
                if tpw > 1:
                    qa, qb = part(hk, tpr, tpw)
                    va, vb = part(hv, tpr, tpw)
                    cw = torch.cat([cw[qa * dk:qb * dk], cw[hk * dk + qa * dk:hk * dk + qb * dk],
                                    cw[2 * hk * dk + va * dv:2 * hk * dk + vb * dv]])
                G.conv_w = cw.to(dtype)
                al = torch.log(torch.linspace(1.0, 8.0, hv, device=device))
                G.A_log = al[part(hv, tpr, tpw)[0]:part(hv, tpr, tpw)[1]].float().contiguous()
                G.dt_bias = torch.zeros(G.v_heads, dtype=torch.float32, device=device)
                G.norm_w = torch.ones(dv, dtype=dtype, device=device)
                L.gdn = G
            if cfg.is_moe:
                M = MoeMlp()
                M.top_k, M.renorm = cfg.num_experts_per_tok, cfg.norm_topk_prob
                order = m._expert_slots(i)
                rw = rnd(cfg.num_experts, H, base + 20, router_std or std)
                M.router = _tag(Linear.from_dense(rw if order is None else rw[order], Format.DENSE, dtype=dtype), Cut.ALL)
                E = Experts()
                E.num_experts = cfg.num_experts
                I = cfg.moe_intermediate_size
                if m.tp.ep:      # expert parallel: whole experts per rank
                    E.first, end = part(cfg.num_experts, tpr, tpw)
                    E.count = end - E.first
                else:
                    E.first, E.count = 0, cfg.num_experts
                gen.manual_seed((seed * 1000003 + base + 21) & 0x7FFFFFFF)
                for slot in range(E.first, E.first + E.count):
                    e = slot if order is None else int(order[slot])
                    gen.manual_seed((seed * 1000003 + (base + 21) * 4099 + e) & 0x7FFFFFFF)
                    wg = torch.randn(2 * I, H, generator=gen, device=device) * std
                    wd = torch.randn(H, I, generator=gen, device=device) * std
                    if not m.tp.ep and tpw > 1:   # tensor-parallel experts: cut the intermediate dim
                        a, b = part(I, tpr, tpw)
                        wg = torch.cat([wg[a:b], wg[I + a:I + b]])
                        wd = wd[:, a:b]
                    E.gate_up.append(Linear.from_dense(wg, fmt, dtype=dtype, segments=[wg.shape[0] // 2] * 2))
                    E.down.append(Linear.from_dense(wd, fmt, dtype=dtype))
                M.experts = E
                if cfg.shared_expert_intermediate_size:
                    S = DenseMlp()
                    Is = cfg.shared_expert_intermediate_size
                    S.gate_up = lin(rnd(2 * Is, H, base + 30), Cut.ROWS, segments=[Is, Is])
                    S.down = lin(rnd(H, Is, base + 31), Cut.COLS)
                    M.shared = S
                    M.shared_gate = _tag(Linear.from_dense(rnd(1, H, base + 32), Format.DENSE, dtype=dtype), Cut.ALL)
                L.mlp = M
            else:
                P = DenseMlp()
                I = cfg.intermediate_size
                P.gate_up = lin(rnd(2 * I, H, base + 40), Cut.ROWS, segments=[I, I])
                P.down = lin(rnd(H, I, base + 41), Cut.COLS)
                L.mlp = P
            m.layers.append(L)
        if m.is_last_stage:
            m.final_norm = ones(H)
            if cfg.has_hc:
                from . import qwen4
                m.hc_final = qwen4.random_hc(rnd, H, cfg.hc_count, cfg.hc_lowrank, 6990, dtype, inject=False)
            if cfg.tie_word_embeddings:
                wl = m.embed.float()
            else:
                wl = rnd(cfg.vocab_size, H, 2)
            if tpw > 1:
                a, b = part(cfg.vocab_size, tpr, tpw)
                wl = wl[a:b]
            m.lm_head = _tag(Linear.from_dense(wl, lm_head_fmt, dtype=dtype), Cut.ROWS if tpw > 1 else Cut.ALL)
        return m

    @classmethod
    def load(cls, model_dir: str, device="cpu", dtype=torch.bfloat16, tp: Optional[TPInfo] = None, ops=None,
             first_layer: int = 0, last_layer: Optional[int] = None, cfg: Optional[ModelConfig] = None) -> "Model":
        """Load a local safetensors checkpoint (tensor names of ``model.rs:1110-1282``)."""
        from ..weights import Checkpoint
        cfg = cfg or ModelConfig.load(model_dir)
        ck = Checkpoint.open(model_dir)
        m = cls(cfg, device, dtype, tp, ops, first_layer, last_layer)
        p = ck.text_prefix()
        tpw, tpr = m.tp.world, m.tp.rank
        D = cfg.head_dim

        def vec(name, cut_heads=None):
            t = ck.get(name)
            return t.to(dtype).to(device)

        def rows(t, n_units, unit):
            if tpw == 1:
                return t
            a, b = part(n_units, tpr, tpw)
            return t[a * unit:b * unit]

        def load_lin(mods, cut, units=None):
            return Linear.load(ck, mods, cut, tpr, tpw, dtype, device)

        if m.is_first_stage or cfg.tie_word_embeddings:
            m.embed = ck.get(f"{p}embed_tokens.weight").to(dtype).to(device)
        for i in range(m.first_layer, m.last_layer):
            L = Layer()
            L.kind = cfg.layer_type(i)
            lp = f"{p}layers.{i}."
            if cfg.has_hc:
                from . import qwen4
                L.hc_attn = qwen4.load_hc(ck, lp + "attn_hyper_connection.", dtype, device)
                L.hc_mlp = qwen4.load_hc(ck, lp + "mlp_hyper_connection.", dtype, device)
                if i in cfg.ple_layers:
                    L.ple = qwen4.load_ple(ck, lp + "ple.", cfg, dtype, device, lambda mods: load_lin(mods, Cut.ALL))
            else:
                L.input_norm = vec(lp + "input_layernorm.weight")
                L.post_norm = vec(lp + "post_attention_layernorm.weight")
            if L.kind == "full_attention":
                A = Attn()
                A.heads, A.kv_heads = cfg.num_heads // tpw, max(cfg.num_kv_heads // tpw, 1)
                sp = lp + "self_attn."
                A.qkv = _load_stacked_heads(ck, [sp + "q_proj", sp + "k_proj", sp + "v_proj"],
                                            [D * (2 if cfg.attn_output_gate else 1), D, D],
                                            [cfg.num_heads, cfg.num_kv_heads, cfg.num_kv_heads], tpr, tpw, dtype, device)
                A.o = load_lin([sp + "o_proj"], Cut.COLS)
                if cfg.qk_norm and (sp + "q_norm.weight") in ck:
                    A.q_norm, A.k_norm = vec(sp + "q_norm.weight"), vec(sp + "k_norm.weight")
                if cfg.indexer_heads:
                    # tensor names of crates/blaze/src/model.rs:1127-1134
                    from . import qwen4
                    A.index = qwen4.Indexer()
                    A.index.proj = load_lin([sp + "indexer.index_qk_proj"], Cut.ALL)
                    A.index.q_norm, A.index.k_norm = vec(sp + "indexer.q_layernorm.weight"), vec(sp + "indexer.k_layernorm.weight")
                L.attn = A
            else:
                G = Gdn()
                hk, hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
                dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
                G.k_heads, G.v_heads = hk // tpw, hv // tpw
                gp = lp + "linear_attn."
                if (gp + "in_proj_qkv.weight") in ck or (gp + "in_proj_qkv.weight_packed") in ck:
                    # rows [q|k|v] in one module: cut each third on head boundaries
                    G.in_proj = _load_gdn_in_proj(ck, gp, hk, hv, dk, dv, tpr, tpw, dtype, device)
                else:
                    G.in_proj = _load_gdn_fused(ck, gp, hk, hv, dk, dv, tpr, tpw, dtype, device)
                G.out_proj = load_lin([gp + "out_proj"], Cut.COLS)
                cw = ck.get(gp + "conv1d.weight").float()
                cw = cw.view(cw.shape[0], -1)
                if tpw > 1:
                    qa, qb = part(hk, tpr, tpw)
                    va, vb = part(hv, tpr, tpw)
                    cw = torch.cat([cw[qa * dk:qb * dk], cw[hk * dk + qa * dk:hk * dk + qb * dk],
                                    cw[2 * hk * dk + va * dv:2 * hk * dk + vb * dv]])
                G.conv_w = cw.to(dtype).to(device)
                G.A_log = rows(ck.get(gp + "A_log").float(), hv, 1).contiguous().to(device)
                G.dt_bias = rows(ck.get(gp + "dt_bias").float(), hv, 1).contiguous().to(device)
                G.norm_w = vec(gp + "norm.weight")
                L.gdn = G
            mp = lp + "mlp."
            if cfg.is_moe and (mp + "gate.weight") in ck:
                M = MoeMlp()
                M.top_k, M.renorm = cfg.num_experts_per_tok, cfg.norm_topk_prob
                M.router = Linear.load(ck, [mp + "gate"], Cut.ALL, 0, 1, dtype, device)
                order = m._expert_slots(i)
                if order is not None:
                    if M.router.fmt != Format.DENSE:
                        raise ValueError("an expert placement needs an unquantised router weight")
                    M.router.w = M.router.w[order.to(M.router.w.device)].contiguous()
                    if getattr(M.router, "bias", None) is not None:
                        M.router.bias = M.router.bias[order.to(M.router.bias.device)].contiguous()
                E = Experts()
                E.num_experts = cfg.num_experts
                if m.tp.ep:
                    E.first, end = part(cfg.num_experts, tpr, tpw)
                    E.count = end - E.first
                else:
                    E.first, E.count = 0, cfg.num_experts
                for slot in range(E.first, E.first + E.count):
                    e = slot if order is None else int(order[slot])
                    ep = f"{mp}experts.{e}."
                    if m.tp.ep or tpw == 1:
                        E.gate_up.append(Linear.load(ck, [ep + "gate_proj", ep + "up_proj"], Cut.ALL, 0, 1, dtype, device))
                        E.down.append(Linear.load(ck, [ep + "down_proj"], Cut.ALL, 0, 1, dtype, device))
                    else:
                        E.gate_up.append(Linear.load(ck, [ep + "gate_proj", ep + "up_proj"], Cut.ROWS, tpr, tpw, dtype, device))
                        E.down.append(Linear.load(ck, [ep + "down_proj"], Cut.COLS, tpr, tpw, dtype, device))
                M.experts = E
                if (mp + "shared_expert.gate_proj.weight") in ck or (mp + "shared_expert.gate_proj.weight_packed") in ck:
                    S = DenseMlp()
                    S.gate_up = load_lin([mp + "shared_expert.gate_proj", mp + "shared_expert.up_proj"], Cut.ROWS)
                    S.down = load_lin([mp + "shared_expert.down_proj"], Cut.COLS)
                    M.shared = S
                    if (mp + "shared_expert_gate.weight") in ck:
                        M.shared_gate = Linear.load(ck, [mp + "shared_expert_gate"], Cut.ALL, 0, 1, dtype, device)
                L.mlp = M
            else:
                P = DenseMlp()
                P.gate_up = load_lin([mp + "gate_proj", mp + "up_proj"], Cut.ROWS)
                P.down = load_lin([mp + "down_proj"], Cut.COLS)
                L.mlp = P
            m.layers.append(L)
        if m.is_last_stage:
            if cfg.has_hc:
                from . import qwen4
                m.hc_final = qwen4.load_hc(ck, f"{p}hyper_connection_mixer.", dtype, device, inject=False)
            else:
                m.final_norm = vec(f"{p}norm.weight")
            if cfg.tie_word_embeddings or "lm_head.weight" not in ck:
                wl = m.embed.float()
                if tpw > 1:
                    a, b = part(cfg.vocab_size, tpr, tpw)
                    wl = wl[a:b]
                m.lm_head = Linear.from_dense(wl, Format.DENSE, dtype=dtype)
                m.lm_head.cut = Cut.ROWS if tpw > 1 else Cut.ALL
            else:
                m.lm_head = Linear.load(ck, ["lm_head"], Cut.ROWS if tpw > 1 else Cut.ALL, tpr, tpw, dtype, device)
        fmts = [L.mlp.gate_up.fmt for L in m.layers if isinstance(L.mlp, DenseMlp)]
        m.weight_format = fmts[0] if fmts else Format.DENSE
        return m

    # ================================================================== forward
    def forward(self, batch: StepBatch, kv: KVCache, hidden_in: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run this stage's layers.  Returns the residual stream ``[T, hidden]`` *before* the final norm
        on the last stage (use :meth:`head` for logits), or the rows to hand to the next stage.

        Every block returns its output as this rank's *partial* sums; the reduction over ranks happens together with
        the residual add and the next RMSNorm — one fused peer-memory kernel when the group has one
        (``reduce_norm`` in ``crates/blaze/src/model.rs:2555``), else all-reduce followed by the norm kernel."""
        ops, cfg = self.ops, self.cfg
        if hidden_in is not None:
            x = hidden_in
        else:
            x = ops.embed(self.embed, batch.tokens)
            if batch.embed_over:
                # image tokens: the vision tower's rows take the place of the pad tokens' embeddings
                for r0, t in batch.embed_over:
                    x[r0:r0 + t.shape[0]] = t.to(device=x.device, dtype=x.dtype)
        if cfg.has_hc:
            return self._forward_streams(x, batch, kv)
        fused = self._fused()
        rope = ops.rope_tables(self, batch)
        residual = None          # full rows, or this rank's row shard on the reduce+norm path
        kind = "full"            # x is: "full" rows | "partial" sums to reduce | "acc" (summed in a symmetric buffer to re-zero)
        prof = _PhaseTimer(self.device) if _PROFILE_PHASES and not torch.cuda.is_current_stream_capturing() else None
        for li, L in enumerate(self.layers):
            gi = self.first_layer + li
            first = L.attn.qkv if L.attn is not None else L.gdn.in_proj
            if gi in self.capture_layers:
                self.captured[gi] = self._materialise(x, residual, kind, fused, keep=True)
            if prof: prof.mark("reduce+norm")
            h, residual = self._reduce_norm(x, residual, kind, L.input_norm, first, fused, defer=True)
            if prof: prof.mark("mixer")
            if L.kind == "full_attention":
                x, kind = self._attention(L.attn, h, batch, kv, gi, rope, fused)
            else:
                x, kind = self._gdn(L.gdn, h, batch, kv, gi, fused)
            nxt = L.mlp.gate_up if isinstance(L.mlp, DenseMlp) else None
            if prof: prof.mark("reduce+norm")
            h, residual = self._reduce_norm(x, residual, kind, L.post_norm, nxt, fused, defer=nxt is not None)
            if prof: prof.mark("mlp")
            x, kind = self._mlp(L.mlp, h, fused, gi)
            if _DUMP_DIR and kind == "full" and not (x.is_cuda and torch.cuda.is_current_stream_capturing()):
                _dump(f"layer{gi:03d}_mlp_out", x)
        if prof:
            prof.finish(rows=int(batch.num_rows), layers=len(self.layers))
        if _DUMP_DIR:
            _dump_step[0] += 1
        return self._materialise(x, residual, kind, fused)

    def _forward_streams(self, x, batch: StepBatch, kv: KVCache) -> torch.Tensor:
        """The layer loop of a hyper-connection model (``scripts/ref_qwen4.py`` :318-340): the embedding is copied into
        ``hc_count`` streams; every block reads a gated mix of the normed streams and writes its output back into each stream
        through a gate; layers with an n-gram embedding add it to the streams first.  Returns the streams ``[T, hc * hidden]``
        (:meth:`final_hidden` reads them out)."""
        from . import qwen4
        ops, cfg = self.ops, self.cfg
        hc, eps = cfg.hc_count, cfg.rms_norm_eps
        rope = ops.rope_tables(self, batch)
        streams = x.repeat(1, hc)
        state = kv.ple
        w1 = w0 = None
        if state is not None:
            w1, w0 = qwen4.window_tokens(batch, state)
            if batch.h_gdn_defer is not None:
                self.ple_records = {}
        for li, L in enumerate(self.layers):
            gi = self.first_layer + li
            if L.ple is not None:
                streams = qwen4.ple_apply(self, L.ple, gi, streams, batch, state, w1, w0)
            h, n = qwen4.hc_mix(streams, L.hc_attn, hc, eps)
            if L.kind == "full_attention":
                y, _ = self._attention(L.attn, h, batch, kv, gi, rope, None)
            else:
                y, _ = self._gdn(L.gdn, h, batch, kv, gi, None)
            streams = qwen4.hc_combine(streams, n, L.hc_attn, y, hc)
            h, n = qwen4.hc_mix(streams, L.hc_mlp, hc, eps)
            y, _ = self._mlp(L.mlp, h, None, gi)
            streams = qwen4.hc_combine(streams, n, L.hc_mlp, y, hc)
            if _DUMP_DIR and not (streams.is_cuda and torch.cuda.is_current_stream_capturing()):
                _dump(f"layer{gi:03d}_streams", streams)
        if state is not None:
            qwen4.advance_history(batch, batch.tokens, state, skip=batch.h_gdn_defer)
        return streams

    def _fused(self):
        g = self.tp.group
        return g.fused if (g is not None and g.world > 1 and getattr(g, "fused", None) is not None and self.ops.is_cuda) else None

    def _reduce_norm(self, x, residual, kind, w, quant_for, fused, defer: bool = False):
        """``defer``: the result goes straight into ``ops.linear`` (attention / GDN input projection, dense MLP), which
        may then take over the wait for the peers' rows."""
        ops, cfg = self.ops, self.cfg
        eps, zc = cfg.rms_norm_eps, cfg.zero_centered_norm
        if fused is not None and fused.mode in ("reduce_norm", "rs_push"):
            if residual is None:                       # first norm of the stage: shard the residual stream by rows
                residual = fused.shard_rows(x)
                h, _ = ops.norm(x, None, w, eps, zc, quant_for=quant_for)
                return h, residual
            if kind != "partial":                      # complete rows: rank 0 contributes them, the others zeros
                x = self._as_partial(x, fused)
            return fused.reduce_norm(x, residual, w, eps, zc, quant_for, defer=defer), residual
        if kind == "acc":                              # already summed by the GEMM epilogue; re-zero the buffer while reading
            return ops.norm(x, residual, w, eps, zc, quant_for=quant_for, zero_src=True)
        if kind == "partial":
            x = ops.all_reduce(x, self.tp.group)
        return ops.norm(x, residual, w, eps, zc, quant_for=quant_for)

    def _as_partial(self, x, fused):
        """Present complete rows as partial sums: rank 0 contributes them, the others contribute zeros."""
        buf = fused.next_input(x.shape[0], x.shape[1])
        if self.tp.rank == 0:
            buf.copy_(x)
        else:
            buf.zero_()
        return buf

    def _materialise(self, x, residual, kind, fused, keep: bool = False):
        """The complete residual stream on every rank."""
        ops = self.ops
        if fused is not None and fused.mode in ("reduce_norm", "rs_push") and residual is not None:
            if kind != "partial":
                x = self._as_partial(x, fused)
            res = residual.clone() if keep else residual
            return fused.reduce_norm(x, res, None, self.cfg.rms_norm_eps, False, None)
        if kind == "partial":
            x = ops.all_reduce(x, self.tp.group)
        out = ops.add(x, residual) if residual is not None else x
        if kind == "acc" and not keep:
            if residual is None:
                out = x.clone()
            x.zero_()
        return out

    def _row_cut(self, lin, a, rows, fused):
        """Row-parallel projection: returns (output, kind)."""
        ops = self.ops
        if fused is None:
            return ops.linear(lin, a), ("partial" if self.tp.world > 1 else "full")
        if fused.mode == "gemm_red":
            return fused.gemm_allreduce(ops, lin, a, rows), "acc"
        if fused.mode == "rs_push" and lin.N % 32 == 0 and fused.group.world * fused.rows_per(rows) * lin.N * 2 <= fused.slot_bytes:
            # the GEMM's epilogue scatters the partial rows to their owner ranks; reduce_norm picks them up from the slots
            return fused.gemm_push(ops, lin, a, rows), "partial"
        return ops.linear(lin, a, out=fused.next_input(rows, lin.N)), "partial"

    def _out_buf(self, fused, rows, cols):
        return fused.next_input(rows, cols) if fused is not None else None

    def _attention(self, A: Attn, h, batch, kv, gi, rope, fused=None):
        ops = self.ops
        qkv = ops.linear(A.qkv, h)
        q, gate = ops.attn_prep_store(qkv, A, self, batch, kv, gi, rope)
        if A.index is not None:
            from . import qwen4
            sel = qwen4.qsa_step(self, A.index, h, batch, kv, gi)
            o = ops.attention(q, self, batch, kv, gi, self.attn_scale, allowed=sel) if sel is not None else \
                ops.attention(q, self, batch, kv, gi, self.attn_scale)
        else:
            o = ops.attention(q, self, batch, kv, gi, self.attn_scale)
        if gate is not None:
            o = ops.mul_sigmoid(o, gate.reshape(o.shape))
        return self._row_cut(A.o, o, o.shape[0], fused)

    def _gdn(self, G: Gdn, h, batch, kv, gi, fused=None):
        ops, cfg = self.ops, self.cfg
        dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        proj = ops.linear(G.in_proj, h)
        nq = 2 * G.k_heads * dk + G.v_heads * dv
        nz = G.v_heads * dv
        mixed, z = proj[:, :nq], proj[:, nq:nq + nz]
        b, a = proj[:, nq + nz:nq + nz + G.v_heads], proj[:, nq + nz + G.v_heads:]
        if batch.gdn_defer is not None:
            # speculative rows: keep what the recurrence consumed, so that the accepted prefix can be replayed
            # (the reference's verify records, crates/blaze/src/model.rs:1322, :3364)
            self.gdn_records[gi] = (mixed, b, a)
        o = ops.gdn(mixed, z, b, a, G, self, batch, kv, gi)
        return self._row_cut(G.out_proj, o, o.shape[0], fused)

    def gdn_replay(self, batch: StepBatch, rows: torch.Tensor, kv: KVCache) -> None:
        """Advance the recurrent state of every GDN layer over ``rows`` (indices into the recorded step's rows, grouped by
        sequence as ``batch`` describes) — the accepted prefix of a verify step whose state update was deferred
        (reference: ``commit_replay``, crates/blaze/src/model.rs:3484)."""
        idx = rows.long()
        for li, L in enumerate(self.layers):
            gi = self.first_layer + li
            if L.gdn is None:
                continue
            rec = self.gdn_records.get(gi)
            if rec is None:
                raise RuntimeError("no deferred step to replay")
            mixed, b, a = rec
            ba = torch.stack([b[idx], a[idx]]).contiguous()      # one buffer: the kernels take a common row stride
            self.ops.gdn(mixed[idx].contiguous(), None, ba[0], ba[1], L.gdn, self, batch, kv, gi, state_only=True)
        if kv.ple is not None:
            from . import qwen4
            qwen4.ple_replay(self, batch, rows, kv.ple)

    heat = None          # expert_heat.ExpertHeat when routing statistics are collected
    _order_dev = None    # tp.expert_order on the device (slot -> checkpoint expert), for the statistics

    def _expert_slots(self, layer: int):
        """Slot order of ``layer``'s experts (a LongTensor), or None when experts keep their checkpoint order."""
        eo = self.tp.expert_order
        if eo is None:
            return None
        row = torch.as_tensor(eo[layer]).long()
        if sorted(row.tolist()) != list(range(self.cfg.num_experts)):
            raise ValueError(f"expert order of layer {layer} is not a permutation of {self.cfg.num_experts} experts")
        return row

    def _mlp(self, M, h, fused=None, layer: int = 0):
        """Returns (output, kind) with kind as in :meth:`forward`."""
        ops = self.ops
        tp = self.tp.world > 1
        if isinstance(M, DenseMlp):
            a = ops.linear_swiglu(M.gate_up, h, quant_for=M.down)
            return self._row_cut(M.down, a, a.rows if hasattr(a, "rows") else a.shape[0], fused)
        hd = h.dense if hasattr(h, "dense") and h.dense is not None else h
        logits = ops.linear(M.router, hd, out_dtype=torch.float32)
        if ops.is_cuda:
            w, ids = ops.router_topk(logits, M.top_k, M.renorm, M.experts.first, M.experts.count)
        else:
            w, ids = ops.router_topk(logits, M.top_k, M.renorm)
        if self.heat is not None:
            if self.tp.expert_order is not None:
                if self._order_dev is None:
                    self._order_dev = torch.as_tensor(self.tp.expert_order).long().to(ids.device)
                self.heat.observe(layer, self._order_dev[layer][ids.long()])      # the profile is in checkpoint numbering
            else:
                self.heat.observe(layer, ids)
        # Tokens are replicated across the ranks, so expert parallelism needs no dispatch: every rank runs the routed
        # pairs whose expert it holds and the partial outputs are summed by the reduce + norm that follows.
        y = ops.moe(hd, w, ids, M.experts)
        routed_partial = tp
        if M.shared is not None:
            s = ops.linear(M.shared.down, ops.linear_swiglu(M.shared.gate_up, hd, quant_for=M.shared.down))
            if tp and not routed_partial:
                s = ops.all_reduce(s, self.tp.group)
            if M.shared_gate is not None:
                y = ops.add_sigmoid_scaled(y, s, ops.linear(M.shared_gate, hd))
            else:
                y = ops.add(y, s)
        return y, ("partial" if routed_partial else "full")

    # ------------------------------------------------------------------ head
    def final_hidden(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if rows is not None:
            x = x[rows.long()]
        if self.hc_final is not None:
            # the read-out mix of the streams stands where the final norm does (``scripts/ref_qwen4.py`` :341)
            from . import qwen4
            return qwen4.hc_mix(x, self.hc_final, self.cfg.hc_count, self.cfg.rms_norm_eps)[0]
        h, _ = self.ops.norm(x, None, self.final_norm, self.cfg.rms_norm_eps, self.cfg.zero_centered_norm)
        return h

    def head(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """fp32 logits ``[R, vocab]`` (this rank's vocab shard gathered over TP)."""
        h = self.final_hidden(x, rows)
        logits = self.ops.linear(self.lm_head, h, out_dtype=torch.float32)
        if self.tp.world > 1 and self.tp.group is not None:
            logits = self.tp.group.all_gather_cols(logits)
        return logits

    def greedy(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Greedy token per row; under TP each rank reduces its shard and (value, index) pairs are merged
        (``model.rs:2669`` ``greedy_sharded``)."""
        h = self.final_hidden(x, rows)
        tp = self.tp.world > 1 and self.tp.group is not None
        if self.ops.is_cuda and _FUSED_HEAD:
            # the logits never reach memory: the head GEMM's epilogue keeps each tile's best column
            if tp:
                idx, val = self.ops.linear_argmax(self.lm_head, h, index_offset=self.tp.rank * self.lm_head.N, want_values=True)
                return self.tp.group.merge_pairs(idx, val)
            return self.ops.linear_argmax(self.lm_head, h)
        logits = self.ops.linear(self.lm_head, h, out_dtype=torch.float32)
        if tp:
            return self.tp.group.argmax_sharded(self.ops, logits, self.lm_head.N)
        return self.ops.argmax(logits)

    def weight_bytes(self) -> int:
        n = 0
        for L in self.layers:
            for obj in (L.attn, L.gdn, L.mlp):
                if obj is None:
                    continue
                for v in vars(obj).values():
                    if isinstance(v, Linear):
                        n += v.nbytes()
                    elif isinstance(v, DenseMlp):
                        n += v.gate_up.nbytes() + v.down.nbytes()
                    elif isinstance(v, Experts):
                        n += sum(l.nbytes() for l in v.gate_up) + sum(l.nbytes() for l in v.down)
        if self.lm_head is not None:
            n += self.lm_head.nbytes()
        if self.embed is not None:
            n += self.embed.numel() * self.embed.element_size()
        return n


# ---------------------------------------------------------------------------------- loader helpers
def _load_stacked_heads(ck, mods, units, counts, rank, world, dtype, device) -> Linear:
    """Stack q/k/v cutting each on head boundaries; KV heads replicate when world > kv_heads."""
    parts = []
    for mod, unit, n in zip(mods, units, counts):
        full = Linear.load(ck, [mod], Cut.ALL, 0, 1, dtype, "cpu")
        if world > 1:
            if n >= world:
                a, b = part(n, rank, world)
            else:
                a = rank * n // world
                b = a + 1
            full = _slice_rows(full, a * unit, b * unit)
        parts.append(full)
    lin = Linear._stack(parts) if len(parts) > 1 else parts[0]
    lin.cut = Cut.ROWS
    return lin.to(device)


def _slice_rows(lin: Linear, a: int, b: int) -> Linear:
    out = Linear(lin.fmt, b - a, lin.K)
    out.block, out.act_quant = lin.block, lin.act_quant
    out.w = lin.w[a:b].contiguous()
    if lin.sf is not None:
        if lin.fmt == Format.FP8_BLOCK:
            bn = lin.block[0]
            assert a % bn == 0
            out.sf = lin.sf[a // bn:-(-b // bn)].contiguous()
        else:
            out.sf = lin.sf[a:b].contiguous()
    if lin.alpha is not None:
        out.alpha = lin.alpha[a:b].contiguous()
    if lin.bias is not None:
        out.bias = lin.bias[a:b].contiguous()
    return out


def _load_gdn_in_proj(ck, gp, hk, hv, dk, dv, rank, world, dtype, device) -> Linear:
    qkv = Linear.load(ck, [gp + "in_proj_qkv"], Cut.ALL, 0, 1, dtype, "cpu")
    z = Linear.load(ck, [gp + "in_proj_z"], Cut.ALL, 0, 1, dtype, "cpu")
    b = Linear.load(ck, [gp + "in_proj_b"], Cut.ALL, 0, 1, dtype, "cpu")
    a = Linear.load(ck, [gp + "in_proj_a"], Cut.ALL, 0, 1, dtype, "cpu")
    ka, kb = part(hk, rank, world)
    va, vb = part(hv, rank, world)
    pieces = [_slice_rows(qkv, ka * dk, kb * dk), _slice_rows(qkv, hk * dk + ka * dk, hk * dk + kb * dk),
              _slice_rows(qkv, 2 * hk * dk + va * dv, 2 * hk * dk + vb * dv), _slice_rows(z, va * dv, vb * dv),
              _slice_rows(b, va, vb), _slice_rows(a, va, vb)]
    if len({p.fmt for p in pieces}) != 1:
        raise ValueError("GDN in_proj modules mix formats")
    lin = Linear._stack(pieces)
    lin.cut = Cut.ROWS
    return lin.to(device)


def _load_gdn_fused(ck, gp, hk, hv, dk, dv, rank, world, dtype, device) -> Linear:
    """Upstream Qwen3-Next layout: ``in_proj_qkvz`` (per key head: q, k, v-group, z-group) and ``in_proj_ba``."""
    qkvz = Linear.load(ck, [gp + "in_proj_qkvz"], Cut.ALL, 0, 1, dtype, "cpu")
    ba = Linear.load(ck, [gp + "in_proj_ba"], Cut.ALL, 0, 1, dtype, "cpu")
    if qkvz.fmt != Format.DENSE or ba.fmt != Format.DENSE:
        raise ValueError("fused GDN projections are supported for dense checkpoints only")
    rep = hv // hk
    per = 2 * dk + 2 * rep * dv
    w = qkvz.w.view(hk, per, -1)
    q, k = w[:, :dk], w[:, dk:2 * dk]
    v, z = w[:, 2 * dk:2 * dk + rep * dv], w[:, 2 * dk + rep * dv:]
    wb = ba.w.view(hk, 2 * rep, -1)
    bb, aa = wb[:, :rep], wb[:, rep:]
    ka, kb = part(hk, rank, world)
    rows = [q[ka:kb].reshape(-1, w.shape[-1]), k[ka:kb].reshape(-1, w.shape[-1]), v[ka:kb].reshape(-1, w.shape[-1]),
            z[ka:kb].reshape(-1, w.shape[-1]), bb[ka:kb].reshape(-1, w.shape[-1]), aa[ka:kb].reshape(-1, w.shape[-1])]
    lin = Linear.from_dense(torch.cat(rows).float(), Format.DENSE, dtype=dtype)
    lin.cut = Cut.ROWS
    return lin.to(device)
