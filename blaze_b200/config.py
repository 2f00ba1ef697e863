"""Model configuration: the keys of a Hugging Face ``config.json`` that the runtime reads.

Covers the same surface as the reference's ``crates/blaze/src/config.rs:117-273``
(``text_config`` nesting, ``layer_types`` / ``full_attention_interval``, Gated DeltaNet dims,
MoE dims, RoPE with YaRN / partial rotary / M-RoPE sections, MTP layer count, eos ids), and
adds the plain Qwen3 / Qwen3-MoE architectures (ungated attention, no shared expert, norms
that are not zero-centred) which the reference refuses to load.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Dict, List, Optional


@dataclass
class RopeConfig:
    theta: float = 1.0e4
    partial_rotary_factor: float = 1.0
    mrope_section: Optional[List[int]] = None
    # YaRN
    yarn_factor: float = 1.0
    yarn_original_max_position: int = 0
    yarn_beta_fast: float = 32.0
    yarn_beta_slow: float = 1.0
    yarn_attention_factor: Optional[float] = None

    def rope_scale(self) -> float:
        """Multiplier of sin/cos under YaRN (1 when YaRN is off)."""
        if self.yarn_factor <= 1.0:
            return 1.0
        if self.yarn_attention_factor is not None:
            return float(self.yarn_attention_factor)
        return 0.1 * math.log(self.yarn_factor) + 1.0


@dataclass
class ModelConfig:
    architecture: str = "Qwen3ForCausalLM"
    model_type: str = "qwen3"
    vocab_size: int = 1024
    hidden_size: int = 256
    num_layers: int = 2
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 64
    intermediate_size: int = 512
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 32768
    rope: RopeConfig = field(default_factory=RopeConfig)
    # layer pattern: "full_attention" | "linear_attention"
    layer_types: List[str] = field(default_factory=list)
    # attention variants
    attn_output_gate: bool = False          # q_proj rows are [q | gate] per head
    qk_norm: bool = True                    # per-head RMSNorm on q and k
    zero_centered_norm: bool = False        # weights stored as (w - 1)
    attention_bias: bool = False
    # Gated DeltaNet
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel_dim: int = 4
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    shared_expert_intermediate_size: int = 0
    norm_topk_prob: bool = True
    # MTP
    mtp_num_hidden_layers: int = 0
    # Qwen4-Exp extras (``crates/blaze/src/config.rs:56-80``, :181-212): hyper-connections, per-layer n-gram embedding,
    # sparse-attention indexer
    hc_count: int = 0                       # residual streams (0 or 1: plain pre-norm residual)
    hc_lowrank: int = 16
    ple_layers: List[int] = field(default_factory=list)      # decoder layers that add an n-gram embedding (0-based)
    ngram_size: int = 3
    heads_per_ngram: int = 0
    ple_embed_dim: int = 0
    ple_conv_kernel: int = 4
    gdn_output_gate: str = "silu"           # activation of the Gated DeltaNet output gate: "silu" | "sigmoid"
    indexer_heads: int = 0                  # > 0: the checkpoint carries a sparse-attention indexer (not used: dense attention)
    indexer_head_dim: int = 0
    indexer_budget: int = 0
    indexer_compress_ratio: int = 0
    # tokens
    eos_token_ids: List[int] = field(default_factory=list)
    bos_token_id: Optional[int] = None
    # quantisation block of config.json (raw), resolved by quant.QuantConfig
    quantization_config: Optional[Dict[str, Any]] = None
    torch_dtype: str = "bfloat16"
    # vision tower (raw dict), if any
    vision_config: Optional[Dict[str, Any]] = None

    # ------------------------------------------------------------------ derived
    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def has_gdn(self) -> bool:
        return any(t == "linear_attention" for t in self.layer_types)

    @property
    def has_hc(self) -> bool:
        return self.hc_count > 1

    @property
    def rotary_dim(self) -> int:
        rd = int(self.head_dim * self.rope.partial_rotary_factor)
        return rd - (rd % 2)

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def layer_type(self, i: int) -> str:
        return self.layer_types[i] if self.layer_types else "full_attention"

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    # ------------------------------------------------------------------ loading
    @classmethod
    def load(cls, model_dir: str) -> "ModelConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            raw = json.load(f)
        cfg = cls.from_json(raw)
        # eos ids may also live in generation_config.json / tokenizer_config.json
        for name in ("generation_config.json",):
            p = os.path.join(model_dir, name)
            if os.path.exists(p):
                try:
                    with open(p) as f:
                        g = json.load(f)
                    cfg._add_eos(g.get("eos_token_id"))
                except (OSError, ValueError):
                    pass
        hq = os.path.join(model_dir, "hf_quant_config.json")
        if cfg.quantization_config is None and os.path.exists(hq):
            with open(hq) as f:
                cfg.quantization_config = {"hf_quant_config": json.load(f)}
        return cfg

    def _add_eos(self, v) -> None:
        if v is None:
            return
        ids = v if isinstance(v, list) else [v]
        for i in ids:
            if isinstance(i, int) and i not in self.eos_token_ids:
                self.eos_token_ids.append(i)

    @classmethod
    def from_json(cls, raw: Dict[str, Any]) -> "ModelConfig":
        archs = raw.get("architectures") or ["Qwen3ForCausalLM"]
        t = raw.get("text_config", raw)
        g = lambda k, d=None: t.get(k, raw.get(k, d))  # noqa: E731
        model_type = g("model_type", "qwen3")
        n_layers = int(g("num_hidden_layers", 2))
        heads = int(g("num_attention_heads", 4))
        hidden = int(g("hidden_size", 256))
        cfg = cls(
            architecture=archs[0],
            model_type=model_type,
            vocab_size=int(g("vocab_size", 1024)),
            hidden_size=hidden,
            num_layers=n_layers,
            num_heads=heads,
            num_kv_heads=int(g("num_key_value_heads", heads)),
            head_dim=int(g("head_dim", hidden // heads)),
            intermediate_size=int(g("intermediate_size", 4 * hidden)),
            rms_norm_eps=float(g("rms_norm_eps", 1e-6)),
            tie_word_embeddings=bool(g("tie_word_embeddings", False)),
            max_position_embeddings=int(g("max_position_embeddings", 32768)),
            attention_bias=bool(g("attention_bias", False)),
            linear_num_key_heads=int(g("linear_num_key_heads", 0) or 0),
            linear_num_value_heads=int(g("linear_num_value_heads", 0) or 0),
            linear_key_head_dim=int(g("linear_key_head_dim", 0) or 0),
            linear_value_head_dim=int(g("linear_value_head_dim", 0) or 0),
            linear_conv_kernel_dim=int(g("linear_conv_kernel_dim", 4) or 4),
            num_experts=int(g("num_experts", 0) or 0),
            num_experts_per_tok=int(g("num_experts_per_tok", 0) or 0),
            moe_intermediate_size=int(g("moe_intermediate_size", 0) or 0),
            shared_expert_intermediate_size=int(g("shared_expert_intermediate_size", 0) or 0),
            norm_topk_prob=bool(g("norm_topk_prob", True)),
            mtp_num_hidden_layers=int(g("mtp_num_hidden_layers", 0) or 0),
            bos_token_id=g("bos_token_id"),
            quantization_config=raw.get("quantization_config", t.get("quantization_config")),
            torch_dtype=str(g("torch_dtype", g("dtype", "bfloat16"))),
            vision_config=raw.get("vision_config"),
        )
        cfg._add_eos(g("eos_token_id"))
        hc = int(g("hc_count", 0) or 0)
        if hc > 1:
            cfg.hc_count, cfg.hc_lowrank = hc, int(g("hc_lowrank", 16) or 16)
        ple_ids = g("ple_layer_ids")
        if ple_ids:
            # the checkpoint counts layers from 1 (SGLang: layer_id + 1 in ple_layer_ids)
            cfg.ple_layers = [int(i) - 1 for i in ple_ids if int(i) >= 1]
            cfg.ngram_size = int(g("ngram_size"))
            cfg.heads_per_ngram = int(g("heads_per_ngram"))
            cfg.ple_embed_dim = int(g("ple_embed_dim"))
            cfg.ple_conv_kernel = int(g("ple_conv_kernel_size", 4) or 4)
        cfg.gdn_output_gate = str(g("output_gate_type", "silu") or "silu")
        if g("indexer_n_heads"):
            cfg.indexer_heads, cfg.indexer_head_dim = int(g("indexer_n_heads")), int(g("indexer_head_dim", 0) or 0)
            cfg.indexer_budget, cfg.indexer_compress_ratio = int(g("indexer_budget", 0) or 0), int(g("indexer_compress_ratio", 0) or 0)
        # layer pattern
        lt = g("layer_types")
        if lt:
            cfg.layer_types = [
                "linear_attention" if x in ("linear_attention", "gdn", "linear") else "full_attention" for x in lt
            ]
        else:
            interval = g("full_attention_interval")
            if interval and cfg.linear_num_value_heads > 0:
                interval = int(interval)
                cfg.layer_types = [
                    "full_attention" if (i + 1) % interval == 0 else "linear_attention" for i in range(n_layers)
                ]
            else:
                cfg.layer_types = ["full_attention"] * n_layers
        # architecture family switches
        hybrid = cfg.has_gdn or model_type in ("qwen3_next", "qwen3_5", "qwen3_5_moe", "qwen3_6", "qwen3_8", "qwen4_exp")
        cfg.attn_output_gate = bool(g("attn_output_gate", hybrid))
        cfg.zero_centered_norm = bool(g("zero_centered_norm", hybrid))
        cfg.qk_norm = bool(g("qk_norm", model_type.startswith(("qwen3", "qwen4"))))
        # rope
        rp = g("rope_parameters") or g("rope_scaling") or {}
        rope = RopeConfig(
            theta=float(rp.get("rope_theta", g("rope_theta", 1.0e4))),
            partial_rotary_factor=float(rp.get("partial_rotary_factor", g("partial_rotary_factor", 1.0))),
            mrope_section=rp.get("mrope_section"),
        )
        rtype = rp.get("rope_type", rp.get("type"))
        if rtype == "yarn":
            rope.yarn_factor = float(rp.get("factor", 1.0))
            rope.yarn_original_max_position = int(
                rp.get("original_max_position_embeddings", cfg.max_position_embeddings)
            )
            rope.yarn_beta_fast = float(rp.get("beta_fast", 32.0))
            rope.yarn_beta_slow = float(rp.get("beta_slow", 1.0))
            if rp.get("attention_factor") is not None:
                rope.yarn_attention_factor = float(rp["attention_factor"])
        cfg.rope = rope
        return cfg


def inv_freq(cfg: ModelConfig, yarn_factor_override: Optional[float] = None):
    """Rotary inverse frequencies (fp32 list), with YaRN blending when enabled.

    Same role as the reference's ``inv_freq`` (``crates/blaze/src/model.rs:991``).
    """
    rd = cfg.rotary_dim
    half = rd // 2
    r = cfg.rope
    base = [r.theta ** (-(2.0 * i) / rd) for i in range(half)]
    factor = yarn_factor_override if yarn_factor_override else r.yarn_factor
    if factor <= 1.0:
        return base
    orig = r.yarn_original_max_position or cfg.max_position_embeddings

    def corr_dim(rot):
        return (rd * math.log(orig / (rot * 2 * math.pi))) / (2 * math.log(r.theta))

    low = max(math.floor(corr_dim(r.yarn_beta_fast)), 0)
    high = min(math.ceil(corr_dim(r.yarn_beta_slow)), rd - 1)
    if low == high:
        high += 0.001
    out = []
    for i, f in enumerate(base):
        ramp = min(max((i - low) / (high - low), 0.0), 1.0)
        extrap = 1.0 - ramp  # 1 → keep original frequency
        out.append((f / factor) * (1 - extrap) + f * extrap)
    return out


# ---------------------------------------------------------------------------------- named shapes
def named_config(name: str) -> ModelConfig:
    """Shapes of the benchmark models (random-init; no checkpoint needed)."""
    n = name.lower()
    if n in ("tiny", "tiny-qwen3"):
        c = ModelConfig(vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                        intermediate_size=512, rope=RopeConfig(theta=1e6))
    elif n in ("tiny-hybrid",):
        # two Gated DeltaNet layers and two gated-attention layers with a small MoE: the Qwen3-Next layer pattern in miniature
        c = ModelConfig(architecture="Qwen3NextForCausalLM", model_type="qwen3_next", vocab_size=1024, hidden_size=256,
                        num_layers=4, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=512, num_experts=8,
                        num_experts_per_tok=2, moe_intermediate_size=128, shared_expert_intermediate_size=128,
                        linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=128, linear_value_head_dim=64,
                        linear_conv_kernel_dim=4, attn_output_gate=True, zero_centered_norm=True,
                        rope=RopeConfig(theta=1e6, partial_rotary_factor=0.25))
        c.layer_types = ["linear_attention", "full_attention", "linear_attention", "full_attention"]
    elif n in ("tiny-qwen4",):
        # the hybrid in miniature with two residual streams and an n-gram embedding on two of its layers
        c = named_config("tiny-hybrid")
        c.architecture, c.model_type = "Qwen4ExpForCausalLM", "qwen4_exp"
        c.hc_count, c.hc_lowrank = 2, 8
        c.ple_layers, c.ngram_size, c.heads_per_ngram, c.ple_embed_dim, c.ple_conv_kernel = [0, 2], 3, 2, 16, 4
        c.eos_token_ids = [1]
    elif n in ("qwen3-8b",):
        c = ModelConfig(vocab_size=151936, hidden_size=4096, num_layers=36, num_heads=32, num_kv_heads=8,
                        head_dim=128, intermediate_size=12288, rope=RopeConfig(theta=1e6))
    elif n in ("qwen3-32b",):
        c = ModelConfig(vocab_size=151936, hidden_size=5120, num_layers=64, num_heads=64, num_kv_heads=8,
                        head_dim=128, intermediate_size=25600, rope=RopeConfig(theta=1e6), mtp_num_hidden_layers=1)
    elif n in ("qwen3-30b-a3b",):
        c = ModelConfig(architecture="Qwen3MoeForCausalLM", model_type="qwen3_moe", vocab_size=151936,
                        hidden_size=2048, num_layers=48, num_heads=32, num_kv_heads=4, head_dim=128,
                        intermediate_size=6144, num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
                        norm_topk_prob=True, rope=RopeConfig(theta=1e6))
    elif n in ("qwen3-next-80b-a3b",):
        c = ModelConfig(architecture="Qwen3NextForCausalLM", model_type="qwen3_next", vocab_size=151936,
                        hidden_size=2048, num_layers=48, num_heads=16, num_kv_heads=2, head_dim=256,
                        intermediate_size=5120, num_experts=512, num_experts_per_tok=10, moe_intermediate_size=512,
                        shared_expert_intermediate_size=512, linear_num_key_heads=16, linear_num_value_heads=32,
                        linear_key_head_dim=128, linear_value_head_dim=128, linear_conv_kernel_dim=4,
                        attn_output_gate=True, zero_centered_norm=True,
                        rope=RopeConfig(theta=1e7, partial_rotary_factor=0.25))
        c.layer_types = ["full_attention" if (i + 1) % 4 == 0 else "linear_attention" for i in range(48)]
    else:
        raise ValueError(f"unknown model shape {name!r}")
    if not c.layer_types:
        c.layer_types = ["full_attention"] * c.num_layers
    return c
