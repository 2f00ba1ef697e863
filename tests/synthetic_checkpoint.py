"""Write a dense random-init model as a local checkpoint with the tensor names real checkpoints use (``config.json`` plus
one safetensors file), so that the loader can be tested without a download.  Covers the hybrid decoder (gated attention,
Gated DeltaNet, MoE with a shared expert) and the Qwen4-Exp extras (hyper-connections, per-layer n-gram embedding; names
as in the reference's ``scripts/ref_qwen4.py``)."""
import json
import os

import torch

from blaze_b200.models.qwen3 import DenseMlp
from blaze_b200.weights import save_safetensors


QUANTISED = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def quantised(name: str, w: torch.Tensor, fmt: str):
    """Tensors of one linear module ``name`` (without ``.weight``) in a checkpoint format: ``nvfp4`` (compressed-tensors names),
    ``nvfp4_modelopt``, ``mxfp8``, ``fp8_block`` (128 x 128), ``fp8_channel``, ``fp8_tensor``."""
    from blaze_b200 import quant
    w = w.float()
    if fmt in ("nvfp4", "nvfp4_modelopt"):
        packed, sf, g = quant.nvfp4_quantize(w)
        if fmt == "nvfp4":
            return {name + ".weight_packed": packed, name + ".weight_scale": sf, name + ".weight_global_scale": (1.0 / g).reshape(1).float()}
        return {name + ".weight": packed, name + ".weight_scale": sf, name + ".weight_scale_2": g.reshape(1).float()}
    if fmt == "mxfp8":
        q, e8 = quant.mxfp8_quantize(w)
        return {name + ".weight": q, name + ".weight_scale": e8.view(torch.uint8)}
    if fmt == "fp8_block":
        q, sc = quant.fp8_block_quantize(w)
        return {name + ".weight": q, name + ".weight_scale_inv": sc.float()}
    if fmt == "fp8_channel":
        q, sc = quant.fp8_channel_quantize(w)
        return {name + ".weight": q, name + ".weight_scale": sc.float().reshape(-1, 1)}
    if fmt == "fp8_tensor":
        sc = (w.abs().amax() / 448.0).clamp_min(1e-12)
        return {name + ".weight": quant.to_e4m3(w / sc), name + ".weight_scale": sc.reshape(1).float()}
    raise ValueError(fmt)


def write(model, out_dir: str, prefix: str = "model.language_model.", ple_shards: int = 2, fmt: str = "dense") -> None:
    """``fmt``: the format of the attention and MLP projections (routers, gates, norms and embeddings stay bf16)."""
    cfg = model.cfg
    D, H = cfg.head_dim, cfg.hidden_size
    t = {}

    def put(name, w):
        if fmt != "dense" and name.endswith(".weight") and name[:-7].rsplit(".", 1)[-1] in QUANTISED and "shared_expert_gate" not in name:
            t.update(quantised(name[:-7], w.detach(), fmt))
            return
        t[name] = w.detach().float().to(torch.bfloat16 if w.is_floating_point() else w.dtype).contiguous()
    put(prefix + "embed_tokens.weight", model.embed)
    put("lm_head.weight", model.lm_head.dequant())
    for i, L in enumerate(model.layers):
        lp = f"{prefix}layers.{i}."
        if cfg.has_hc:
            for name, blk in (("attn_hyper_connection.", L.hc_attn), ("mlp_hyper_connection.", L.hc_mlp)):
                put(lp + name + "hc_norm.weight", blk.norm)
                put(lp + name + "input_mix_weight_down.weight", blk.down)
                put(lp + name + "input_mix_weight_up.weight", blk.up)
                put(lp + name + "block_inject_weight.weight", blk.inject)
            if L.ple is not None:
                P, e = L.ple, lp + "ple.ple_embedding."
                t[e + "layer_multipliers"], t[e + "ngram_heads_vocab_sizes"], t[e + "ngram_heads_offsets"] = P.mult, P.sizes, P.offs
                rows = (P.table.shape[0] + ple_shards - 1) // ple_shards
                for s in range(ple_shards):
                    put(e + f"ngram_embedding.shard_{s}.weight", P.table[s * rows:(s + 1) * rows])
                put(lp + "ple.key_proj.weight", P.key.dequant())
                put(lp + "ple.value_proj.weight", P.value.dequant())
                for n in ("norm_key", "norm_query", "norm_conv"):
                    put(lp + f"ple.{n}.weight", getattr(P, n))
                put(lp + "ple.conv1d.weight", P.conv_w[:, None, :])
        else:
            put(lp + "input_layernorm.weight", L.input_norm)
            put(lp + "post_attention_layernorm.weight", L.post_norm)
        if L.attn is not None:
            A, sp = L.attn, lp + "self_attn."
            w = A.qkv.dequant()
            nq = cfg.num_heads * D * (2 if cfg.attn_output_gate else 1)
            nk = cfg.num_kv_heads * D
            put(sp + "q_proj.weight", w[:nq])
            put(sp + "k_proj.weight", w[nq:nq + nk])
            put(sp + "v_proj.weight", w[nq + nk:])
            put(sp + "o_proj.weight", A.o.dequant())
            if A.q_norm is not None:
                put(sp + "q_norm.weight", A.q_norm)
                put(sp + "k_norm.weight", A.k_norm)
            if A.index is not None:
                put(sp + "indexer.index_qk_proj.weight", A.index.proj.dequant())
                put(sp + "indexer.q_layernorm.weight", A.index.q_norm)
                put(sp + "indexer.k_layernorm.weight", A.index.k_norm)
        else:
            G, gp = L.gdn, lp + "linear_attn."
            hk, hv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
            w = G.in_proj.dequant()
            nq, nz = 2 * hk * dk + hv * dv, hv * dv
            put(gp + "in_proj_qkv.weight", w[:nq])
            put(gp + "in_proj_z.weight", w[nq:nq + nz])
            put(gp + "in_proj_b.weight", w[nq + nz:nq + nz + hv])
            put(gp + "in_proj_a.weight", w[nq + nz + hv:])
            put(gp + "out_proj.weight", G.out_proj.dequant())
            put(gp + "conv1d.weight", G.conv_w[:, None, :])
            t[gp + "A_log"], t[gp + "dt_bias"] = G.A_log.float(), G.dt_bias.float()
            put(gp + "norm.weight", G.norm_w)
        mp = lp + "mlp."
        if isinstance(L.mlp, DenseMlp):
            w = L.mlp.gate_up.dequant()
            put(mp + "gate_proj.weight", w[:w.shape[0] // 2])
            put(mp + "up_proj.weight", w[w.shape[0] // 2:])
            put(mp + "down_proj.weight", L.mlp.down.dequant())
        else:
            M = L.mlp
            put(mp + "gate.weight", M.router.dequant())
            for e in range(M.experts.count):
                w = M.experts.gate_up[e].dequant()
                put(f"{mp}experts.{e}.gate_proj.weight", w[:w.shape[0] // 2])
                put(f"{mp}experts.{e}.up_proj.weight", w[w.shape[0] // 2:])
                put(f"{mp}experts.{e}.down_proj.weight", M.experts.down[e].dequant())
            if M.shared is not None:
                w = M.shared.gate_up.dequant()
                put(mp + "shared_expert.gate_proj.weight", w[:w.shape[0] // 2])
                put(mp + "shared_expert.up_proj.weight", w[w.shape[0] // 2:])
                put(mp + "shared_expert.down_proj.weight", M.shared.down.dequant())
                put(mp + "shared_expert_gate.weight", M.shared_gate.dequant())
    if cfg.has_hc:
        for n, w in (("hc_norm", model.hc_final.norm), ("input_mix_weight_down", model.hc_final.down), ("input_mix_weight_up", model.hc_final.up)):
            put(f"{prefix}hyper_connection_mixer.{n}.weight", w)
    else:
        put(prefix + "norm.weight", model.final_norm)
    text = {"model_type": cfg.model_type, "vocab_size": cfg.vocab_size, "hidden_size": H, "num_hidden_layers": cfg.num_layers,
            "num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_kv_heads, "head_dim": D,
            "intermediate_size": cfg.intermediate_size, "rms_norm_eps": cfg.rms_norm_eps, "layer_types": cfg.layer_types,
            "linear_num_key_heads": cfg.linear_num_key_heads, "linear_num_value_heads": cfg.linear_num_value_heads,
            "linear_key_head_dim": cfg.linear_key_head_dim, "linear_value_head_dim": cfg.linear_value_head_dim,
            "linear_conv_kernel_dim": cfg.linear_conv_kernel_dim, "num_experts": cfg.num_experts,
            "num_experts_per_tok": cfg.num_experts_per_tok, "moe_intermediate_size": cfg.moe_intermediate_size,
            "shared_expert_intermediate_size": cfg.shared_expert_intermediate_size, "norm_topk_prob": cfg.norm_topk_prob,
            "rope_parameters": {"rope_theta": cfg.rope.theta, "partial_rotary_factor": cfg.rope.partial_rotary_factor},
            "eos_token_id": cfg.eos_token_ids[0] if cfg.eos_token_ids else None, "output_gate_type": cfg.gdn_output_gate}
    if cfg.indexer_heads:
        text.update({"indexer_n_heads": cfg.indexer_heads, "indexer_head_dim": cfg.indexer_head_dim,
                     "indexer_budget": cfg.indexer_budget, "indexer_compress_ratio": cfg.indexer_compress_ratio})
    if cfg.has_hc:
        text.update({"hc_count": cfg.hc_count, "hc_lowrank": cfg.hc_lowrank})
    if cfg.ple_layers:
        text.update({"ple_layer_ids": [i + 1 for i in cfg.ple_layers], "ngram_size": cfg.ngram_size, "heads_per_ngram": cfg.heads_per_ngram,
                     "ple_embed_dim": cfg.ple_embed_dim, "ple_conv_kernel_size": cfg.ple_conv_kernel})
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump({"architectures": [cfg.architecture], "text_config": text}, f)
    save_safetensors(os.path.join(out_dir, "model.safetensors"), t)
