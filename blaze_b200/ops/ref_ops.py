"""The oracle op set: composes :mod:`blaze_b200.ops.ref` functions behind the model's op interface."""
from __future__ import annotations

from typing import Optional

import torch

from . import ref
from ..linear import Linear, QuantAct


class RefOps:
    is_cuda = False
    name = "ref"

    # -------------------------------------------------------------- basics
    def embed(self, table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
        return table[tokens.long()]

    def norm(self, x, residual, w, eps, zero_centered=False, quant_for: Optional[Linear] = None):
        return ref.rmsnorm(x, w, eps, residual, zero_centered)

    def linear(self, lin: Linear, x, out_dtype=None):
        return lin.ref(x, out_dtype)

    def silu_mul(self, gu, quant_for: Optional[Linear] = None):
        return ref.silu_mul(gu)

    def linear_swiglu(self, lin: Linear, x, quant_for: Optional[Linear] = None):
        return ref.silu_mul(self.linear(lin, x))

    def mul_sigmoid(self, x, gate):
        return (x.float() * torch.sigmoid(gate.float())).to(x.dtype)

    def add(self, a, b):
        return (a.float() + b.float()).to(a.dtype)

    def add_sigmoid_scaled(self, a, b, gate_logit):
        """a + b * sigmoid(gate_logit) with the sigmoid rounded to the activation dtype (``ops_basic.cu:175``)."""
        s = torch.sigmoid(gate_logit.float()).to(a.dtype).float()
        return (a.float() + b.float() * s).to(a.dtype)

    def all_reduce(self, x, group=None):
        if group is None or group.world == 1:
            return x
        return group.all_reduce(x)

    # -------------------------------------------------------------- attention
    def rope_tables(self, model, batch):
        inv = model.inv_freq
        pos = batch.positions3 if getattr(batch, "positions3", None) is not None else batch.positions
        return ref.rope_cos_sin(pos, inv, model.rope_scale, model.cfg.rope.mrope_section)

    def attn_prep_store(self, qkv, attn, model, batch, kv, layer_idx, rope):
        cfg = model.cfg
        cos, sin = rope
        q, k, v, gate = ref.attn_prep(qkv, attn.heads, attn.kv_heads, cfg.head_dim, attn.q_norm, attn.k_norm,
                                      cfg.rms_norm_eps, cos, sin, gated=cfg.attn_output_gate,
                                      zero_centered=cfg.zero_centered_norm, rotate=getattr(model, "kv_rotate", False))
        valid = batch.slot_mapping >= 0
        if kv.kv_dtype in ("nvfp4", "nvfp4_4over6"):
            kv.write_fp4(layer_idx, k[valid], v[valid], batch.slot_mapping[valid])
        elif kv.layout == "umma":
            kl, vl = kv.logical_kv(layer_idx)
            ref.kv_write(kl, vl, k[valid], v[valid], batch.slot_mapping[valid])
            # write back in kernel layout
            D = cfg.head_dim
            P, H = kl.shape[0], kl.shape[1]
            kb = kl.view(torch.uint8).view(P, H, 2, 8, D // 16, 16).permute(0, 1, 2, 4, 3, 5).reshape(P, H, -1)
            vb = vl.view(torch.uint8).transpose(2, 3).reshape(P, H, -1)
            kv.kv[layer_idx][:, :, 0] = kb
            kv.kv[layer_idx][:, :, 1] = vb
        else:
            ref.kv_write(kv.k[layer_idx], kv.v[layer_idx], k[valid], v[valid], batch.slot_mapping[valid])
        return q, gate

    def attention(self, q, model, batch, kv, layer_idx, scale, allowed=None):
        """``allowed``: per sequence a bool ``[q_len, ctx_len]`` of the keys its rows may see (None: all), a sparse selection."""
        kl, vl = kv.logical_kv(layer_idx)
        o = ref.paged_attention(q, kl, vl, kv.block_table, batch.h_slots, batch.h_q_start, batch.h_ctx_len, scale,
                                tree_mask=getattr(batch, "tree_mask", None), allowed=allowed)
        return o.reshape(q.shape[0], -1)

    # -------------------------------------------------------------- MoE
    def router_topk(self, logits, k, renorm=True):
        return ref.router_topk(logits, k, renorm)

    def moe(self, x, topk_w, topk_id, experts):
        """experts: an object with ``num_experts`` and ``forward_one(e, x)``."""
        return ref.moe_forward(x, topk_w, topk_id, experts.forward_one, experts.num_experts)

    # -------------------------------------------------------------- GDN
    def gdn(self, mixed_qkv, z, b, a, gdn, model, batch, kv, layer_idx, state_only: bool = False):
        """Causal conv + gates + delta-rule recurrence + gated norm, one sequence at a time.  Sequences flagged in
        ``batch.h_gdn_defer`` leave their state untouched; ``state_only`` advances the states and returns nothing."""
        cfg = model.cfg
        dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        hk, hv = gdn.k_heads, gdn.v_heads
        T = mixed_qkv.shape[0]
        out = torch.empty(T, hv * dv, dtype=mixed_qkv.dtype, device=mixed_qkv.device)
        conv_state, rec_state = kv.conv_state[layer_idx], kv.rec_state[layer_idx]
        defer = getattr(batch, "h_gdn_defer", None)
        for bidx, slot in enumerate(batch.h_slots):
            r0, r1 = batch.h_q_start[bidx], batch.h_q_start[bidx + 1]
            if r1 == r0:
                continue
            fresh = batch.h_ctx_len[bidx] - (r1 - r0) == 0
            keep = not (defer is not None and defer[bidx])
            if fresh:
                conv_state[slot].zero_()
                rec_state[slot].zero_()
            y, cs = ref.gdn_conv(mixed_qkv[r0:r1], conv_state[slot], gdn.conv_w)
            if keep:
                conv_state[slot].copy_(cs)
            q = y[:, :hk * dk].view(-1, hk, dk)
            k = y[:, hk * dk:2 * hk * dk].view(-1, hk, dk)
            v = y[:, 2 * hk * dk:].view(-1, hv, dv)
            g, beta = ref.gdn_gates(a[r0:r1], b[r0:r1], gdn.A_log, gdn.dt_bias)
            if model.gdn_chunked and (r1 - r0) > 1:
                o, S = ref.gdn_chunked(q, k, v, g, beta, rec_state[slot])
            else:
                o, S = ref.gdn_recurrent(q, k, v, g, beta, rec_state[slot])
            if keep:
                rec_state[slot].copy_(S)
            if state_only:
                continue
            zz = z[r0:r1].view(-1, hv, dv)
            on = ref.gated_rmsnorm(o, zz, gdn.norm_w, cfg.rms_norm_eps, zero_centered=False, gate=cfg.gdn_output_gate)
            out[r0:r1] = on.reshape(r1 - r0, hv * dv)
        return None if state_only else out

    # -------------------------------------------------------------- head
    def argmax(self, logits):
        return ref.argmax_lowest(logits.float())
