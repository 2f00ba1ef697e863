"""Plain PyTorch reference of every fused op (the oracle for the CUDA kernels; also the CPU path).

Semantics follow the reference's kernels: RMSNorm with the residual add rounded to the activation
dtype before the norm and optional zero-centred weights (``kernels/src/cuda/ops_basic.cu:42-67``);
per-head q/k RMSNorm + NeoX rotary on the first ``rotary_dim`` dims, optional ``[q | gate]`` row
layout (``ops_basic.cu:95-164``); softmax → top-k → renormalise routing with lowest-id tie-break
(``ops_basic.cu:196-245``); the Gated DeltaNet recurrence (``kernels/src/cuda/gdn_recurrent.cu:47-92``)
with its causal conv and gates (``ops_basic.cu:301-344``); lowest-index argmax (``ops_basic.cu:249``).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

PAGE = 16


# ----------------------------------------------------------------------------------- norms
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None,
            zero_centered: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (normed, new_residual); ``new_residual = x + residual`` rounded to x.dtype."""
    if residual is not None:
        x = (x.float() + residual.float()).to(x.dtype)
    xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    wf = w.float() + 1.0 if zero_centered else w.float()
    y = xf * torch.rsqrt(var + eps) * wf
    return y.to(x.dtype), x


def gated_rmsnorm(x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float, zero_centered: bool = False,
                  gate: str = "silu") -> torch.Tensor:
    """Per-head RMSNorm of the GDN output, then multiplied by silu(z) (or sigmoid(z))."""
    xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    wf = w.float() + 1.0 if zero_centered else w.float()
    y = xf * torch.rsqrt(var + eps) * wf
    g = F.silu(z.float()) if gate == "silu" else torch.sigmoid(z.float())
    return (y * g).to(x.dtype)


# ----------------------------------------------------------------------------------- rotary
def rope_cos_sin(positions: torch.Tensor, inv_freq: torch.Tensor, scale: float = 1.0,
                 mrope_section: Optional[Sequence[int]] = None):
    """positions ``[T]`` (or ``[3, T]`` with M-RoPE) → cos, sin ``[T, rotary_dim/2]`` fp32."""
    if positions.dim() == 2:
        ang3 = positions.float().unsqueeze(-1) * inv_freq.float()  # [3, T, half]
        if mrope_section:
            half = inv_freq.numel()
            sel = torch.zeros(half, dtype=torch.long, device=inv_freq.device)
            o = 0
            for i, n in enumerate(mrope_section):
                sel[o:o + n] = i
                o += n
            ang = ang3.gather(0, sel.view(1, 1, half).expand(1, ang3.shape[1], half)).squeeze(0)
        else:
            ang = ang3[0]
    else:
        ang = positions.float().unsqueeze(-1) * inv_freq.float()
    return torch.cos(ang) * scale, torch.sin(ang) * scale


def apply_rope_neox(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x ``[T, H, D]`` fp32; rotates pairs (i, i + half) over the first ``2*half`` dims."""
    half = cos.shape[-1]
    x1, x2, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)


def hadamard_rotate(x: torch.Tensor) -> torch.Tensor:
    """Randomised Hadamard rotation of the last dimension (a power of two): element i changes sign when bit 15 of
    ``i * 2654435761 mod 2**32`` is set, then a Walsh-Hadamard transform scaled by 1/sqrt(D).  Orthogonal, so the dot
    product of two rotated vectors is the dot product of the originals (reference: ``rht_kernel``,
    kernels/src/cuda/nvfp4_kv.cu :356, behind ``--kv-rotate``)."""
    D = x.shape[-1]
    assert D & (D - 1) == 0
    idx = torch.arange(D, dtype=torch.int64)
    sign = 1.0 - 2.0 * (((idx * 2654435761) % (1 << 32)) >> 15 & 1).to(torch.float32)
    y = x.float() * sign.to(x.device)
    h = 1
    while h < D:
        y = y.reshape(*x.shape[:-1], D // (2 * h), 2, h)
        y = torch.stack([y[..., 0, :] + y[..., 1, :], y[..., 0, :] - y[..., 1, :]], dim=-2)
        h *= 2
    return y.reshape(x.shape) * D ** -0.5


def attn_prep(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
              q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
              cos: torch.Tensor, sin: torch.Tensor, gated: bool = False, zero_centered: bool = False,
              rotate: bool = False):
    """Split qkv rows, per-head RMSNorm of q and k, rotary, optionally the Hadamard rotation of q and k.
    Returns (q, k, v, gate|None) as [T,H,D]."""
    T = qkv.shape[0]
    dt = qkv.dtype
    qw = num_heads * head_dim * (2 if gated else 1)
    q_raw, k_raw, v_raw = qkv[:, :qw], qkv[:, qw:qw + num_kv_heads * head_dim], qkv[:, qw + num_kv_heads * head_dim:]
    gate = None
    if gated:
        qg = q_raw.view(T, num_heads, 2, head_dim)
        q, gate = qg[:, :, 0], qg[:, :, 1]
    else:
        q = q_raw.view(T, num_heads, head_dim)
    k = k_raw.view(T, num_kv_heads, head_dim)
    v = v_raw.view(T, num_kv_heads, head_dim)

    def hn(x, w):
        if w is None:
            return x.float()
        xf = x.float()
        wf = w.float() + 1.0 if zero_centered else w.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * wf
        return y.to(dt).float()

    q = apply_rope_neox(hn(q, q_norm_w), cos, sin)
    k = apply_rope_neox(hn(k, k_norm_w), cos, sin)
    if rotate:
        q, k = hadamard_rotate(q), hadamard_rotate(k)
    return q.to(dt), k.to(dt), v.contiguous(), gate


# ----------------------------------------------------------------------------------- paged KV
def kv_write(k_pool: torch.Tensor, v_pool: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
             slot_mapping: torch.Tensor) -> None:
    """Pools ``[pages, kv_heads, 16, D]``; slot = page * 16 + offset for each of the T new tokens."""
    page, off = slot_mapping.long() // PAGE, slot_mapping.long() % PAGE
    k_pool[page, :, off] = k.to(k_pool.dtype)
    v_pool[page, :, off] = v.to(v_pool.dtype)


def paged_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                    slots: Sequence[int], q_start: Sequence[int], ctx_len: Sequence[int], scale: float,
                    tree_mask: Optional[torch.Tensor] = None, allowed: Optional[Sequence] = None) -> torch.Tensor:
    """Causal GQA attention of q ``[T, H, D]`` over the paged pools.

    Sequence ``b`` owns rows ``q_start[b]:q_start[b+1]``; its KV length *including* those rows is
    ``ctx_len[b]``; row i attends to positions ``<= ctx_len - q_len + i``.  With ``tree_mask`` (``[T]`` int32) row i
    sees, among its sequence's own new tokens, only those whose bit is set in its word (a draft tree's ancestors).
    ``allowed[b]`` (bool ``[q_len, ctx_len]`` or None) further restricts what sequence b's rows see (a sparse selection).
    """
    T, H, D = q.shape
    KH = k_pool.shape[1]
    group = H // KH
    out = torch.empty(T, H, D, dtype=torch.float32, device=q.device)
    for b, slot in enumerate(slots):
        r0, r1 = q_start[b], q_start[b + 1]
        ql, n = r1 - r0, ctx_len[b]
        if ql == 0:
            continue
        npg = (n + PAGE - 1) // PAGE
        pages = block_table[slot, :npg].long()
        K = k_pool[pages].float().permute(1, 0, 2, 3).reshape(KH, npg * PAGE, D)[:, :n]
        V = v_pool[pages].float().permute(1, 0, 2, 3).reshape(KH, npg * PAGE, D)[:, :n]
        qq = q[r0:r1].float().view(ql, KH, group, D).permute(1, 2, 0, 3)       # [KH, g, ql, D]
        s = torch.einsum("hgqd,hnd->hgqn", qq, K) * scale
        pos_q = torch.arange(n - ql, n, device=q.device).view(ql, 1)
        pos_k = torch.arange(n, device=q.device).view(1, n)
        mask = pos_k <= pos_q
        if tree_mask is not None:
            words = tree_mask[r0:r1].to(torch.int64).view(ql, 1) & 0xFFFFFFFF
            own = ((words >> torch.arange(min(ql, 32), device=q.device).view(1, -1)) & 1).bool()      # [ql, min(ql, 32)]
            mask = mask.clone()
            mask[:, n - ql:n - ql + own.shape[1]] &= own
        if allowed is not None and allowed[b] is not None:
            mask = mask & allowed[b]
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("hgqn,hnd->hgqd", p, V)                               # [KH, g, ql, D]
        out[r0:r1] = o.permute(2, 0, 1, 3).reshape(ql, H, D)
    return out.to(q.dtype)


# ----------------------------------------------------------------------------------- MLP / MoE
def silu_mul(gu: torch.Tensor) -> torch.Tensor:
    """``[T, 2I]`` laid out as ``[gate | up]`` → ``silu(gate) * up`` in the input dtype."""
    I = gu.shape[-1] // 2
    return (F.silu(gu[..., :I].float()) * gu[..., I:].float()).to(gu.dtype)


def router_topk(logits: torch.Tensor, k: int, renorm: bool = True):
    """Softmax over all experts (fp32), top-k by probability, lowest id wins ties."""
    p = torch.softmax(logits.float(), dim=-1)
    E = p.shape[-1]
    # stable lowest-id tie break: sort by (-p, id)
    order = torch.argsort(-p, dim=-1, stable=True)[..., :k]
    w = torch.gather(p, -1, order)
    if renorm:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, order.to(torch.int32)


def moe_forward(x: torch.Tensor, topk_w: torch.Tensor, topk_id: torch.Tensor, expert_fn, num_experts: int):
    """Reference mixture: ``out[t] = sum_j w[t,j] * expert_fn(e_j, x[t])`` evaluated per expert."""
    out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    first = getattr(getattr(expert_fn, "__self__", None), "first", 0)
    count = getattr(getattr(expert_fn, "__self__", None), "count", num_experts)
    for e in range(first, first + count):
        tok, slot = (topk_id == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        y = expert_fn(e, x[tok]).float()
        out.index_add_(0, tok, y * topk_w[tok, slot].float().unsqueeze(-1))
    return out.to(x.dtype)


# ----------------------------------------------------------------------------------- Gated DeltaNet
def gdn_conv(x: torch.Tensor, conv_state: torch.Tensor, w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Causal depthwise conv + SiLU over one sequence.

    ``x [T, C]``, ``conv_state [C, k-1]`` (the last k-1 inputs), ``w [C, k]``.  The conv result is
    rounded to the activation dtype before SiLU.  Returns (y [T, C], new_state).
    """
    T, C = x.shape
    k = w.shape[1]
    hist = torch.cat([conv_state.t().to(x.dtype), x], dim=0)          # [k-1+T, C]
    win = hist.float().unfold(0, k, 1)                                 # [T, C, k]
    y = (win * w.float().unsqueeze(0)).sum(-1).to(x.dtype)
    y = F.silu(y.float()).to(x.dtype)
    new_state = hist[-(k - 1):].t().contiguous().to(conv_state.dtype) if k > 1 else conv_state
    return y, new_state


def gdn_gates(a: torch.Tensor, b: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor):
    """g = -exp(A_log) * softplus(a + dt_bias) (fp32);  beta = sigmoid(b) rounded to b.dtype."""
    g = -torch.exp(A_log.float()) * F.softplus(a.float() + dt_bias.float())
    beta = torch.sigmoid(b.float()).to(b.dtype).float()
    return g, beta


def gdn_recurrent(q, k, v, g, beta, state):
    """Exact token-by-token gated delta rule for one sequence.

    q,k ``[T, Hk, dk]``; v ``[T, Hv, dv]``; g, beta ``[T, Hv]``; state ``[Hv, dk, dv]`` fp32.
    q and k are L2-normalised, q is scaled by dk^-1/2.  Hv is a multiple of Hk (key heads shared).
    """
    T, Hk, dk = q.shape
    Hv, dv = v.shape[1], v.shape[2]
    rep = Hv // Hk
    qf = F.normalize(q.float(), dim=-1, eps=1e-6) * (dk ** -0.5)
    kf = F.normalize(k.float(), dim=-1, eps=1e-6)
    qf = qf.repeat_interleave(rep, dim=1)
    kf = kf.repeat_interleave(rep, dim=1)
    S = state.float().clone()
    out = torch.empty(T, Hv, dv, dtype=torch.float32, device=q.device)
    for t in range(T):
        S = S * torch.exp(g[t]).view(Hv, 1, 1)
        kv = torch.einsum("hk,hkv->hv", kf[t], S)
        delta = (v[t].float() - kv) * beta[t].view(Hv, 1)
        S = S + torch.einsum("hk,hv->hkv", kf[t], delta)
        out[t] = torch.einsum("hk,hkv->hv", qf[t], S)
    return out.to(v.dtype), S


def gdn_chunked(q, k, v, g, beta, state, chunk: int = 64):
    """Chunked (WY / UT-transform) evaluation of the same recurrence; what the GPU kernel computes."""
    T, Hk, dk = q.shape
    Hv, dv = v.shape[1], v.shape[2]
    rep = Hv // Hk
    qf = (F.normalize(q.float(), dim=-1, eps=1e-6) * (dk ** -0.5)).repeat_interleave(rep, dim=1)
    kf = F.normalize(k.float(), dim=-1, eps=1e-6).repeat_interleave(rep, dim=1)
    vf = v.float()
    S = state.float().clone()                                         # [Hv, dk, dv]
    out = torch.empty(T, Hv, dv, dtype=torch.float32, device=q.device)
    for c0 in range(0, T, chunk):
        c1 = min(c0 + chunk, T)
        L = c1 - c0
        Q, K, V = qf[c0:c1].transpose(0, 1), kf[c0:c1].transpose(0, 1), vf[c0:c1].transpose(0, 1)  # [Hv, L, *]
        G = g[c0:c1].t().float().cumsum(dim=1)                         # [Hv, L] cumulative log decay
        B = beta[c0:c1].t().float()                                    # [Hv, L]
        decay = torch.exp(G.unsqueeze(2) - G.unsqueeze(1))             # [Hv, i, j] = exp(G_i - G_j)
        tril = torch.tril(torch.ones(L, L, device=q.device, dtype=torch.bool), -1)
        A = torch.einsum("hik,hjk->hij", K, K) * decay * B.unsqueeze(2)
        A = A.masked_fill(~tril, 0.0)                                  # strictly lower
        eye = torch.eye(L, device=q.device).unsqueeze(0)
        Tm = torch.linalg.solve_triangular(eye + A, eye.expand(Hv, L, L).contiguous(), upper=False)
        # u_i = beta_i (v_i - exp(G_i) k_i^T S0) - sum_{j<i} A_ij u_j
        rhs = B.unsqueeze(2) * (V - torch.exp(G).unsqueeze(2) * torch.einsum("hik,hkv->hiv", K, S))
        U = torch.einsum("hij,hjv->hiv", Tm, rhs)                      # deltas  [Hv, L, dv]
        incl = torch.tril(torch.ones(L, L, device=q.device, dtype=torch.bool), 0)
        QK = (torch.einsum("hik,hjk->hij", Q, K) * decay).masked_fill(~incl, 0.0)
        O = torch.exp(G).unsqueeze(2) * torch.einsum("hik,hkv->hiv", Q, S) + torch.einsum("hij,hjv->hiv", QK, U)
        out[c0:c1] = O.transpose(0, 1)
        GL = G[:, -1]
        S = S * torch.exp(GL).view(Hv, 1, 1) + torch.einsum(
            "hjk,hjv->hkv", K * torch.exp(GL.unsqueeze(1) - G).unsqueeze(2), U)
    return out.to(v.dtype), S


# ----------------------------------------------------------------------------------- head
def argmax_lowest(logits: torch.Tensor) -> torch.Tensor:
    """Row-wise argmax; the lowest index wins ties."""
    m = logits.max(dim=-1, keepdim=True).values
    idx = torch.arange(logits.shape[-1], device=logits.device).expand_as(logits)
    big = torch.full_like(idx, logits.shape[-1])
    return torch.where(logits == m, idx, big).min(dim=-1).values
