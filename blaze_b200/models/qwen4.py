"""The Qwen4-Exp extras on top of the hybrid decoder: hyper-connections (several residual streams with gated low-rank
mixing in place of the pre-norm residual) and the per-layer n-gram embedding (PLE).

What is computed follows the reference's PyTorch statement of the model (``scripts/ref_qwen4.py``: ``grouped_norm`` :145,
``hc_mix`` :152, ``hc_combine`` :161, ``ple`` :265, the layer loop :318-340) and its kernel tests
(``kernels/tests/test_qwen4.cu``, ``test_hc_mix.cu``); the reference runs them as ``hc_mix.cu`` / ``qwen4.cu`` kernels fed by
a host-side row service (``runtime/ple_service.cpp``).  Here the n-gram tables are resident in HBM (a B200 holds them), so
a lookup is a device gather and there is no host service, mailbox or row cache.  The functions are written on torch
tensors and run on whichever device the model lives on; sums are fp32 and results are rounded to the model's dtype at the
points where the reference rounds to bf16.

Per-sequence state (kept with the recurrent state rows of :class:`blaze_b200.kv.KVCache`): the two tokens before the
next one (the n-gram window) and the last ``3 * ngram_size`` rows that entered each PLE layer's dilated convolution.

The sparse-attention indexer of the same family (QSA; reference: ``kernels/src/cuda/qsa_index.cu``, driven by
``crates/blaze/src/model.rs:2809`` ``qsa_index``, stated by ``kernels/tests/test_qsa_index.cu``): every softmax layer projects
index queries (a few heads) and one index key per token; the keys of each complete block of ``compress_ratio`` tokens are
averaged, normed and rotated to the block's first position; a row scores a block by the sum over heads of
``relu(q . k)`` over ``sqrt(dim)`` and attends to the tokens of its ``budget / compress_ratio`` best blocks (ties: the
earlier block) plus those of the incomplete block it stands in.  While a context has no more blocks than that, every key
is selected and attention is dense.  Here the raw index keys are paged like K and V (``KVCache.idx_k``), compressed keys
are formed when a row scores them, and the selection is a mask for the torch attention; the attention kernels read whole
sequences, so steps with a context beyond the budget take the masked torch attention on either op set."""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F


class HcBlock:
    """Weights of one hyper-connection: ``norm`` [HC*H] (stored as w - 1), ``down`` [R, HC*H], ``up`` [HC*H, R] and, for a
    block that writes back into the streams, ``inject`` [HC, HC*H]."""

    def __init__(self):
        self.norm = self.down = self.up = None
        self.inject: Optional[torch.Tensor] = None


class Ple:
    """One layer's n-gram embedding: hash constants, the table, projections, norms and the dilated conv."""

    def __init__(self):
        self.mult = self.sizes = self.offs = None      # int64 [3], [2 * heads_per_ngram] x 2
        self.table: Optional[torch.Tensor] = None      # [sum(sizes), embed_dim]
        self.key = self.value = None                   # Linear: 2 * hpn * embed_dim -> HC*H / H
        self.norm_key = self.norm_query = self.norm_conv = None     # [HC*H], stored as w - 1
        self.conv_w: Optional[torch.Tensor] = None     # [HC*H, kernel]


def grouped_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """RMSNorm of each of the ``groups`` equal slices of every row, times ``1 + w``; fp32 in, fp32 out."""
    t = x.shape[0]
    g = x.float().view(t, groups, -1)
    g = g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + eps)
    return g.reshape(t, -1) * (1.0 + w.float())


def hc_mix(streams: torch.Tensor, blk: HcBlock, hc: int, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """The streams' input to a block: per-stream norm ``n``, gates ``sigmoid(silu(n @ down^T / hc) @ up^T)`` per stream and
    feature, and the mean over streams of ``gate * n``.  Returns ``(x [T, H], n [T, HC*H])`` in the streams' dtype."""
    dt = streams.dtype
    n = grouped_norm(streams, blk.norm, hc, eps).to(dt)
    nf = n.float()
    t = F.silu((nf @ blk.down.float().t()) / hc).to(dt).float()
    u = t @ blk.up.float().t()
    x = (torch.sigmoid(u) * nf).view(n.shape[0], hc, -1).mean(1)
    return x.to(dt), n


def hc_combine(streams: torch.Tensor, n: torch.Tensor, blk: HcBlock, y: torch.Tensor, hc: int) -> torch.Tensor:
    """A block's output ``y`` [T, H] back into the streams: stream c gets ``2 * sigmoid(n . inject[c] / hc) * y``."""
    a = 2.0 * torch.sigmoid((n.float() @ blk.inject.float().t()) / hc)                    # [T, HC]
    out = streams.float().view(streams.shape[0], hc, -1) + a[..., None] * y.float()[:, None, :]
    return out.to(streams.dtype).reshape(streams.shape[0], -1)


def ngram_ids(w2: torch.Tensor, w1: torch.Tensor, w0: torch.Tensor, eos: int, P: Ple, heads_per_ngram: int) -> torch.Tensor:
    """Table rows ``[T, 2 * heads_per_ngram]`` of tokens ``w2`` with the tokens one (``w1``) and two (``w0``) places before
    them.  A window does not reach across an end-of-sequence token; missing places count as that token.  The first
    ``heads_per_ngram`` heads hash the bigram, the others the trigram; products wrap at 64 bits."""
    w2, w1, w0 = w2.long(), w1.long(), w0.long()
    e = torch.full_like(w2, eos)
    t1 = torch.where(w1 == eos, e, w1)
    t2 = torch.where((w1 == eos) | (w0 == eos), e, w0)
    m2 = (w2 * P.mult[0]) ^ (t1 * P.mult[1])
    m3 = m2 ^ (t2 * P.mult[2])
    mix = torch.cat([m2[:, None].expand(-1, heads_per_ngram), m3[:, None].expand(-1, heads_per_ngram)], 1)
    return torch.remainder(mix, P.sizes[None, :]) + P.offs[None, :]


def ple_gate(key: torch.Tensor, streams: torch.Tensor, value: torch.Tensor, P: Ple, hc: int, eps: float) -> torch.Tensor:
    """``gated [T, HC*H]``: stream c's gate is ``sigmoid(sign(d) * sqrt(max(|d|, 1e-6)))`` with ``d`` the dot product of the
    normed key slice and the normed stream over ``sqrt(H)``; it scales the value row."""
    t = key.shape[0]
    kn = grouped_norm(key, P.norm_key, hc, eps).to(key.dtype).float().view(t, hc, -1)
    qn = grouped_norm(streams, P.norm_query, hc, eps).to(key.dtype).float().view(t, hc, -1)
    d = (kn * qn).sum(-1) / math.sqrt(kn.shape[-1])
    g = torch.sigmoid(d.abs().clamp_min(1e-6).sqrt() * d.sign())
    return (g[..., None] * value.float()[:, None, :]).to(key.dtype).reshape(t, -1)


def ple_conv(gn: torch.Tensor, history: torch.Tensor, conv_w: torch.Tensor, dilation: int) -> torch.Tensor:
    """Causal convolution of one sequence's rows ``gn [t, C]`` with taps ``dilation`` rows apart; ``history`` holds the
    ``(kernel - 1) * dilation`` rows before them (oldest first).  The last tap multiplies the row itself."""
    k = conv_w.shape[1]
    pad = torch.cat([history.float(), gn.float()])
    t = gn.shape[0]
    w = conv_w.float()
    return sum(w[:, j] * pad[j * dilation:j * dilation + t] for j in range(k))


def random_hc(rnd, H: int, hc: int, R: int, tag: int, dtype, inject: bool = True) -> HcBlock:
    b = HcBlock()
    b.norm = torch.zeros(hc * H, dtype=dtype, device=rnd(1, 1, tag).device)
    b.down = rnd(R, hc * H, tag + 1).to(dtype)
    b.up = rnd(hc * H, R, tag + 2, 0.05).to(dtype)
    if inject:
        b.inject = rnd(hc, hc * H, tag + 3, 0.01).to(dtype)
    return b


def load_hc(ck, prefix: str, dtype, device, inject: bool = True) -> HcBlock:
    """Tensor names of a hyper-connection (``ref_qwen4.py`` :152-163)."""
    b = HcBlock()
    b.norm = ck.get(prefix + "hc_norm.weight").to(dtype).to(device)
    b.down = ck.get(prefix + "input_mix_weight_down.weight").to(dtype).to(device)
    b.up = ck.get(prefix + "input_mix_weight_up.weight").to(dtype).to(device)
    if inject:
        b.inject = ck.get(prefix + "block_inject_weight.weight").to(dtype).to(device)
    return b


def load_ple(ck, prefix: str, cfg, dtype, device, load_lin) -> Ple:
    """Tensor names of a layer's PLE (``ref_qwen4.py`` :265-310); the table's shards are joined into one tensor."""
    P = Ple()
    e = prefix + "ple_embedding."
    P.mult = ck.get(e + "layer_multipliers").long().to(device)
    P.sizes = ck.get(e + "ngram_heads_vocab_sizes").long().to(device)
    P.offs = ck.get(e + "ngram_heads_offsets").long().to(device)
    shards: List[torch.Tensor] = []
    while (e + f"ngram_embedding.shard_{len(shards)}.weight") in ck:
        shards.append(ck.get(e + f"ngram_embedding.shard_{len(shards)}.weight").to(dtype))
    if not shards:
        raise ValueError(f"{e}ngram_embedding has no shards")
    P.table = torch.cat(shards).to(device)
    P.key = load_lin([prefix + "key_proj"])
    P.value = load_lin([prefix + "value_proj"])
    P.norm_key = ck.get(prefix + "norm_key.weight").to(dtype).to(device)
    P.norm_query = ck.get(prefix + "norm_query.weight").to(dtype).to(device)
    P.norm_conv = ck.get(prefix + "norm_conv.weight").to(dtype).to(device)
    cw = ck.get(prefix + "conv1d.weight").float()
    P.conv_w = cw.view(cw.shape[0], -1).to(dtype).to(device)
    return P


def random_ple(rnd, cfg, tag: int, dtype, device, make_lin) -> Ple:
    """A small random PLE: prime-sized head tables (as the checkpoints have) of a few hundred rows."""
    P = Ple()
    hpn, d, H, hc = cfg.heads_per_ngram, cfg.ple_embed_dim, cfg.hidden_size, cfg.hc_count
    primes = [251, 257, 263, 269, 271, 277, 281, 283, 293, 307, 311, 313, 317, 331, 337, 347]
    sizes = [primes[(tag + h) % len(primes)] for h in range(2 * hpn)]
    P.mult = torch.tensor([123456789123 + tag, 98765432101 + 2 * tag, 55555555555 + 3 * tag], dtype=torch.int64, device=device)
    P.sizes = torch.tensor(sizes, dtype=torch.int64, device=device)
    P.offs = torch.tensor([sum(sizes[:h]) for h in range(2 * hpn)], dtype=torch.int64, device=device)
    P.table = rnd(sum(sizes), d, tag + 1, 1.0).to(dtype)
    P.key = make_lin(rnd(hc * H, 2 * hpn * d, tag + 2, 0.05))
    P.value = make_lin(rnd(H, 2 * hpn * d, tag + 3, 0.05))
    P.norm_key = torch.zeros(hc * H, dtype=dtype, device=device)
    P.norm_query = torch.zeros(hc * H, dtype=dtype, device=device)
    P.norm_conv = torch.zeros(hc * H, dtype=dtype, device=device)
    P.conv_w = rnd(hc * H, cfg.ple_conv_kernel, tag + 4, 0.3).to(dtype)
    return P


class PleState:
    """Per-row state of the PLE layers: ``hist [rows, 2]`` int64 (the two tokens before the next one, end-of-sequence at a
    sequence's start) and per PLE layer ``conv[layer] [rows, (kernel - 1) * dilation, HC*H]``."""

    def __init__(self, cfg, layers: List[int], rows: int, dtype, device):
        self.eos = int(cfg.eos_token_ids[0]) if cfg.eos_token_ids else 0
        self.layers = list(layers)
        self.hist = torch.full((rows, 2), self.eos, dtype=torch.int64, device=device)
        depth = (cfg.ple_conv_kernel - 1) * cfg.ngram_size
        self.conv = {i: torch.zeros(rows, depth, cfg.hc_count * cfg.hidden_size, dtype=dtype, device=device) for i in layers}

    def copy(self, src: int, dst: int) -> None:
        self.hist[dst].copy_(self.hist[src])
        for c in self.conv.values():
            c[dst].copy_(c[src])

    def zero(self, row: int) -> None:
        self.hist[row].fill_(self.eos)
        for c in self.conv.values():
            c[row].zero_()

    def nbytes(self) -> int:
        return self.hist.numel() * 8 + sum(c.numel() * c.element_size() for c in self.conv.values())


def window_tokens(batch, state: PleState) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(w1, w0)``: for every row of the step the token one and two places before it in its sequence (from this step's
    rows where they reach, else from the sequence's history)."""
    tok = batch.tokens.long()
    T = tok.shape[0]
    seq = batch.seq_of_row.long()
    pos = torch.arange(T, device=tok.device) - batch.q_start.long()[seq]
    h = state.hist[batch.slots.long()[seq]]                              # [T, 2]: (two before, one before) the step's first row
    w1 = torch.where(pos >= 1, tok.roll(1), h[:, 1])
    w0 = torch.where(pos >= 2, tok.roll(2), torch.where(pos == 1, h[:, 1], h[:, 0]))
    return w1, w0


def advance_history(batch, tok: torch.Tensor, state: PleState, skip=None) -> None:
    """Move every sequence's two-token history past its rows of ``tok`` (laid out as ``batch`` describes); sequences flagged in
    ``skip`` keep theirs."""
    tok = tok.long()
    for b, slot in enumerate(batch.h_slots):
        r0, r1 = batch.h_q_start[b], batch.h_q_start[b + 1]
        if r1 <= r0 or (skip is not None and skip[b]):
            continue
        if r1 - r0 >= 2:
            state.hist[slot] = tok[r1 - 2:r1]
        else:
            state.hist[slot] = torch.stack([state.hist[slot, 1], tok[r0]])


def ple_apply(model, P: Ple, layer: int, streams: torch.Tensor, batch, state: PleState, w1, w0) -> torch.Tensor:
    """Add a layer's n-gram embedding to the streams (``ref_qwen4.py`` :265).  Sequences that defer their state
    (``batch.h_gdn_defer``) read the convolution history without moving it; the rows they fed are kept in
    ``model.ple_records`` for :func:`ple_replay`."""
    cfg, ops = model.cfg, model.ops
    hc, eps, dil = cfg.hc_count, cfg.rms_norm_eps, cfg.ngram_size
    ids = ngram_ids(batch.tokens, w1, w0, state.eos, P, cfg.heads_per_ngram)
    emb = P.table[ids.reshape(-1)].reshape(ids.shape[0], -1)
    key = ops.linear(P.key, emb)
    value = ops.linear(P.value, emb)
    gated = ple_gate(key, streams, value, P, hc, eps)
    gn = grouped_norm(gated, P.norm_conv, hc, eps).to(streams.dtype)
    conv = torch.empty(gn.shape, dtype=torch.float32, device=gn.device)
    hist = state.conv[layer]
    defer = batch.h_gdn_defer
    depth = hist.shape[1]
    if batch.max_q_len == 1 and defer is None:
        # plain decode: one row per sequence, all sequences at once
        slots = batch.slots.long()
        pad = torch.cat([hist[slots], gn[:, None, :]], 1).float()                       # [B, depth + 1, C]
        w = P.conv_w.float()
        conv = sum(w[:, j] * pad[:, j * dil] for j in range(w.shape[1]))
        hist[slots] = pad[:, 1:].to(hist.dtype)
    else:
        for b, slot in enumerate(batch.h_slots):
            r0, r1 = batch.h_q_start[b], batch.h_q_start[b + 1]
            if r1 == r0:
                continue
            if batch.h_ctx_len[b] - (r1 - r0) == 0:
                hist[slot].zero_()
            conv[r0:r1] = ple_conv(gn[r0:r1], hist[slot], P.conv_w, dil)
            if not (defer is not None and defer[b]):
                hist[slot] = torch.cat([hist[slot], gn[r0:r1]])[-depth:]
        if defer is not None:
            model.ple_records[layer] = gn
            model.ple_records["tokens"] = batch.tokens
    dt = streams.dtype
    out = (gated.float() + F.silu(conv.to(dt).float()).to(dt).float()).to(dt)
    return (streams.float() + out.float()).to(dt)


def ple_replay(model, batch, rows: torch.Tensor, state: PleState) -> None:
    """Advance the PLE state over ``rows`` of the recorded (deferred) step — the accepted rows, grouped by sequence as
    ``batch`` describes."""
    idx = rows.long()
    for layer, hist in state.conv.items():
        gn = model.ple_records.get(layer)
        if gn is None:
            raise RuntimeError("no deferred step to replay")
        g = gn[idx]
        depth = hist.shape[1]
        for b, slot in enumerate(batch.h_slots):
            r0, r1 = batch.h_q_start[b], batch.h_q_start[b + 1]
            if r1 > r0:
                hist[slot] = torch.cat([hist[slot], g[r0:r1]])[-depth:]
    advance_history(batch, model.ple_records["tokens"][idx], state)


# ----------------------------------------------------------------------------------- sparse-attention indexer (QSA)
class Indexer:
    """Weights of a softmax layer's indexer: ``proj`` (hidden -> heads * dim index queries, then one index key of dim),
    ``q_norm`` / ``k_norm`` [dim] (stored as w - 1)."""

    def __init__(self):
        self.proj = None
        self.q_norm = self.k_norm = None


def _norm_rope(x: torch.Tensor, w: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, rot: int, eps: float, scale: float, dt):
    """RMSNorm times ``1 + w`` over the last axis (rounded to ``dt``), then the rotation of the first ``rot`` dims (pairs
    ``i, i + rot / 2``) by ``pos`` (broadcast over the axes between), rounded again; fp32 out."""
    xf = x.float()
    xf = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w.float())).to(dt).float()
    half = rot // 2
    ang = pos.float()[..., None] * inv_freq.float()[:half]
    c, s = torch.cos(ang) * scale, torch.sin(ang) * scale
    while c.dim() < xf.dim():
        c, s = c.unsqueeze(-2), s.unsqueeze(-2)
    a, b = xf[..., :half], xf[..., half:rot]
    return torch.cat([a * c - b * s, b * c + a * s, xf[..., rot:]], -1).to(dt).float()


def compressed_keys(kraw: torch.Tensor, I: Indexer, ratio: int, inv_freq, rot: int, eps: float, scale: float) -> torch.Tensor:
    """Keys of the complete blocks of one sequence: ``kraw [n, dim]`` raw index keys in position order -> ``[n // ratio, dim]``."""
    nb = kraw.shape[0] // ratio
    dt = kraw.dtype
    mean = (kraw[:nb * ratio].float().view(nb, ratio, -1).sum(1) / ratio).to(dt)
    pos = torch.arange(nb, device=kraw.device) * ratio
    return _norm_rope(mean, I.k_norm, pos, inv_freq, rot, eps, scale, dt)


def block_scores(iq: torch.Tensor, comp: torch.Tensor) -> torch.Tensor:
    """``iq [rows, heads, dim]`` (normed, rotated) against ``comp [blocks, dim]``: ``sum_h relu(q_h . k) / sqrt(dim)``."""
    return torch.relu(torch.einsum("rhd,bd->rhb", iq.float(), comp.float())).sum(1) / math.sqrt(iq.shape[-1])


def select_keys(scores: torch.Tensor, pos: torch.Tensor, ratio: int, top_blocks: int, n: int) -> torch.Tensor:
    """bool ``[rows, n]``: for the row at position ``pos[r]`` the tokens of its best ``top_blocks`` blocks among the
    ``(pos + 1) // ratio`` complete ones it can see (equal scores: the earlier block), and the tokens after them up to
    ``pos`` (the incomplete block)."""
    rows, nb = scores.shape
    nvis = (pos.long() + 1) // ratio
    blk = torch.arange(nb, device=scores.device)
    sc = scores.float().masked_fill(blk[None, :] >= nvis[:, None], float("-inf"))
    order = torch.sort(sc, dim=1, descending=True, stable=True).indices             # stable: ties keep block order
    rank = torch.empty_like(order)
    rank.scatter_(1, order, blk[None, :].expand(rows, nb).contiguous())
    chosen = (rank < top_blocks) & (blk[None, :] < nvis[:, None])                  # [rows, nb]
    tok = torch.arange(n, device=scores.device)
    out = torch.zeros(rows, n, dtype=torch.bool, device=scores.device)
    full = min(nb * ratio, n)
    out[:, :full] = chosen.repeat_interleave(ratio, dim=1)[:, :full]
    tail = (tok[None, :] >= (nvis * ratio)[:, None]) & (tok[None, :] <= pos.long()[:, None])
    return out | tail


def qsa_step(model, I: Indexer, h: torch.Tensor, batch, kv, layer: int):
    """The indexer's part of a softmax layer's step: index keys of the new tokens go to their slots; sequences whose
    context exceeds the budget get the selection of every row.  Returns the per-sequence masks for the attention (None
    when every sequence is within the budget)."""
    cfg, ops = model.cfg, model.ops
    Hi, Di, ratio = cfg.indexer_heads, cfg.indexer_head_dim, cfg.indexer_compress_ratio
    proj = ops.linear(I.proj, h)
    pool = kv.idx_k[layer]
    valid = batch.slot_mapping >= 0
    pool.view(-1, Di)[batch.slot_mapping[valid].long()] = proj[valid, Hi * Di:].to(pool.dtype)
    top_blocks = cfg.indexer_budget // ratio
    if max(batch.h_ctx_len, default=0) // ratio <= top_blocks:
        return None
    rot, eps, dt = cfg.rotary_dim, cfg.rms_norm_eps, pool.dtype
    pos_all = batch.positions if batch.positions.dim() == 1 else batch.positions[0]
    iq = _norm_rope(proj[:, :Hi * Di].reshape(-1, Hi, Di), I.q_norm, pos_all, model.inv_freq, rot, eps, model.rope_scale, dt)
    table = kv.block_table
    out = []
    for b, slot in enumerate(batch.h_slots):
        r0, r1 = batch.h_q_start[b], batch.h_q_start[b + 1]
        n = batch.h_ctx_len[b]
        if r1 == r0 or n // ratio <= top_blocks:
            out.append(None)
            continue
        npg = (n + pool.shape[1] - 1) // pool.shape[1]
        kraw = pool[table[slot, :npg].long()].reshape(-1, Di)[:n]
        comp = compressed_keys(kraw, I, ratio, model.inv_freq, rot, eps, model.rope_scale)
        pos = torch.arange(n - (r1 - r0), n, device=h.device)
        out.append(select_keys(block_scores(iq[r0:r1], comp), pos, ratio, top_blocks, n))
    return out
