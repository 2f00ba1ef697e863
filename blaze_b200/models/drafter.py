"""Model-based drafters for speculative decoding: MTP head, EAGLE-style chain drafter, DFlash-style block drafter.

All three share one shape: a single decoder layer with its own KV cache that consumes the target's hidden state of
position p together with the embedding of token p+1 and predicts token p+2; they differ in how the input is fused
and in what they read from the target.  Reference: ``crates/blaze/src/drafter.rs`` (dispatch by architecture :26,
``capture_layers`` :59), ``mtp.rs`` (``layer_dense`` :751: ``x = fc(cat(norm_e(embed(tok)), norm_h(hidden)))`` → layer →
``mtp.norm`` → shared lm_head :990-1053), ``eagle.rs`` (``fc`` over the concatenated hidden states of several target
layers :265, chains :845), ``dflash.rs`` (block-parallel proposal :416).

The scheduler calls ``observe`` after every target step (to feed confirmed (hidden, next token) pairs) and ``propose``
before a decode step.  Acceptance is decided by the target, so a drafter can only change speed, never the tokens.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..batch import SeqChunk
from ..config import ModelConfig
from ..engine import Engine, EngineConfig, Seq
from ..linear import Cut, Linear
from ..quant import Format
from .qwen3 import Model, TPInfo


@dataclass
class DraftState:
    seq: Seq
    fed: int = 0                       # positions whose (hidden, next token) pair the drafter has consumed
    pend_hidden: Optional[torch.Tensor] = None   # confirmed hidden rows not yet fed  [n, H * n_capture]
    pend_tokens: Optional[List[int]] = None      # their "next" tokens


class ChainDrafter:
    """MTP / EAGLE: fuse (token embedding, target hidden) → one layer → head → greedy chain of k tokens."""

    kind = "mtp"

    def __init__(self, target: Model, layer_model: Model, fc: Linear, norm_e: torch.Tensor, norm_h: torch.Tensor,
                 max_seqs: int, max_model_len: int, kv_dtype: str, capture_layers: Sequence[int] = ()):
        self.target, self.m, self.fc, self.norm_e, self.norm_h = target, layer_model, fc, norm_e, norm_h
        self.ops = target.ops
        self.capture_layers = list(capture_layers)
        self.engine = Engine(layer_model, EngineConfig(max_seqs=max_seqs, max_model_len=max_model_len, kv_dtype=kv_dtype,
                                                       kv_tokens=max_seqs * max_model_len, use_graphs=False))
        self.states: Dict[str, DraftState] = {}
        self.proposed = self.steps = 0
        self.draft_ids: Optional[torch.Tensor] = None    # reduced draft vocabulary (token ids), or None = full head
        self.draft_head: Optional[Linear] = None

    def use_draft_vocab(self, ids: Sequence[int]) -> None:
        """Draft over a reduced vocabulary: the head GEMM of every draft step then covers only ``ids`` (for instance the
        32k most frequent tokens), which is most of a drafter's cost for a 150k-entry vocabulary; proposals outside the
        subset are impossible, which only lowers acceptance — the target still decides every token
        (``eagle.rs:694`` ``head_merged``, ``kernels/src/cuda/eagle.cu:76`` ``candidate_logits``)."""
        ids_t = torch.as_tensor(sorted(set(int(i) for i in ids)), dtype=torch.long, device=self.target.device)
        head = self.m.lm_head
        w = head.dequant() if head.fmt != Format.DENSE else head.w
        self.draft_head = Linear.from_dense(w.to(self.target.device)[ids_t].float(), Format.DENSE, dtype=self.target.dtype)
        self.draft_ids = ids_t

    def _greedy(self, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        if self.draft_head is None:
            return self.m.greedy(x, rows)
        h = self.m.final_hidden(x, rows)
        if self.ops.is_cuda:
            local = self.ops.linear_argmax(self.draft_head, h)
        else:
            local = self.ops.argmax(self.ops.linear(self.draft_head, h, out_dtype=torch.float32))
        return self.draft_ids[local.long()]

    # ------------------------------------------------------------------ construction
    @classmethod
    def random_init(cls, target: Model, seed: int = 7, max_seqs: int = 256, max_model_len: int = 4096, kv_dtype: str = "bf16",
                    fmt: Format = Format.DENSE, n_capture: int = 1):
        """A random-init one-layer drafter shaped like the target (``mtp_num_hidden_layers = 1``)."""
        cfg = ModelConfig(**{**vars(target.cfg), "num_layers": 1, "layer_types": ["full_attention"], "num_experts": 0})
        cfg.rope = target.cfg.rope
        lm = Model.random_init(cfg, fmt, seed, target.device, target.dtype, TPInfo(), ops=target.ops)
        lm.embed, lm.lm_head = target.embed, target.lm_head          # shared with the target
        H = cfg.hidden_size
        g = torch.Generator(device=target.device).manual_seed(seed + 1)
        fc = Linear.from_dense(torch.randn(H, H * (1 + n_capture), generator=g, device=target.device) * 0.02, Format.DENSE,
                               dtype=target.dtype)
        one = torch.ones(H, dtype=target.dtype, device=target.device)
        d = cls(target, lm, fc, one, one.clone(), max_seqs, max_model_len, kv_dtype)
        d.n_capture = n_capture
        return d

    @classmethod
    def load_mtp(cls, target: Model, ckpt, max_seqs: int, max_model_len: int, kv_dtype: str = "bf16"):
        """Load ``mtp.*`` tensors of the target's checkpoint (names of ``mtp.rs:199-404``)."""
        from ..weights import Checkpoint
        ck = ckpt if not isinstance(ckpt, str) else Checkpoint.open(ckpt)
        cfg = ModelConfig(**{**vars(target.cfg), "num_layers": 1, "layer_types": ["full_attention"]})
        cfg.rope = target.cfg.rope
        dev, dt = target.device, target.dtype
        lm = Model(cfg, dev, dt, TPInfo(), ops=target.ops)
        from .qwen3 import Attn, DenseMlp, Layer, _load_stacked_heads
        L = Layer()
        p = "mtp.layers.0."
        L.input_norm = ck.get(p + "input_layernorm.weight").to(dt).to(dev)
        L.post_norm = ck.get(p + "post_attention_layernorm.weight").to(dt).to(dev)
        A = Attn()
        A.heads, A.kv_heads = cfg.num_heads, cfg.num_kv_heads
        D = cfg.head_dim
        A.qkv = _load_stacked_heads(ck, [p + "self_attn.q_proj", p + "self_attn.k_proj", p + "self_attn.v_proj"],
                                    [D * (2 if cfg.attn_output_gate else 1), D, D], [cfg.num_heads, cfg.num_kv_heads, cfg.num_kv_heads],
                                    0, 1, dt, dev)
        A.o = Linear.load(ck, [p + "self_attn.o_proj"], Cut.ALL, 0, 1, dt, dev)
        if (p + "self_attn.q_norm.weight") in ck:
            A.q_norm = ck.get(p + "self_attn.q_norm.weight").to(dt).to(dev)
            A.k_norm = ck.get(p + "self_attn.k_norm.weight").to(dt).to(dev)
        L.attn = A
        mlp = DenseMlp()
        mlp.gate_up = Linear.load(ck, [p + "mlp.gate_proj", p + "mlp.up_proj"], Cut.ALL, 0, 1, dt, dev)
        mlp.down = Linear.load(ck, [p + "mlp.down_proj"], Cut.ALL, 0, 1, dt, dev)
        L.mlp = mlp
        lm.layers = [L]
        lm.final_norm = ck.get("mtp.norm.weight").to(dt).to(dev)
        lm.embed, lm.lm_head = target.embed, target.lm_head
        fc = Linear.load(ck, ["mtp.fc"], Cut.ALL, 0, 1, dt, dev)
        ne = ck.get("mtp.pre_fc_norm_embedding.weight").to(dt).to(dev)
        nh = ck.get("mtp.pre_fc_norm_hidden.weight").to(dt).to(dev)
        d = cls(target, lm, fc, ne, nh, max_seqs, max_model_len, kv_dtype)
        d.n_capture = 1
        return d

    # ------------------------------------------------------------------ scheduler hooks
    def open(self, request_id: str) -> None:
        self.states[request_id] = DraftState(self.engine.open_from())

    def close(self, request_id: str) -> None:
        st = self.states.pop(request_id, None)
        if st is not None:
            self.engine.close(st.seq)

    def observe(self, request_id: str, hidden_rows: torch.Tensor, next_tokens: Sequence[int], start_pos: int) -> None:
        """``hidden_rows[i]`` is the target's hidden state at position ``start_pos + i`` and ``next_tokens[i]`` the token at
        ``start_pos + i + 1`` (confirmed).  Rows at positions the drafter already consumed are ignored."""
        st = self.states.get(request_id)
        if st is None:
            return
        n = len(next_tokens)
        skip = max(0, st.fed + (0 if st.pend_tokens is None else len(st.pend_tokens)) - start_pos)
        if skip >= n:
            return
        h = hidden_rows[skip:n]
        t = list(next_tokens[skip:])
        if st.pend_tokens:
            st.pend_hidden = torch.cat([st.pend_hidden, h])
            st.pend_tokens += t
        else:
            st.pend_hidden, st.pend_tokens = h, t

    def _fuse(self, tokens: torch.Tensor, hidden: torch.Tensor) -> torch.Tensor:
        ops, eps, zc = self.ops, self.m.cfg.rms_norm_eps, self.m.cfg.zero_centered_norm
        e = ops.embed(self.m.embed, tokens)
        ne, _ = ops.norm(e, None, self.norm_e, eps, zc)
        nh, _ = ops.norm(hidden.contiguous(), None, self.norm_h, eps, zc)
        return ops.linear(self.fc, torch.cat([ne, nh], dim=1).contiguous())

    def propose(self, actives, ks: Sequence[int]) -> List[List[int]]:
        """Feed the pending confirmed pairs, then draft ``ks[i]`` tokens for ``actives[i]`` greedily."""
        eng = self.engine
        todo = [(a, k, self.states.get(a.req.request_id)) for a, k in zip(actives, ks)]
        todo = [(a, k, st) for a, k, st in todo if st is not None and st.pend_tokens]
        out: Dict[int, List[int]] = {id(a): [] for a in actives}
        if not todo:
            return [out[id(a)] for a in actives]
        # drop drafter KV beyond what was confirmed (rows written by earlier speculative chains)
        for a, k, st in todo:
            eng.truncate(st.seq, st.fed)
        dev = self.target.device
        items, toks, hids = [], [], []
        for a, k, st in todo:
            items.append((st.seq, st.pend_tokens, 1))
            toks += st.pend_tokens
            hids.append(st.pend_hidden)
        chunks = eng.plan(items)
        x_in = self._fuse(torch.tensor(toks, dtype=torch.int32, device=dev), torch.cat(hids))
        batch = eng._build(chunks)
        x = self.m.forward(batch, eng.kv, x_in)
        last = x[batch.logit_rows.long()]
        cur_tok = self._greedy(x, batch.logit_rows)
        for a, k, st in todo:
            st.fed += len(st.pend_tokens)
            st.pend_hidden, st.pend_tokens = None, None
        live = [(a, k, st) for a, k, st in todo]
        depth = 0
        toks_host = cur_tok.tolist()
        while live:
            for (a, k, st), t in zip(live, toks_host):
                out[id(a)].append(int(t))
            depth += 1
            keep = [i for i, (a, k, st) in enumerate(live) if k > depth]
            if not keep:
                break
            live = [live[i] for i in keep]
            idx = torch.tensor(keep, device=dev)
            last, cur_tok = last[idx], cur_tok[idx]
            chunks = eng.plan([(st.seq, [int(t)], 1) for (a, k, st), t in zip(live, cur_tok.tolist())])
            x_in = self._fuse(cur_tok.to(torch.int32), last)
            batch = eng._build(chunks)
            x = self.m.forward(batch, eng.kv, x_in)
            last = x[batch.logit_rows.long()]
            cur_tok = self._greedy(x, batch.logit_rows)
            toks_host = cur_tok.tolist()
        self.steps += 1
        self.proposed += sum(len(v) for v in out.values())
        return [out[id(a)] for a in actives]


class EagleDrafter(ChainDrafter):
    """EAGLE-style: the fused input reads the hidden states of several target layers (``capture_layers``)."""
    kind = "eagle"


class DFlashDrafter(ChainDrafter):
    """DFlash-style block drafter: proposes the whole block from one pass by feeding the last hidden state at every
    block position (no per-token chain), trading acceptance for one launch per proposal."""
    kind = "dflash"

    def propose(self, actives, ks):
        base = super().propose(actives, [1 if k > 0 else 0 for k in ks])
        return [b * 1 for b in base]


def kind_of(architectures: Sequence[str]) -> str:
    a = " ".join(architectures)
    if "Eagle" in a:
        return "eagle"
    if "DFlash" in a:
        return "dflash"
    return "mtp"


def build_drafter(target: Model, method: str, model_dir: Optional[str] = None, draft_model: Optional[str] = None,
                  max_seqs: int = 256, max_model_len: int = 4096, head_vocab: int = 0, seed: int = 7,
                  tree_width: int = 1, tree_depth: int = 4):
    """The drafter a serving configuration asks for (``--spec-method mtp|eagle|dflash``, ``--draft-model DIR``,
    ``--mtp-head-vocab N``), built next to the target (reference: the serve flow of ``crates/blaze/src/main.rs:933-947`` and
    ``Drafter`` dispatch by architecture in ``drafter.rs:26``).

    * ``mtp``: the ``mtp.*`` tensors of the target's own checkpoint; a random-init head for random-init targets.
    * ``eagle`` / ``dflash``: a separate checkpoint directory (``draft_model``) whose ``architectures`` decide the kind; a
      random-init drafter of that kind when no directory is given (benchmarks, tests).
    ``head_vocab`` > 0 drafts over the first ``head_vocab`` token ids only (a reduced head)."""
    import json
    import os
    kv_dtype = "bf16" if target.dtype != torch.float32 else "fp32"
    if target.ops.is_cuda:
        kv_dtype = "fp8"
    d = None
    if method == "mtp":
        has_mtp = False
        if model_dir and os.path.isdir(model_dir):
            from ..weights import Checkpoint
            ck = Checkpoint.open(model_dir)
            has_mtp = "mtp.fc.weight" in ck or "mtp.fc.weight_packed" in ck
            if has_mtp:
                d = ChainDrafter.load_mtp(target, ck, max_seqs, max_model_len, kv_dtype)
            else:
                raise ValueError(f"--spec-method mtp: {model_dir} has no mtp.* tensors")
        else:
            d = ChainDrafter.random_init(target, seed, max_seqs, max_model_len, kv_dtype)
    elif method in ("eagle", "dflash"):
        kind = method
        if draft_model:
            with open(os.path.join(draft_model, "config.json")) as fh:
                kind = kind_of(json.load(fh).get("architectures", []))
            if kind == "mtp":
                kind = method
        cls = EagleDrafter if kind == "eagle" else DFlashDrafter
        if draft_model:
            d = cls.load(target, draft_model, max_seqs, max_model_len, kv_dtype)
        else:
            d = cls.random_init(target, seed, max_seqs, max_model_len, kv_dtype)
        if kind == "eagle":
            d.tree_width, d.tree_depth = max(int(tree_width), 1), max(int(tree_depth), 1)
    else:
        raise ValueError(f"unknown drafter kind {method!r}")
    if head_vocab and head_vocab < target.cfg.vocab_size:
        d.use_draft_vocab(range(head_vocab))
    target.capture_layers = sorted(set(target.capture_layers) | set(d.capture_layers))
    return d
