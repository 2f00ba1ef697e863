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
        if self.target.tp.world > 1:
            return          # the head is cut over the ranks: every rank reduces its own vocabulary shard, the pairs are merged
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
        # cut over the tensor-parallel ranks like the target's layers (every rank draws the full matrices from the seed and
        # keeps its part), so the drafter's steps run the target's collectives and its head is the target's sharded head
        tp = target.tp if target.tp.world > 1 else TPInfo()
        lm = Model.random_init(cfg, fmt, seed, target.device, target.dtype, tp, ops=target.ops)
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
        tp = target.tp if target.tp.world > 1 else TPInfo()
        tpr, tpw = tp.rank, tp.world
        lm = Model(cfg, dev, dt, tp, ops=target.ops)
        from .qwen3 import Attn, DenseMlp, Layer, _load_stacked_heads
        L = Layer()
        p = "mtp.layers.0."
        L.input_norm = ck.get(p + "input_layernorm.weight").to(dt).to(dev)
        L.post_norm = ck.get(p + "post_attention_layernorm.weight").to(dt).to(dev)
        A = Attn()
        A.heads, A.kv_heads = max(cfg.num_heads // tpw, 1), max(cfg.num_kv_heads // tpw, 1)
        D = cfg.head_dim
        A.qkv = _load_stacked_heads(ck, [p + "self_attn.q_proj", p + "self_attn.k_proj", p + "self_attn.v_proj"],
                                    [D * (2 if cfg.attn_output_gate else 1), D, D], [cfg.num_heads, cfg.num_kv_heads, cfg.num_kv_heads],
                                    tpr, tpw, dt, dev)
        A.o = Linear.load(ck, [p + "self_attn.o_proj"], Cut.COLS if tpw > 1 else Cut.ALL, tpr, tpw, dt, dev)
        if (p + "self_attn.q_norm.weight") in ck:
            A.q_norm = ck.get(p + "self_attn.q_norm.weight").to(dt).to(dev)
            A.k_norm = ck.get(p + "self_attn.k_norm.weight").to(dt).to(dev)
        L.attn = A
        mlp = DenseMlp()
        mlp.gate_up = Linear.load(ck, [p + "mlp.gate_proj", p + "mlp.up_proj"], Cut.ROWS if tpw > 1 else Cut.ALL, tpr, tpw, dt, dev)
        mlp.down = Linear.load(ck, [p + "mlp.down_proj"], Cut.COLS if tpw > 1 else Cut.ALL, tpr, tpw, dt, dev)
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
    def hidden_source(self, model: Model, hidden: torch.Tensor) -> torch.Tensor:
        """The rows the drafter consumes from a target step: the residual stream after the last layer."""
        return hidden

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

    def _step(self, chunks, x_in: torch.Tensor):
        """One pass of the drafter's layer over ``chunks`` → (greedy token, pre-norm hidden row) of every chunk's last row.
        The pass goes through the drafter engine's ``forward`` so that, under tensor parallelism, the other ranks run it too."""
        eng = self.engine
        if self.draft_head is not None:          # reduced draft vocabulary (single rank): head GEMM over the subset only
            batch = eng._build(chunks)
            x = self.m.forward(batch, eng.kv, x_in)
            return self._greedy(x, batch.logit_rows), x[batch.logit_rows.long()]
        ends, r = [], 0
        for c in chunks:
            r += len(c.tokens)
            ends.append(r - 1)
        toks, x = eng.forward(chunks, "greedy_hidden", hidden_in=x_in)
        return toks, x[torch.tensor(ends, dtype=torch.long, device=x.device)]

    MAX_FEED_ROWS = 4096          # rows per catch-up pass (a step's rows must fit the tensor-parallel exchange buffers)

    def _feed(self, states, dev):
        """Run the pending confirmed (token, hidden) pairs of ``states`` through the drafter's layer, at most MAX_FEED_ROWS rows
        per pass (a request's rows may be cut over passes) → (first draft token, pre-norm hidden of the last row) per state."""
        eng = self.engine
        if self.draft_head is not None or sum(len(st.pend_tokens) for st in states) <= self.MAX_FEED_ROWS:
            items, toks, hids = [], [], []
            for st in states:
                items.append((st.seq, st.pend_tokens, 1))
                toks += st.pend_tokens
                hids.append(st.pend_hidden)
            x_in = self._fuse(torch.tensor(toks, dtype=torch.int32, device=dev), torch.cat(hids))
            return self._step(eng.plan(items), x_in)
        out_tok: List[Optional[torch.Tensor]] = [None] * len(states)
        out_hid: List[Optional[torch.Tensor]] = [None] * len(states)
        batch, rows = [], 0                       # (state index, first row, last row, is the request's last piece)

        def flush():
            nonlocal batch, rows
            if not batch:
                return
            items, toks, hids, finals, ends, r = [], [], [], [], [], 0
            for i, a, b, fin in batch:
                st = states[i]
                items.append((st.seq, st.pend_tokens[a:b], 1 if fin else 0))
                toks += st.pend_tokens[a:b]
                hids.append(st.pend_hidden[a:b])
                r += b - a
                if fin:
                    finals.append(i)
                    ends.append(r - 1)
            x_in = self._fuse(torch.tensor(toks, dtype=torch.int32, device=dev), torch.cat(hids))
            chunks = eng.plan(items)
            if finals:
                tk, x = eng.forward(chunks, "greedy_hidden", hidden_in=x_in)
                for j, i in enumerate(finals):
                    out_tok[i] = tk[j:j + 1]
                    out_hid[i] = x[ends[j]:ends[j] + 1]
            else:
                eng.forward(chunks, "none", hidden_in=x_in)
            batch, rows = [], 0
        for i, st in enumerate(states):
            n, a = len(st.pend_tokens), 0
            while a < n:
                b = min(n, a + self.MAX_FEED_ROWS - rows)
                batch.append((i, a, b, b == n))
                rows += b - a
                a = b
                if rows >= self.MAX_FEED_ROWS:
                    flush()
        flush()
        return torch.cat(out_tok), torch.cat(out_hid)

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
        cur_tok, last = self._feed([st for _, _, st in todo], dev)
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
            cur_tok, last = self._step(chunks, x_in)
            toks_host = cur_tok.tolist()
        self.steps += 1
        self.proposed += sum(len(v) for v in out.values())
        return [out[id(a)] for a in actives]


class _Shell:
    """What the attention ops read from a model: config, rotary tables, the op set."""

    def __init__(self, cfg, target: Model):
        from ..config import inv_freq
        self.cfg, self.ops, self.device, self.dtype = cfg, target.ops, target.device, target.dtype
        self.tp = TPInfo()
        self.inv_freq = torch.tensor(inv_freq(cfg), dtype=torch.float32, device=target.device)
        self.rope_scale = cfg.rope.rope_scale()
        self.first_layer, self.last_layer = 0, 1
        self.is_first_stage = self.is_last_stage = True
        self.kv_rotate = False


class EagleDrafter:
    """EAGLE-style drafter: one decoder layer whose attention reads ``[norm(embed(token)) | norm(hidden)]`` (2H wide), fed
    with the target's hidden states of several layers fused by ``fc``; a low-rank candidate head picks a short list of
    tokens whose exact logits come from the full head; chains, or trees grown level by level from the top-k candidates.

    Reference: ``crates/blaze/src/eagle.rs`` — tensors ``fc``, ``fc_norm.{i}``, one ``layers.0`` block with a 2H-wide
    qkv, ``norm``, ``efficient_lm_head_down_proj`` + ``efficient_lm_head`` (:265-360); data flow of ``layer_with`` (:888);
    ``run`` chains (:565); ``run_tree`` / ``grow`` (:601-690: every level expands the K frontier rows, adds each row's
    top-K candidates as children and keeps the best K by path probability); ``head_merged`` (:694)."""

    kind = "eagle"

    def __init__(self, target: Model, cfg: ModelConfig, w: Dict[str, object], max_seqs: int, max_model_len: int, kv_dtype: str,
                 capture_layers: Sequence[int], candidates: int = 128, norm_output: bool = False):
        self.target, self.ops, self.cfg, self.w = target, target.ops, cfg, w
        self.capture_layers = list(capture_layers)
        self.candidates, self.norm_output = candidates, norm_output
        self.shell = _Shell(cfg, target)
        self.engine = Engine(self.shell, EngineConfig(max_seqs=max_seqs, max_model_len=max_model_len, kv_dtype=kv_dtype,
                                                      kv_tokens=max_seqs * max_model_len, use_graphs=False))
        from .qwen3 import Attn
        self.attn = Attn()
        self.attn.heads, self.attn.kv_heads = cfg.num_heads, cfg.num_kv_heads
        self.states: Dict[str, DraftState] = {}
        self.tree_width, self.tree_depth = 1, 4
        self.proposed = self.steps = 0
        self.draft_ids: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ construction
    @classmethod
    def random_init(cls, target: Model, seed: int = 7, max_seqs: int = 256, max_model_len: int = 4096, kv_dtype: str = "bf16",
                    n_capture: int = 3, rank: int = 64, candidates: int = 64):
        tc = target.cfg
        cfg = ModelConfig(**{**vars(tc), "num_layers": 1, "layer_types": ["full_attention"], "num_experts": 0,
                             "attn_output_gate": False, "qk_norm": False})
        cfg.rope = tc.rope
        H, D, I, V = cfg.hidden_size, cfg.head_dim, cfg.intermediate_size, cfg.vocab_size
        dev, dt = target.device, target.dtype
        g = torch.Generator(device=dev).manual_seed(seed)

        def lin(n, k):
            return Linear.from_dense(torch.randn(n, k, generator=g, device=dev) * 0.02, Format.DENSE, dtype=dt)
        one = lambda: torch.ones(H, dtype=dt, device=dev)      # noqa: E731
        L = tc.num_layers
        caps = sorted({min(L - 1, max(0, (i + 1) * L // (n_capture + 1))) for i in range(n_capture)})
        w = {"fc": lin(H, len(caps) * H), "fc_norm": [one() for _ in caps], "input_ln": one(), "hidden_ln": one(),
             "qkv": lin((cfg.num_heads + 2 * cfg.num_kv_heads) * D, 2 * H), "o": lin(H, cfg.num_heads * D), "post_ln": one(),
             "gate_up": lin(2 * I, H), "down": lin(H, I), "norm": one(), "lr_down": lin(rank, H), "lr_head": lin(V, rank),
             "lm_head": target.lm_head, "embed": target.embed}
        return cls(target, cfg, w, max_seqs, max_model_len, kv_dtype, caps, candidates)

    @classmethod
    def load(cls, target: Model, draft_dir: str, max_seqs: int, max_model_len: int, kv_dtype: str = "bf16"):
        """A drafter checkpoint directory (``config.json`` + safetensors) with the tensor names of ``eagle.rs:265-360``."""
        import json
        import os
        from ..weights import Checkpoint
        with open(os.path.join(draft_dir, "config.json")) as fh:
            raw = json.load(fh)
        ck = Checkpoint.open(draft_dir)
        tc = target.cfg
        cfg = ModelConfig(**{**vars(tc), "num_layers": 1, "layer_types": ["full_attention"], "num_experts": 0,
                             "attn_output_gate": False, "qk_norm": False,
                             "num_heads": int(raw.get("num_attention_heads", tc.num_heads)),
                             "num_kv_heads": int(raw.get("num_key_value_heads", tc.num_kv_heads)),
                             "head_dim": int(raw.get("head_dim", tc.head_dim)),
                             "intermediate_size": int(raw.get("intermediate_size", tc.intermediate_size))})
        cfg.rope = tc.rope
        dev, dt = target.device, target.dtype
        if int(raw.get("hidden_size", tc.hidden_size)) != tc.hidden_size or int(raw.get("vocab_size", tc.vocab_size)) != tc.vocab_size:
            raise ValueError("the drafter's hidden size / vocabulary differ from the target's")
        aux = (raw.get("eagle_config") or {}).get("eagle_aux_hidden_state_layer_ids") or []
        caps = [int(l) + 1 for l in aux] or [tc.num_layers - 1]         # the input of the layer after each aux layer

        def vec(name):
            return ck.get(name).to(dt).to(dev)

        def lin(*mods):
            return Linear.load(ck, list(mods), Cut.ALL, 0, 1, dt, dev)
        p = "layers.0." if "layers.0.self_attn.q_proj.weight" in ck else "midlayer."
        w = {"fc": lin("fc"), "fc_norm": [vec(f"fc_norm.{i}.weight") for i in range(len(caps))] if "fc_norm.0.weight" in ck else None,
             "input_ln": vec(p + "input_layernorm.weight"), "hidden_ln": vec(p + "hidden_norm.weight"),
             "qkv": lin(p + "self_attn.q_proj", p + "self_attn.k_proj", p + "self_attn.v_proj"), "o": lin(p + "self_attn.o_proj"),
             "post_ln": vec(p + "post_attention_layernorm.weight"), "gate_up": lin(p + "mlp.gate_proj", p + "mlp.up_proj"),
             "down": lin(p + "mlp.down_proj"), "norm": vec("norm.weight"),
             "lr_down": lin("efficient_lm_head_down_proj") if "efficient_lm_head_down_proj.weight" in ck else None,
             "lr_head": lin("efficient_lm_head") if "efficient_lm_head.weight" in ck else None,
             "lm_head": lin("lm_head") if "lm_head.weight" in ck else target.lm_head,
             "embed": vec("embed_tokens.weight") if "embed_tokens.weight" in ck else target.embed}
        head = raw.get("efficient_lm_head_config") or {}
        return cls(target, cfg, w, max_seqs, max_model_len, kv_dtype, caps, int(head.get("num_candidates", 128)),
                   bool(raw.get("norm_output", False)))

    def use_draft_vocab(self, ids: Sequence[int]) -> None:
        """Restrict proposals to ``ids`` (candidates outside are dropped before the exact logits are taken)."""
        self.draft_ids = torch.as_tensor(sorted(set(int(i) for i in ids)), dtype=torch.long, device=self.target.device)

    # ------------------------------------------------------------------ scheduler hooks
    def hidden_source(self, model: Model, hidden: torch.Tensor) -> torch.Tensor:
        """The rows the drafter consumes from a target step: the captured inputs of its capture layers, side by side."""
        return torch.cat([model.captured[l] for l in self.capture_layers], dim=1)

    def open(self, request_id: str) -> None:
        self.states[request_id] = DraftState(self.engine.open_from())

    def close(self, request_id: str) -> None:
        st = self.states.pop(request_id, None)
        if st is not None:
            self.engine.close(st.seq)

    observe = ChainDrafter.observe

    # ------------------------------------------------------------------ the layer
    def _fuse(self, hidden_cat: torch.Tensor) -> torch.Tensor:
        ops, eps = self.ops, self.cfg.rms_norm_eps
        H = self.cfg.hidden_size
        parts = []
        for i in range(len(self.capture_layers)):
            h = hidden_cat[:, i * H:(i + 1) * H].contiguous()
            if self.w["fc_norm"] is not None:
                h, _ = ops.norm(h, None, self.w["fc_norm"][i], eps, False)
            parts.append(h)
        return ops.linear(self.w["fc"], torch.cat(parts, dim=1).contiguous())

    def _layer(self, batch, tokens: torch.Tensor, hin: torch.Tensor):
        """One pass of the drafter's layer over the rows of ``batch``: returns (hidden for the next step, normed rows)."""
        ops, eps, w = self.ops, self.cfg.rms_norm_eps, self.w
        e = ops.embed(w["embed"], tokens)
        a, _ = ops.norm(e, None, w["input_ln"], eps, False)
        b, _ = ops.norm(hin.contiguous(), None, w["hidden_ln"], eps, False)
        qkv = ops.linear(w["qkv"], torch.cat([a, b], dim=1).contiguous())
        rope = ops.rope_tables(self.shell, batch)
        q, _ = ops.attn_prep_store(qkv, self.attn, self.shell, batch, self.engine.kv, 0, rope)
        o = ops.attention(q, self.shell, batch, self.engine.kv, 0, self.cfg.head_dim ** -0.5)
        x = ops.add(hin.contiguous(), ops.linear(w["o"], o))
        h2, _ = ops.norm(x, None, w["post_ln"], eps, False)
        x = ops.add(x, ops.linear(w["down"], ops.silu_mul(ops.linear(w["gate_up"], h2))))
        normed, _ = ops.norm(x, None, w["norm"], eps, False)
        return (normed if self.norm_output else x), normed

    def _head_topk(self, normed: torch.Tensor, k: int):
        """Top ``k`` tokens per row with their probabilities: low-rank scores over the vocabulary pick ``candidates`` ids, the
        full head gives those ids' exact logits, a softmax over the candidates gives the probabilities."""
        ops, w = self.ops, self.w
        nf = normed.float()
        if w["lr_down"] is not None:
            scores = ops.linear(w["lr_head"], ops.linear(w["lr_down"], normed), out_dtype=torch.float32)
        else:
            scores = ops.linear(w["lm_head"], normed, out_dtype=torch.float32)
        if self.draft_ids is not None:
            keep = torch.full_like(scores, float("-inf"))
            keep[:, self.draft_ids] = scores[:, self.draft_ids]
            scores = keep
        C = min(self.candidates, scores.shape[1])
        cand = scores.topk(C, dim=1).indices                                   # [R, C]
        head = w["lm_head"]
        hw = (head.dequant() if head.fmt != Format.DENSE else head.w).to(nf.device)
        exact = torch.einsum("rh,rch->rc", nf, hw[cand].float())                # exact logits of the candidates
        probs = torch.softmax(exact, dim=1)
        top = probs.topk(min(k, C), dim=1)
        return cand.gather(1, top.indices), top.values

    def _extend(self, todo):
        """Feed the confirmed (hidden, next token) pairs of every request in ``todo``; returns per request the drafter's
        last hidden row and normed row (the state a chain or a tree starts from)."""
        eng, dev = self.engine, self.target.device
        for a, st in todo:
            eng.truncate(st.seq, st.fed)
        items, toks, hids = [], [], []
        for a, st in todo:
            items.append((st.seq, st.pend_tokens, 1))
            toks += st.pend_tokens
            hids.append(st.pend_hidden)
        chunks = eng.plan(items)
        batch = eng._build(chunks)
        x, normed = self._layer(batch, torch.tensor(toks, dtype=torch.int32, device=dev), self._fuse(torch.cat(hids)))
        rows = batch.logit_rows.long()
        for a, st in todo:
            st.fed += len(st.pend_tokens)
            st.pend_hidden, st.pend_tokens = None, None
        return x[rows], normed[rows]

    # ------------------------------------------------------------------ chains
    def propose(self, actives, ks: Sequence[int]) -> List[List[int]]:
        eng, dev = self.engine, self.target.device
        todo = [(a, self.states.get(a.req.request_id)) for a in actives]
        live = [(a, k, st) for (a, st), k in zip(todo, ks) if st is not None and st.pend_tokens]
        out: Dict[int, List[int]] = {id(a): [] for a in actives}
        if not live:
            return [out[id(a)] for a in actives]
        hid, normed = self._extend([(a, st) for a, k, st in live])
        depth = 0
        while live:
            tok, _ = self._head_topk(normed, 1)
            tok = tok[:, 0]
            for (a, k, st), t in zip(live, tok.tolist()):
                out[id(a)].append(int(t))
            depth += 1
            keep = [i for i, (a, k, st) in enumerate(live) if k > depth]
            if not keep:
                break
            live = [live[i] for i in keep]
            idx = torch.tensor(keep, device=dev)
            hid, tok = hid[idx], tok[idx]
            chunks = eng.plan([(st.seq, [int(t)], 1) for (a, k, st), t in zip(live, tok.tolist())])
            batch = eng._build(chunks)
            hid, normed = self._layer(batch, tok.to(torch.int32), hid)
        self.steps += 1
        self.proposed += sum(len(v) for v in out.values())
        return [out[id(a)] for a in actives]

    # ------------------------------------------------------------------ trees
    def propose_tree(self, actives, width: int, depth: int, max_nodes: int = 16):
        """One draft tree per request (``tree.DraftTree``; node 0 = the last accepted token).  Level 1 = the top ``width``
        candidates after the confirmed rows; every further level runs the ``width`` frontier nodes (each sees the committed
        context and its own path), adds every frontier node's top ``width`` candidates as children, and keeps the best
        ``width`` of them by path probability as the next frontier.  ``max_nodes`` caps the rows handed to verification:
        the best nodes by path probability, parents before children."""
        from ..tree import DraftTree
        eng, dev = self.engine, self.target.device
        sts = [self.states.get(a.req.request_id) for a in actives]
        live = [(i, a, st) for i, (a, st) in enumerate(zip(actives, sts)) if st is not None and st.pend_tokens]
        result: List[Optional[DraftTree]] = [None] * len(actives)
        if not live:
            return result
        hid0, normed0 = self._extend([(a, st) for _, a, st in live])
        K = max(1, width)
        toks, probs = self._head_topk(normed0, K)
        # per request: nodes[n] = (token, parent node or -1, path probability); hid[n] = the layer's output row of node n
        trees = []
        for j in range(len(live)):
            nodes = [(int(toks[j, c]), -1, float(probs[j, c])) for c in range(toks.shape[1])]
            trees.append({"nodes": nodes, "frontier": list(range(len(nodes))), "hid": {-1: hid0[j]}})
        group = max(self.cfg.num_heads // max(self.cfg.num_kv_heads, 1), 1)
        row_cap = min(32, max(64 // group, 1))                    # rows of one sequence the verify attention takes
        for level in range(2, max(depth, 1) + 1):
            # one pass over, for every request, the path closure of its frontier (node ids grow with depth, so sorting puts
            # parents first): a level-1 node is a root of the chunk (it sees the committed context), deeper nodes see
            # their ancestors among the chunk's rows as well
            chunks, tok_rows, hid_rows, spans = [], [], [], []
            for (i, a, st), t in zip(live, trees):
                need = set()
                for n in t["frontier"]:
                    m = n
                    while m >= 0:
                        need.add(m)
                        m = t["nodes"][m][1]
                order = sorted(need)
                if len(order) > row_cap:
                    order = order[:row_cap]
                    t["frontier"] = [n for n in t["frontier"] if n in set(order)]
                row_of = {n: r for r, n in enumerate(order)}
                eng.truncate(st.seq, st.fed)
                tokens = [t["nodes"][n][0] for n in order]
                parents = [-1 if t["nodes"][n][1] < 0 else row_of[t["nodes"][n][1]] for n in order]
                chunks += eng.plan_tree([(st.seq, tokens, parents)])
                tok_rows += tokens
                hid_rows += [t["hid"][t["nodes"][n][1]] for n in order]
                spans.append((order, row_of))
            batch = eng._build(chunks)
            x, normed = self._layer(batch, torch.tensor(tok_rows, dtype=torch.int32, device=dev), torch.stack(hid_rows))
            r0 = 0
            for t, (order, row_of) in zip(trees, spans):
                for n in order:
                    t["hid"][n] = x[r0 + row_of[n]]
                if t["frontier"]:
                    ct, cp = self._head_topk(normed[torch.tensor([r0 + row_of[n] for n in t["frontier"]], device=dev)], K)
                    cands = []
                    for fi, n in enumerate(t["frontier"]):
                        for c in range(ct.shape[1]):
                            cands.append((t["nodes"][n][2] * float(cp[fi, c]), int(ct[fi, c]), n))
                    cands.sort(key=lambda z: (-z[0], z[1]))
                    front = []
                    for score, tok, n in cands:
                        t["nodes"].append((tok, n, score))
                        if len(front) < K:
                            front.append(len(t["nodes"]) - 1)
                    t["frontier"] = front
                r0 += len(order)
        for (i, a, st), t in zip(live, trees):
            eng.truncate(st.seq, st.fed)
            # the rows handed to verification: best nodes by path probability, closed under parents, parents first
            ranked = sorted(range(len(t["nodes"])), key=lambda n: (-t["nodes"][n][2], n))
            chosen = set()
            for n in ranked:
                path, m = [], n
                while m >= 0 and m not in chosen:
                    path.append(m)
                    m = t["nodes"][m][1]
                if len(chosen) + len(path) + 1 <= max_nodes:
                    chosen.update(path)
            tree = DraftTree()
            idx = {}
            for n in sorted(chosen):
                tok, par, _ = t["nodes"][n]
                idx[n] = tree.add(0 if par < 0 else idx[par], tok)
            result[i] = tree if len(tree.token) > 1 else None
            self.proposed += len(tree.token) - 1
        self.steps += 1
        return result


class DFlashDrafter(ChainDrafter):
    """DFlash-style block drafter: the whole block of ``k`` tokens comes from ONE pass over ``k`` rows that all read the last
    confirmed hidden state (row j stands for position p + 1 + j and feeds the last confirmed token), instead of ``k``
    dependent passes; rows attend causally to the rows before them.  Cheaper per proposal than a chain, lower acceptance at
    depth (reference: ``crates/blaze/src/dflash.rs`` ``run`` :342, ``block`` :416, ``candidates`` :571)."""
    kind = "dflash"

    def propose(self, actives, ks: Sequence[int]) -> List[List[int]]:
        eng, dev = self.engine, self.target.device
        todo = [(a, k, self.states.get(a.req.request_id)) for a, k in zip(actives, ks)]
        todo = [(a, k, st) for a, k, st in todo if st is not None and st.pend_tokens and k > 0]
        out: Dict[int, List[int]] = {id(a): [] for a in actives}
        if not todo:
            return [out[id(a)] for a in actives]
        for a, k, st in todo:
            eng.truncate(st.seq, st.fed)
        # context pass: the confirmed pairs (their KV is what the block attends to)
        items, toks, hids = [], [], []
        for a, k, st in todo:
            items.append((st.seq, st.pend_tokens, 1))
            toks += st.pend_tokens
            hids.append(st.pend_hidden)
        batch = eng._build(eng.plan(items))
        x = self.m.forward(batch, eng.kv, self._fuse(torch.tensor(toks, dtype=torch.int32, device=dev), torch.cat(hids)))
        last = x[batch.logit_rows.long()]
        first = self._greedy(x, batch.logit_rows)
        for a, k, st in todo:
            st.fed += len(st.pend_tokens)
            st.pend_hidden, st.pend_tokens = None, None
        # block pass: k - 1 more rows per request, all fed with the first proposal and the last hidden row
        blk = [(a, k, st, j) for j, (a, k, st) in enumerate(todo) if k > 1]
        for (a, k, st), t in zip(todo, first.tolist()):
            out[id(a)].append(int(t))
        if blk:
            items, toks, hids = [], [], []
            for a, k, st, j in blk:
                t0 = int(first[j])
                items.append((st.seq, [t0] * (k - 1), k - 1))
                toks += [t0] * (k - 1)
                hids.append(last[j].unsqueeze(0).expand(k - 1, -1))
            batch = eng._build(eng.plan(items))
            x = self.m.forward(batch, eng.kv, self._fuse(torch.tensor(toks, dtype=torch.int32, device=dev), torch.cat(hids).contiguous()))
            more = self._greedy(x, batch.logit_rows).tolist()
            r = 0
            for a, k, st, j in blk:
                out[id(a)] += [int(t) for t in more[r:r + k - 1]]
                r += k - 1
        self.steps += 1
        self.proposed += sum(len(v) for v in out.values())
        return [out[id(a)] for a in actives]

    @classmethod
    def load(cls, target: Model, draft_dir: str, max_seqs: int, max_model_len: int, kv_dtype: str = "bf16"):
        """A DFlash checkpoint uses the one-layer head tensors under the ``mtp.`` names of ``load_mtp``."""
        return cls.load_mtp(target, draft_dir, max_seqs, max_model_len, kv_dtype)


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
