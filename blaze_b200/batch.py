"""One engine step's metadata: which rows belong to which sequence, where their KV goes.

Plays the role of the reference's ``StepMeta`` (``crates/blaze/src/engine.rs:43``) and ``plan``
(``engine.rs:1168``): built on the host, packed into ONE pinned int32 staging buffer and sent to
the device with a single copy (``engine.rs:220-326``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

PAGE = 16
TINY_ROWS = 8       # ... of which those with at most this many rows run in the two-CTAs-per-SM configuration
SMALL_ROWS = 64     # sequences with q_len * group <= this use the decode attention kernel


@dataclass
class SeqChunk:
    """Rows of one sequence in this step."""
    slot: int                 # row of the block table / recurrent-state table
    tokens: Sequence[int]     # new token ids (1 for decode, k+1 for verify, a chunk for prefill)
    start_pos: int            # position of tokens[0]  (== KV length before this step)
    want_logits: int = 1      # how many trailing rows need logits (0 = headless prefill chunk)
    pos3: Optional[Sequence[Sequence[int]]] = None   # M-RoPE: rotary positions (temporal, height, width) of the rows, 3 x n;
                                                     # None = all three equal start_pos + i + rope_delta
    rope_delta: int = 0       # added to the rotary position of text rows after image blocks (KV slots still follow start_pos)
    embeds: Optional[Sequence] = None                # (row offset in this chunk, tensor [k, hidden]) blocks that replace the
                                                     # token embeddings of those rows (image tokens)
    defer_state: bool = False # recurrent (GDN) layers read this sequence's state but do not store the advanced state:
                              # the rows are speculative and the accepted prefix is replayed afterwards (Engine.commit_state)
    parents: Optional[Sequence[int]] = None   # draft tree: parent row of each token within this chunk (-1 for the first,
                                              # parents[i] < i).  Row i then sits at position start_pos + depth(i), its KV at
                                              # slot start_pos + i, and it attends to the context plus its ancestors and itself.


@dataclass
class StepBatch:
    tokens: torch.Tensor          # [T] int32
    positions: torch.Tensor       # [T] int32
    slot_mapping: torch.Tensor    # [T] int32  flat KV slot (page*16 + offset) of each new token
    seq_of_row: torch.Tensor      # [T] int32  index into the per-sequence arrays
    slots: torch.Tensor           # [B] int32
    q_start: torch.Tensor         # [B+1] int32
    ctx_len: torch.Tensor         # [B] int32 KV length including this step's rows
    logit_rows: torch.Tensor      # [R] int32 rows whose logits are wanted
    item_seq: Optional[torch.Tensor] = None   # [items] attention row-block items (None = one per sequence)
    item_q0: Optional[torch.Tensor] = None
    positions3: Optional[torch.Tensor] = None # [3, T] int32 rotary positions when a chunk carries M-RoPE positions
    embed_over: Optional[List] = None         # (first row, tensor) blocks that overwrite token embeddings (image tokens)
    gdn_defer: Optional[torch.Tensor] = None  # [B] int32, set when a chunk defers its recurrent state: 1 = do not store
    h_gdn_defer: Optional[List[int]] = None
    tree_mask: Optional[torch.Tensor] = None  # [T] int32, set when a chunk carries a draft tree: bit j = the row may see the
                                              # j-th new token of its sequence (causal rows: bits 0..own index)
    tiny_rows_max: int = 0        # largest q_len * group among sequences with at most TINY_ROWS rows (plain decode)
    num_tiny: int = 0
    small_rows_max: int = 0       # largest q_len * group among the other sequences handled by the decode attention kernel
    num_small: int = 0
    num_large: int = 0            # sequences handled by the row-block (prefill) attention kernel
    # host mirrors (python ints) for the oracle path and for planning
    h_slots: List[int] = field(default_factory=list)
    h_q_start: List[int] = field(default_factory=list)
    h_ctx_len: List[int] = field(default_factory=list)
    h_logit_rows: List[int] = field(default_factory=list)
    num_rows: int = 0
    max_q_len: int = 1
    max_ctx: int = 0
    h2d_bytes: int = 0

    @property
    def num_seqs(self) -> int:
        return len(self.h_slots)

    @property
    def is_decode_only(self) -> bool:
        return self.max_q_len == 1


def tree_depths(parents: Sequence[int]) -> np.ndarray:
    """Depth of each row of a draft tree given as parent rows (-1 = the chunk's first token, depth 0)."""
    d = np.zeros(len(parents), np.int32)
    for i, p in enumerate(parents):
        if p >= i:
            raise ValueError("a draft tree lists parents before children")
        d[i] = 0 if p < 0 else d[p] + 1
    return d


def tree_masks(parents: Sequence[int]) -> np.ndarray:
    """Bit masks of a draft tree's rows: bit j of word i is set when row j is row i or one of its ancestors (at most 32 rows)."""
    if len(parents) > 32:
        raise ValueError("a draft tree has at most 32 rows")
    m = np.zeros(len(parents), np.int64)
    for i, p in enumerate(parents):
        m[i] = (1 << i) | (0 if p < 0 else m[p])
    return m.astype(np.uint32).view(np.int32) if len(parents) else m.astype(np.int32)


def build_batch(chunks: Sequence[SeqChunk], block_table_host: np.ndarray, device, pinned: Optional[torch.Tensor] = None,
                pad_rows_to: int = 0, attn_group: int = 0, all_items: bool = False) -> StepBatch:
    """Pack the step metadata into one int32 buffer and copy it to ``device`` once.

    ``attn_group`` > 0 sorts the sequences into the attention kernels' tiers (decode kernel: tiny / small row counts; row-block
    kernel: the rest, cut into items of 128 rows); ``all_items`` sends every sequence to the row-block kernel (models whose
    head_dim the decode kernel does not cover).

    ``pad_rows_to`` pads T (with rows of a dummy sequence that writes to slot -1 … never; rows are
    clamped to the last real row's data but flagged by ``seq_of_row = -1``) so that CUDA-graph
    buckets see fixed shapes.
    """
    B = len(chunks)
    T = sum(len(c.tokens) for c in chunks)
    Tp = max(T, pad_rows_to)
    tokens = np.zeros(Tp, np.int32)
    positions = np.zeros(Tp, np.int32)
    slot_map = np.full(Tp, -1, np.int32)
    seq_of_row = np.full(Tp, -1, np.int32)
    slots = np.zeros(B, np.int32)
    q_start = np.zeros(B + 1, np.int32)
    ctx_len = np.zeros(B, np.int32)
    logit_rows: List[int] = []
    has_tree = any(c.parents is not None for c in chunks)
    tree_mask = np.zeros(Tp if has_tree else 0, np.int32)
    has_p3 = any(c.pos3 is not None or c.rope_delta for c in chunks)
    pos3 = np.zeros((3, Tp) if has_p3 else (0,), np.int32)
    embed_over: List = []
    r = 0
    max_q = 1
    max_ctx = 0
    for b, c in enumerate(chunks):
        n = len(c.tokens)
        tokens[r:r + n] = np.asarray(c.tokens, dtype=np.int64).astype(np.int32)
        pos = np.arange(c.start_pos, c.start_pos + n, dtype=np.int32)
        if c.parents is not None:
            positions[r:r + n] = c.start_pos + tree_depths(c.parents)
            tree_mask[r:r + n] = tree_masks(c.parents)
        else:
            positions[r:r + n] = pos
            if has_tree:
                tree_mask[r:r + n] = [-1 if j >= 31 else (2 << j) - 1 for j in range(n)]
        if has_p3:
            if c.pos3 is not None:
                pos3[:, r:r + n] = np.asarray(c.pos3, dtype=np.int32).reshape(3, n)
            else:
                pos3[:, r:r + n] = positions[r:r + n] + c.rope_delta
        if c.embeds:
            for off, t in c.embeds:
                embed_over.append((r + int(off), t))
        pages = block_table_host[c.slot, pos // PAGE]
        slot_map[r:r + n] = pages * PAGE + pos % PAGE
        seq_of_row[r:r + n] = b
        slots[b] = c.slot
        q_start[b + 1] = r + n
        ctx_len[b] = c.start_pos + n
        for j in range(n - c.want_logits, n):
            logit_rows.append(r + j)
        r += n
        max_q = max(max_q, n)
        max_ctx = max(max_ctx, c.start_pos + n)
    lr = np.asarray(logit_rows, np.int32)
    items_s: List[int] = []
    items_q: List[int] = []
    small_rows_max = num_large = tiny_rows_max = num_tiny = num_small = 0
    if attn_group > 0:
        tpb = max(128 // attn_group, 1)
        for b, c in enumerate(chunks):
            rows = len(c.tokens) * attn_group
            if all_items:
                rows = SMALL_ROWS + 1
            if rows <= TINY_ROWS:
                tiny_rows_max = max(tiny_rows_max, rows)
                num_tiny += 1
                continue
            if rows <= SMALL_ROWS:
                small_rows_max = max(small_rows_max, rows)
                num_small += 1
                continue
            num_large += 1
            for q0 in range(0, len(c.tokens), tpb):
                items_s.append(b)
                items_q.append(q0)
    has_defer = any(c.defer_state for c in chunks)
    defer = np.asarray([1 if c.defer_state else 0 for c in chunks] if has_defer else [], np.int32)
    parts = [tokens, positions, slot_map, seq_of_row, slots, q_start, ctx_len, lr,
             np.asarray(items_s, np.int32), np.asarray(items_q, np.int32), tree_mask, defer, pos3.reshape(-1)]
    total = sum(p.size for p in parts)
    if pinned is not None and pinned.numel() >= total:
        stage = pinned[:total]
    else:
        stage = torch.empty(total, dtype=torch.int32, pin_memory=torch.device(device).type == "cuda")
    sn = stage.numpy()
    off = 0
    offs = []
    for p in parts:
        sn[off:off + p.size] = p
        offs.append((off, p.size))
        off += p.size
    dev = stage.to(device, non_blocking=True)
    v = [dev[o:o + n] for o, n in offs]
    return StepBatch(tokens=v[0], positions=v[1], slot_mapping=v[2], seq_of_row=v[3], slots=v[4], q_start=v[5],
                     ctx_len=v[6], logit_rows=v[7], item_seq=v[8] if items_s else None,
                     item_q0=v[9] if items_s else None, tree_mask=v[10] if has_tree else None,
                     positions3=v[12].view(3, Tp) if has_p3 else None, embed_over=embed_over or None,
                     gdn_defer=v[11] if has_defer else None, h_gdn_defer=[int(x) for x in defer] if has_defer else None, h_slots=[int(s) for s in slots],
                     h_q_start=[int(x) for x in q_start], h_ctx_len=[int(x) for x in ctx_len],
                     h_logit_rows=logit_rows, tiny_rows_max=tiny_rows_max, num_tiny=num_tiny, small_rows_max=small_rows_max,
                     num_small=num_small, num_large=num_large, num_rows=Tp, max_q_len=max_q, max_ctx=max_ctx, h2d_bytes=total * 4)
