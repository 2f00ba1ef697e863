"""Paged KV pools, block tables and recurrent (Gated DeltaNet) state rows.

Pages hold 16 tokens.  Two pool layouts exist:

* ``logical`` — ``k[layer]``, ``v[layer]`` of shape ``[pages, kv_heads, 16, head_dim]`` in fp32 / bf16 /
  e4m3; used by the PyTorch oracle and on CPU.
* ``umma`` — one uint8 tensor ``[pages, kv_heads, 2, 16*head_dim]`` per layer holding e4m3 K in the
  shared-memory layout the tcgen05 attention kernel consumes directly (8-row × 16-byte core matrices:
  byte of token t, dim j at ``(t//8)*8*D + (j//16)*128 + (t%8)*16 + j%16``) followed by V transposed
  (``[head_dim][16 tokens]``), so that one 1-D bulk copy per (page, head) feeds both MMAs.

The reference keeps one-token pages and several KV dtypes (``crates/blaze/src/model.rs:499-583``,
``alloc_kv`` :517); its page bookkeeping is in ``engine.rs:1083-1164``.
"""
from __future__ import annotations

import os

from typing import Tuple, Sequence, Dict, List, Optional

import numpy as np
import torch

from .config import ModelConfig

PAGE = 16


def kv_bytes_per_token(cfg: ModelConfig, kv_dtype: str, tp_world: int = 1) -> int:
    n_attn = sum(1 for i in range(cfg.num_layers) if cfg.layer_type(i) == "full_attention")
    kvh = max(cfg.num_kv_heads // tp_world, 1)
    if kv_dtype in FP4_KV:
        return n_attn * 2 * kvh * (cfg.head_dim // 2 + cfg.head_dim // 16)      # 4-bit codes and one scale byte per 16
    esz = {"fp32": 4, "bf16": 2, "fp8": 1}[kv_dtype]
    return n_attn * 2 * kvh * cfg.head_dim * esz


FP4_KV = ("nvfp4", "nvfp4_4over6")       # NVFP4 rows with the plain block scale, or with the searched one


class Fp4Pool:
    """A K or V pool of NVFP4 rows seen as ``[pages, kv_heads, 16, D]``: indexing by pages dequantises those pages."""

    def __init__(self, rows: torch.Tensor, D: int):
        self.rows, self.D = rows, D
        self.shape = (*rows.shape[:-1], D)
        self.device = rows.device

    def __getitem__(self, pages):
        from .quant import nvfp4_kv_dequantize
        return nvfp4_kv_dequantize(self.rows[pages], self.D)


HEAD_MAJOR = os.environ.get("BLAZE_KV_HEAD_MAJOR", "0") == "1"


class KVCache:
    def __init__(self, cfg: ModelConfig, num_pages: int, max_seqs: int, max_pages_per_seq: int,
                 kv_dtype: str = "bf16", device="cpu", layout: str = "logical", tp_world: int = 1,
                 state_rows: Optional[int] = None, layers: Optional[Tuple[int, int]] = None):
        self.cfg, self.num_pages, self.max_seqs = cfg, num_pages, max_seqs
        self.max_pages_per_seq = max_pages_per_seq
        self.kv_dtype, self.layout, self.device = kv_dtype, layout, torch.device(device)
        self.kv_heads = max(cfg.num_kv_heads // tp_world, 1)
        D = cfg.head_dim
        tdt = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp8": torch.float8_e4m3fn, "nvfp4": torch.uint8,
               "nvfp4_4over6": torch.uint8}[kv_dtype]
        row = D // 2 + D // 16 if kv_dtype in FP4_KV else D       # NVFP4: a row's codes, then its block scales
        lo, hi = layers if layers is not None else (0, cfg.num_layers)      # a pipeline stage holds the caches of its layers only
        self.attn_layers = [i for i in range(lo, hi) if cfg.layer_type(i) == "full_attention"]
        self.gdn_layers = [i for i in range(lo, hi) if cfg.layer_type(i) == "linear_attention"]
        self.k: Dict[int, torch.Tensor] = {}
        self.v: Dict[int, torch.Tensor] = {}
        self.kv: Dict[int, torch.Tensor] = {}
        for i in self.attn_layers:
            if layout == "umma":
                assert kv_dtype == "fp8"
                if HEAD_MAJOR:
                    # storage [kv_heads, pages, 2, 16*D]: the pages of one head are neighbours in memory, so a CTA that
                    # walks a sequence's (mostly consecutive) pages for one head streams DRAM instead of hopping by
                    # kv_heads * 4 KB; the tensor is exposed page-first like the page-major form (strides tell the kernels)
                    self.kv[i] = torch.zeros(self.kv_heads, num_pages, 2, PAGE * D, dtype=torch.uint8, device=device).permute(1, 0, 2, 3)
                else:
                    self.kv[i] = torch.zeros(num_pages, self.kv_heads, 2, PAGE * D, dtype=torch.uint8, device=device)
            else:
                self.k[i] = torch.zeros(num_pages, self.kv_heads, PAGE, row, dtype=tdt, device=device)
                self.v[i] = torch.zeros(num_pages, self.kv_heads, PAGE, row, dtype=tdt, device=device)
        self._block_table = torch.zeros(max_seqs, max_pages_per_seq, dtype=torch.int32, device=device)
        self.block_table_host = np.zeros((max_seqs, max_pages_per_seq), dtype=np.int32)
        self._dirty: List[tuple] = []          # (row, first page slot, count) not yet uploaded
        # recurrent state rows: one per sequence row plus snapshot rows for the prefix cache / speculation
        self.state_rows = state_rows if state_rows is not None else max_seqs
        self.conv_state: Dict[int, torch.Tensor] = {}
        self.rec_state: Dict[int, torch.Tensor] = {}
        if self.gdn_layers:
            hk = max(cfg.linear_num_key_heads // tp_world, 1)
            hv = max(cfg.linear_num_value_heads // tp_world, 1)
            conv_dim = 2 * hk * cfg.linear_key_head_dim + hv * cfg.linear_value_head_dim
            act = torch.float32 if kv_dtype == "fp32" else torch.bfloat16
            for i in self.gdn_layers:
                self.conv_state[i] = torch.zeros(self.state_rows, conv_dim, cfg.linear_conv_kernel_dim - 1,
                                                 dtype=act, device=device)
                self.rec_state[i] = torch.zeros(self.state_rows, hv, cfg.linear_key_head_dim,
                                                cfg.linear_value_head_dim, dtype=torch.float32, device=device)

        # sparse-attention indexer: the raw index key of every token, paged like K and V (shared prefixes share them)
        self.idx_k: Dict[int, torch.Tensor] = {}
        if getattr(cfg, "indexer_heads", 0) > 0:
            act = torch.float32 if kv_dtype == "fp32" else torch.bfloat16
            for i in self.attn_layers:
                self.idx_k[i] = torch.zeros(num_pages, PAGE, cfg.indexer_head_dim, dtype=act, device=device)
        # n-gram embedding layers of this stage keep a token window and a convolution history per row
        self.ple = None
        ple_layers = [i for i in range(lo, hi) if i in set(getattr(cfg, "ple_layers", ()) or ())]
        if ple_layers:
            if not self.gdn_layers:
                raise ValueError("per-layer n-gram embeddings are kept with the recurrent state rows: the model needs linear-attention layers")
            from .models.qwen4 import PleState
            self.ple = PleState(cfg, ple_layers, self.state_rows, torch.float32 if kv_dtype == "fp32" else torch.bfloat16, device)

    # ------------------------------------------------------------------ block table
    def set_pages(self, row: int, pages: List[int], start: int = 0) -> None:
        """Record pages ``start..`` of sequence row ``row`` (host mirror + device)."""
        if not pages:
            return
        n = len(pages)
        self.block_table_host[row, start:start + n] = pages
        self._dirty.append((row, start, n))

    @property
    def block_table(self) -> torch.Tensor:
        """The device block table, with every pending ``set_pages`` applied (so no reader can see a stale table)."""
        if self._dirty:
            self.flush()
        return self._block_table

    def flush(self) -> None:
        """Upload the block-table entries changed since the last flush: one copy and one scatter, in stream order
        before the step that needs them (page boundaries are crossed by many sequences in the same step)."""
        if not self._dirty:
            return
        dirty, self._dirty = self._dirty, []
        if len(dirty) == 1 or self._block_table.device.type != "cuda":
            for row, start, n in dirty:
                self._block_table[row, start:start + n] = torch.from_numpy(
                    self.block_table_host[row, start:start + n].copy()).to(self._block_table.device)
            return
        W = self._block_table.shape[1]
        flat = np.concatenate([np.arange(row * W + start, row * W + start + n, dtype=np.int64) for row, start, n in dirty])
        vals = self.block_table_host.reshape(-1)[flat]
        buf = torch.empty(2, flat.size, dtype=torch.int64).pin_memory()
        buf[0].numpy()[:] = flat
        buf[1].numpy()[:] = vals
        d = buf.to(self._block_table.device, non_blocking=True)
        self._block_table.view(-1).index_put_((d[0],), d[1].to(torch.int32))

    def nbytes(self) -> int:
        n = 0
        for d in (self.k, self.v, self.kv, self.conv_state, self.rec_state, self.idx_k):
            n += sum(t.numel() * t.element_size() for t in d.values())
        return n + (self.ple.nbytes() if self.ple is not None else 0)

    # ------------------------------------------------------------------ recurrent state rows
    def copy_state(self, src: int, dst: int) -> None:
        """Copy the GDN conv + recurrent state of row ``src`` to row ``dst`` (``model.rs:2718``)."""
        for i in self.gdn_layers:
            self.conv_state[i][dst].copy_(self.conv_state[i][src])
            self.rec_state[i][dst].copy_(self.rec_state[i][src])
        if self.ple is not None:
            self.ple.copy(src, dst)

    def zero_state(self, row: int) -> None:
        for i in self.gdn_layers:
            self.conv_state[i][row].zero_()
            self.rec_state[i][row].zero_()
        if self.ple is not None:
            self.ple.zero(row)

    def write_fp4(self, layer: int, k: torch.Tensor, v: torch.Tensor, slot_mapping: torch.Tensor) -> None:
        """Quantise the new tokens' K and V rows ``[T, kv_heads, D]`` to NVFP4 into their slots (``nvfp4_4over6``: with the
        block-scale search)."""
        from .quant import nvfp4_kv_quantize
        search = self.kv_dtype == "nvfp4_4over6"
        page, off = slot_mapping.long() // PAGE, slot_mapping.long() % PAGE
        self.k[layer][page, :, off] = nvfp4_kv_quantize(k, search=search)
        self.v[layer][page, :, off] = nvfp4_kv_quantize(v, search=search)

    # ------------------------------------------------------------------ row moves (tree speculation)
    def move_rows(self, moves: Sequence[Sequence[tuple]], ops=None) -> None:
        """``moves[i]`` = ordered (src slot, dst slot) pairs of sequence i (flat slots: page * 16 + offset): copy the K/V
        rows in every attention layer.  Within a sequence the pairs apply in order (a later pair may overwrite an earlier
        pair's source); sequences share no slot.  With the CUDA op set and the kernel page layout this is one launch per
        layer (reference: ``Model::tree_moves``, crates/blaze/src/model.rs :3387)."""
        moves = [[(int(a), int(b)) for a, b in seq if a != b] for seq in moves]
        moves = [m for m in moves if m]
        if not moves:
            return
        D = self.cfg.head_dim
        if self.layout == "umma" and ops is not None and getattr(ops, "is_cuda", False):
            flat = [p for m in moves for p in m]
            seg = np.cumsum([0] + [len(m) for m in moves])
            src = torch.tensor([a for a, _ in flat], dtype=torch.int32, device=self.device)
            dst = torch.tensor([b for _, b in flat], dtype=torch.int32, device=self.device)
            segt = torch.tensor(seg.tolist(), dtype=torch.int32, device=self.device)
            for i in self.attn_layers:
                ops.kv_move_rows(self.kv[i], src, dst, segt, D)
            return
        for i in self.attn_layers:
            for a, b in (p for m in moves for p in m):
                sp, so, dp, do = a // PAGE, a % PAGE, b // PAGE, b % PAGE
                if self.layout == "umma":
                    buf = self.kv[i]
                    H = buf.shape[1]
                    for h in range(H):
                        kview = buf[dp, h, 0].view(2, D // 16, 8, 16)
                        kview[do // 8, :, do % 8] = buf[sp, h, 0].view(2, D // 16, 8, 16)[so // 8, :, so % 8].clone()
                        buf[dp, h, 1].view(D, 16)[:, do] = buf[sp, h, 1].view(D, 16)[:, so].clone()
                else:
                    self.k[i][dp, :, do] = self.k[i][sp, :, so].clone()
                    self.v[i][dp, :, do] = self.v[i][sp, :, so].clone()

    # ------------------------------------------------------------------ layout helpers (tests, host tier)
    @staticmethod
    def pack_umma_page(k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """k, v ``[16, D]`` e4m3 (viewed as uint8) → ``[2, 16*D]`` bytes in the kernel layout."""
        D = k.shape[1]
        kb = k.view(torch.uint8).view(2, 8, D // 16, 16).permute(0, 2, 1, 3).contiguous().view(-1)
        vb = v.view(torch.uint8).t().contiguous().view(-1)
        return torch.stack([kb, vb])

    @staticmethod
    def unpack_umma_page(buf: torch.Tensor, D: int):
        kb = buf[0].view(2, D // 16, 8, 16).permute(0, 2, 1, 3).contiguous().view(16, D)
        vb = buf[1].view(D, 16).t().contiguous()
        return kb.view(torch.float8_e4m3fn), vb.view(torch.float8_e4m3fn)

    def logical_kv(self, layer: int):
        """Return (k, v) ``[pages, kv_heads, 16, D]`` e4m3 whatever the layout (copy for ``umma``)."""
        if self.kv_dtype in FP4_KV:
            return Fp4Pool(self.k[layer], self.cfg.head_dim), Fp4Pool(self.v[layer], self.cfg.head_dim)
        if self.layout != "umma":
            return self.k[layer], self.v[layer]
        D = self.cfg.head_dim
        buf = self.kv[layer]
        P, H = buf.shape[0], buf.shape[1]
        kb = buf[:, :, 0].reshape(P, H, 2, D // 16, 8, 16).permute(0, 1, 2, 4, 3, 5).contiguous().view(P, H, 16, D)
        vb = buf[:, :, 1].reshape(P, H, D, 16).transpose(2, 3).contiguous()
        return kb.view(torch.float8_e4m3fn), vb.view(torch.float8_e4m3fn)
