"""Symmetric memory over NVLink and the in-kernel collectives built on it.

One allocation per rank is mapped into every peer (``torch.distributed._symmetric_memory``: cuMem handles exchanged
over the process group; an NVSwitch multicast address when the fabric supports it).  The arena is carved into the
buffers the fused kernels use: two alternating partial-sum buffers that the row-cut GEMMs write directly, the
broadcast targets for normed / quantised activations, and the flag pads of the rank barrier.

``SymmAllReduce`` is what ``TPGroup.fused`` holds.  It offers
  * ``all_reduce``   — in place on a partial-sum buffer (multimem or peer loads/stores inside one kernel);
  * ``reduce_norm``  — all-reduce + residual add + RMSNorm (+ NVFP4 / MXFP8 quantisation) in one kernel, leaving
    the residual stream sharded by rows between the two collectives of a layer.

The reference's transport for the same two operations is pinned host memory (``kernels/src/cuda/host_allreduce.cu``,
``blz_host_ar_open`` :420 with POSIX shm, ``host_ar_rmsnorm_kernel`` :280).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Tuple

import torch

from .._native import kernels
from ..linear import Linear, QuantAct
from ..quant import Format

VP = ctypes.c_void_p


def _arr(ptrs: List[int]):
    return (VP * len(ptrs))(*[VP(p) for p in ptrs])


class SymmArena:
    """A symmetric byte buffer: local tensor, peer base pointers, multicast base pointer (0 when absent)."""

    def __init__(self, group, device, nbytes: int):
        import torch.distributed._symmetric_memory as symm_mem
        self.nbytes = (nbytes + 4095) // 4096 * 4096
        self.local = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=torch.device(device))
        self.handle = symm_mem.rendezvous(self.local, group.pg)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        mc = 0
        try:
            mc = int(self.handle.multicast_ptr or 0)
        except Exception:
            mc = 0
        self.mc = mc
        self.rank, self.world = group.rank, group.world
        self.off = 0

    def carve(self, nbytes: int, align: int = 4096) -> int:
        off = (self.off + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError("symmetric arena exhausted")
        self.off = off + nbytes
        return off

    def view(self, off: int, nbytes: int) -> torch.Tensor:
        return self.local[off:off + nbytes]

    def peers(self, off: int) -> List[int]:
        return [p + off for p in self.ptrs]

    def mcast(self, off: int) -> int:
        return self.mc + off if self.mc else 0


class PushedRows:
    """Partial sums that a row-cut GEMM scattered into the owner ranks' slot buffers (``SymmAllReduce.gemm_push``)."""
    __slots__ = ("buf", "rows", "cols")

    def __init__(self, buf: int, rows: int, cols: int):
        self.buf, self.rows, self.cols = buf, rows, cols

    @property
    def shape(self):
        return (self.rows, self.cols)


class SymmAllReduce:
    def __init__(self, group, device, max_rows: int, hidden: int, use_multicast: bool = True, timeout_ms: int = 0):
        self.group, self.device = group, torch.device(device)
        self.lib = kernels()
        lib = self.lib
        lib.blz_comm_create.restype = VP
        lib.blz_comm_create.argtypes = [ctypes.c_int, ctypes.c_int, VP, VP, ctypes.c_int]
        lib.blz_gemm_fuse_allreduce.argtypes = [VP, VP, VP, VP, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        lib.blz_comm_allreduce.argtypes = [VP, VP, VP, VP, VP, ctypes.c_longlong, ctypes.c_int, VP]
        lib.blz_comm_allreduce_norm.argtypes = [VP] + [VP] * 8 + [VP, VP, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                                  ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                                  ctypes.c_int, VP]
        lib.blz_comm_slots_norm.argtypes = [VP] + [VP] * 9 + [VP, VP, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                              ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                              ctypes.c_int, VP]
        lib.blz_gemm_push_rs.argtypes = [VP, VP, VP, VP, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        self.max_rows, self.hidden = max_rows, hidden
        row_tiles = (max_rows + 127) // 128
        self.in_bytes = max_rows * hidden * 2
        self.q_bytes = max_rows * hidden                      # e4m3 rows (NVFP4 uses half of it)
        self.sf_bytes = row_tiles * ((hidden + 63) // 64) * 512
        self.rs_bytes = max_rows * 4
        pad_bytes = int(lib.blz_comm_pad_bytes())
        # reduce-scatter by push: per rank two slot buffers [world][rows_per][hidden] that the peers' GEMM epilogues fill
        self.slot_bytes = group.world * ((max_rows + group.world - 1) // group.world) * hidden * 2
        total = (4 * self.in_bytes + self.in_bytes + self.q_bytes + self.sf_bytes + self.rs_bytes + pad_bytes + 2 * self.slot_bytes
                 + 48 * 4096)
        self.arena = SymmArena(group, device, total)
        a = self.arena
        self.off_in = [a.carve(self.in_bytes), a.carve(self.in_bytes)]
        self.off_out = a.carve(self.in_bytes)
        self.off_q = a.carve(self.q_bytes)
        self.off_sf = a.carve(self.sf_bytes)
        self.off_rs = a.carve(self.rs_bytes)
        self.off_pad = a.carve(pad_bytes)
        a.view(self.off_pad, pad_bytes).zero_()
        # fused GEMM + all-reduce: two zeroed accumulation buffers that every rank's epilogue reduces into, a flag row
        self.off_acc = [a.carve(self.in_bytes), a.carve(self.in_bytes)]
        for o in self.off_acc:
            a.view(o, self.in_bytes).zero_()
        self.off_pad2 = a.carve(4096)
        a.view(self.off_pad2, 4096).zero_()
        self.off_sig = a.carve(4096)               # arrival counters of kernels that signal instead of waiting
        a.view(self.off_sig, 4096).zero_()
        self.off_slot = [a.carve(self.slot_bytes), a.carve(self.slot_bytes)]
        self.off_slot_flag = a.carve(4096)         # two flag rows (one per slot buffer), 64 bytes apart
        a.view(self.off_slot_flag, 4096).zero_()
        self.push_state = torch.zeros(4, dtype=torch.int32, device=self.device)     # [finished CTAs, epoch]
        self.push_cur = 0
        self.sig_expect = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.gemm_state = torch.zeros(4, dtype=torch.int32, device=self.device)     # [done counter, epoch]
        self.acc_cur = 0
        self.timeout_ms = int(timeout_ms or os.environ.get("BLAZE_COMM_TIMEOUT_MS", "10000"))
        self.epoch = torch.zeros(int(lib.blz_comm_epoch_bytes()) // 4, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        group.barrier()
        self.comm = lib.blz_comm_create(group.rank, group.world, _arr(a.peers(self.off_pad)), VP(self.epoch.data_ptr()),
                                        int(timeout_ms or os.environ.get("BLAZE_COMM_TIMEOUT_MS", "10000")))
        if not self.comm:
            raise RuntimeError("blz_comm_create failed")
        lib.blz_comm_set_signals.argtypes = [VP, VP, VP]
        lib.blz_comm_set_signals(self.comm, _arr(a.peers(self.off_sig)), VP(self.sig_expect.data_ptr()))
        self.use_mc = bool(use_multicast and a.mc)
        # "gemm_red": the row-cut GEMM's epilogue reduces through the switch (one kernel per reduction, replicated norm);
        # "reduce_norm": GEMM writes partial sums, one kernel reduces + norms + quantises a row slice per rank.
        # measured on 2 B200s (Qwen3-8B, 256 rows): reduce_norm 21 us per reduction against 55 us for gemm_red, whose
        # epilogue also collapses on prefill-sized tiles; gemm_red stays available for experiments
        # "rs_push": the row-cut GEMM's epilogue sends each partial row into its owner rank's slot buffer through peer memory
        # (bulk copies from shared memory) and raises a flag; the owner's reduce + norm + quantise kernel starts without a rank
        # barrier (it waits for the flags and sums the slots from local memory).  Measured on 2 B200s (Qwen3-8B, 256 rows):
        # the flag-started reduction takes 9.8 us against 21.9 us, but the pushing GEMM takes 25.5 us against 15.3 us (the
        # same with every slot in local memory, so it is not NVLink: the per-CTA system-scope fence and the drain of the
        # asynchronous stores at the end of the kernel), 39.0 us against 35.9 us for the pair and 7.09 against 6.71 ms per
        # decode step - so it is opt-in.
        default = "reduce_norm"
        self.mode = os.environ.get("BLAZE_TP_FUSION", default)
        if self.mode == "gemm_red" and not self.use_mc:
            self.mode = "reduce_norm"
        # letting the consumer GEMM take over the closing wait measured equal on 2 B200s (33.2 us against 33.1 us for the
        # reduction + GEMM pair, 7.13 against 7.16 ms per decode step), so it stays opt-in
        self.defer_ok = os.environ.get("BLAZE_TP_DEFER", "0") == "1"
        self.cur = 0
        self.launches = 0

    @classmethod
    def create(cls, group, device, max_rows: int = 8192, hidden: int = 4096, **kw) -> "SymmAllReduce":
        return cls(group, device, max_rows, hidden, **kw)

    # ------------------------------------------------------------------ buffers
    def next_input(self, rows: int, cols: int) -> torch.Tensor:
        """A bf16 ``[rows, cols]`` view of the next partial-sum buffer; the producing GEMM writes into it."""
        n = rows * cols * 2
        if n > self.in_bytes:
            raise ValueError(f"partial-sum buffer too small for {rows}x{cols}")
        self.cur ^= 1
        return self.arena.view(self.off_in[self.cur], n).view(torch.bfloat16).view(rows, cols)

    def _which(self, x: torch.Tensor) -> Optional[int]:
        base = self.arena.local.data_ptr()
        for i, off in enumerate(self.off_in):
            if x.data_ptr() == base + off:
                return i
        return None

    def _stream(self) -> VP:
        return VP(torch.cuda.current_stream(self.device).cuda_stream)

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """Sum ``x`` over ranks.  ``x`` should be a buffer from :meth:`next_input` (otherwise it is copied in)."""
        if x.dtype != torch.bfloat16 or not x.is_contiguous():
            return None
        nbytes = x.numel() * 2
        if nbytes > self.in_bytes or nbytes % 16:
            return None
        i = self._which(x)
        if i is None:
            buf = self.next_input(x.shape[0], x.numel() // x.shape[0]).view(x.shape)
            buf.copy_(x)
            x, i = buf, self.cur
        a = self.arena
        off = self.off_in[i]
        mc = a.mcast(off) if self.use_mc else 0
        blocks = max(1, min(64, (nbytes // 16 + 511) // 512 // max(self.group.world, 1) + 1))
        rc = self.lib.blz_comm_allreduce(self.comm, _arr(a.peers(off)), _arr(a.peers(off)), VP(mc), VP(mc), nbytes, blocks,
                                         self._stream())
        if rc != 0:
            raise RuntimeError(f"blz_comm_allreduce failed: {rc}")
        self.launches += 1
        return x

    def gemm_allreduce(self, ops, lin: Linear, x, rows: int) -> torch.Tensor:
        """``sum over ranks of (x @ W_shard^T)`` in ONE kernel: the tcgen05 GEMM's epilogue adds each bf16 tile into every
        rank's accumulation buffer with ``multimem.red`` and the kernel ends with a cross-rank barrier.  Returns the
        complete ``[rows, N]`` sum in local memory; the consumer must hand the buffer back zeroed (``zero_src``)."""
        n = rows * lin.N * 2
        if n > self.in_bytes:
            raise ValueError("accumulation buffer too small")
        self.acc_cur ^= 1
        off = self.off_acc[self.acc_cur]
        a = self.arena
        rc = self.lib.blz_gemm_fuse_allreduce(VP(a.mcast(off)), VP(self.gemm_state.data_ptr()), _arr(a.peers(self.off_pad2)),
                                              VP(self.gemm_state.data_ptr() + 4), self.group.rank, self.group.world,
                                              self.timeout_ms)
        if rc != 0:
            raise RuntimeError(f"blz_gemm_fuse_allreduce failed: {rc}")
        out = a.view(off, n).view(torch.bfloat16).view(rows, lin.N)
        ops.linear(lin, x, out=out, wide=False)
        self.launches += 1
        return out

    def gemm_push(self, ops, lin: Linear, x, rows: int):
        """Row-cut projection whose epilogue scatters the partial sums to their owner ranks (reduce-scatter by push): returns
        a token for :meth:`reduce_norm` instead of a tensor — the sums only exist once the owners have reduced their slots."""
        per = self.rows_per(rows)
        if self.group.world * per * lin.N * 2 > self.slot_bytes or lin.N % 32:
            raise ValueError("slot buffer too small (or N not a multiple of 32) for the pushed reduce-scatter")
        self.push_cur ^= 1
        b = self.push_cur
        a = self.arena
        rc = self.lib.blz_gemm_push_rs(_arr(a.peers(self.off_slot[b])), _arr(a.peers(self.off_slot_flag + 64 * b)),
                                       VP(self.push_state.data_ptr()), VP(self.push_state.data_ptr() + 4), self.group.rank,
                                       self.group.world, per)
        if rc != 0:
            raise RuntimeError(f"blz_gemm_push_rs failed: {rc}")
        # C is not written in this mode; any valid [rows, N] bf16 view serves as the output argument
        dummy = a.view(self.off_in[0], rows * lin.N * 2).view(torch.bfloat16).view(rows, lin.N)
        ops.linear(lin, x, out=dummy, wide=False, sk=False)
        self.launches += 1
        return PushedRows(b, rows, lin.N)

    def rows_per(self, T: int) -> int:
        return (T + self.group.world - 1) // self.group.world

    def shard_rows(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's slice of a full ``[T, H]`` tensor as a fresh ``[rows_per, H]`` residual shard."""
        T = x.shape[0]
        per = self.rows_per(T)
        lo = self.group.rank * per
        out = torch.zeros(per, x.shape[1], dtype=x.dtype, device=x.device)
        hi = min(T, lo + per)
        if hi > lo:
            out[:hi - lo] = x[lo:hi]
        return out

    def reduce_norm(self, partial: torch.Tensor, residual: Optional[torch.Tensor], norm_w: Optional[torch.Tensor],
                    eps: float, zero_centered: bool, quant_for: Optional[Linear] = None, defer: bool = False):
        """``partial``: this rank's ``[T, H]`` partial sums in a buffer from :meth:`next_input`.
        ``residual``: this rank's ``[rows_per, H]`` slice of the residual stream (updated in place).
        Returns the normed rows on every rank: a bf16 ``[T, H]`` tensor or a :class:`QuantAct`.
        With ``norm_w=None`` the summed (+ residual) rows are returned unnormalised.
        ``defer``: the caller promises that the result's first consumer is ``ops.linear``; for quantised results of
        decode-sized steps the kernel then only signals the peers on its way out and the GEMM waits for their flags
        after it has started fetching its weights (``QuantAct.wait``)."""
        pushed = partial if isinstance(partial, PushedRows) else None
        if pushed is not None:
            T, H, i = pushed.rows, pushed.cols, 0
        else:
            T, H = partial.shape
            i = self._which(partial)
            if i is None:
                buf = self.next_input(T, H)
                buf.copy_(partial)
                partial, i = buf, self.cur
        mode = 0
        if quant_for is not None and quant_for.act_quant and norm_w is not None:
            # (an FP8 block-scale consumer takes MXFP8 rows only when its weight was re-expressed in MXFP8; its exact kernel
            # quantises bf16 rows itself)
            mx = quant_for.fmt == Format.MXFP8 or (quant_for.fmt == Format.FP8_BLOCK and (quant_for.cuda_pack or {}).get("kind") == 2)
            mode = 1 if quant_for.fmt == Format.NVFP4 else (2 if mx else 0)
        a = self.arena
        off_in = self.off_in[i]
        off_out = self.off_out if mode == 0 else self.off_q
        mc = self.use_mc
        per = self.rows_per(T)
        blocks = max(1, min(per, 512))
        defer = bool(defer and self.defer_ok and mode != 0 and T <= 256)
        if pushed is not None:
            rc = self.lib.blz_comm_slots_norm(
                self.comm, VP(a.local.data_ptr() + self.off_slot[pushed.buf]), VP(a.local.data_ptr() + self.off_slot_flag + 64 * pushed.buf),
                VP(self.push_state.data_ptr() + 4), _arr(a.peers(off_out)), _arr(a.peers(self.off_sf)), _arr(a.peers(self.off_rs)),
                VP(a.mcast(off_out) if mc else 0), VP(a.mcast(self.off_sf) if mc else 0), VP(a.mcast(self.off_rs) if mc else 0),
                VP(residual.data_ptr() if residual is not None else 0), VP(norm_w.data_ptr() if norm_w is not None else 0),
                T, H, per, eps, int(zero_centered), mode, blocks, int(defer), self._stream())
        else:
            rc = self._allreduce_norm(a, off_in, off_out, mc, residual, norm_w, T, H, per, eps, zero_centered, mode, blocks, defer)
        if rc != 0:
            raise RuntimeError(f"fused reduce + norm failed: {rc}")
        return self._result(a, off_out, mode, T, H, defer)

    def _allreduce_norm(self, a, off_in, off_out, mc, residual, norm_w, T, H, per, eps, zero_centered, mode, blocks, defer):
        return self.lib.blz_comm_allreduce_norm(
            self.comm, _arr(a.peers(off_in)), _arr(a.peers(off_out)), _arr(a.peers(self.off_sf)), _arr(a.peers(self.off_rs)),
            VP(a.mcast(off_in) if mc else 0), VP(a.mcast(off_out) if mc else 0), VP(a.mcast(self.off_sf) if mc else 0),
            VP(a.mcast(self.off_rs) if mc else 0), VP(residual.data_ptr() if residual is not None else 0),
            VP(norm_w.data_ptr() if norm_w is not None else 0), T, H, per, eps, int(zero_centered), mode, blocks, int(defer),
            self._stream())

    def _result(self, a, off_out, mode, T, H, defer):
        self.launches += 1
        if mode == 0:
            return a.view(off_out, T * H * 2).view(torch.bfloat16).view(T, H)
        if mode == 1:
            data = a.view(off_out, T * H // 2).view(T, H // 2)
            sf = a.view(self.off_sf, ((T + 127) // 128) * ((H + 63) // 64) * 512)
            rs = a.view(self.off_rs, T * 4).view(torch.float32)
            qa = QuantAct(Format.NVFP4, data, sf, rs, T, H)
        else:
            data = a.view(off_out, T * H).view(T, H)
            sf = a.view(self.off_sf, ((T + 127) // 128) * ((H + 127) // 128) * 512)
            qa = QuantAct(Format.MXFP8, data, sf, None, T, H)
        if defer:
            qa.wait = (a.local.data_ptr() + self.off_sig, self.sig_expect.data_ptr(), self.group.world, self.timeout_ms)
        return qa
