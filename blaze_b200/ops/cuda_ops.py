"""Kernel-backed op set (sm_100a).  Every method launches hand-written kernels from ``libblaze_kernels.so``
through its C ABI; nothing here falls back to the PyTorch oracle.

The op boundaries are those of the reference's forward pass (``crates/blaze/src/model.rs:2330-2551``), fused
differently: norm → (quantised) activation handed straight to the next GEMM, RoPE + q/k norm + FP8 page write in
one kernel, one attention kernel for prefill / decode / verify rows.
"""
from __future__ import annotations

import os

import ctypes
from typing import Dict, Optional, Tuple

import torch

from .. import quant
from .._native import kernels
from ..linear import Linear, QuantAct
from ..quant import Format

_c = ctypes
VP = ctypes.c_void_p


class CudaError(RuntimeError):
    pass


def _ptr(t: Optional[torch.Tensor]) -> VP:
    return VP(0) if t is None else VP(t.data_ptr())


class CudaOps:
    is_cuda = True
    name = "sm100a"

    def __init__(self, device):
        self.device = torch.device(device)
        self.lib = kernels()
        self.launches = 0
        self._held_stream = None
        self._held_depth = 0
        self.attn_prof = None      # optional int64 [8*3*16] wait-cycle counters of the decode attention kernel
        self._scratch: Dict[str, torch.Tensor] = {}
        self._retired: list = []
        self._sm = torch.cuda.get_device_properties(self.device).multi_processor_count
        lib = self.lib
        lib.blz_gemm_tc.restype = _c.c_int
        lib.blz_gemm_tc.argtypes = [_c.c_int, VP, _c.c_longlong, VP, _c.c_longlong, VP, _c.c_longlong, _c.c_int, _c.c_int,
                                    _c.c_int, VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int, VP, _c.c_int, _c.c_int, _c.c_int, VP]
        lib.blz_gemm_wait_flags.restype = _c.c_int
        lib.blz_gemm_wait_flags.argtypes = [VP, VP, _c.c_int, _c.c_int]
        lib.blz_gemm_argmax_parts.argtypes = [VP, VP]
        lib.blz_argmax_parts.argtypes = [VP, VP, _c.c_int, _c.c_int, VP, VP, _c.c_int, VP]
        lib.blz_gemm_wide.restype = _c.c_int
        lib.blz_gemm_wide.argtypes = [_c.c_int, VP, _c.c_longlong, VP, _c.c_longlong, VP, _c.c_longlong, _c.c_int, _c.c_int,
                                      _c.c_int, VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int, VP, _c.c_longlong, VP,
                                      _c.c_int, _c.c_int, _c.c_int, VP]
        lib.blz_gemm_sk.restype = _c.c_int
        lib.blz_gemm_sk.argtypes = [_c.c_int, VP, _c.c_longlong, VP, _c.c_longlong, VP, _c.c_longlong, _c.c_int, _c.c_int,
                                    _c.c_int, VP, VP, VP, VP, VP, _c.c_int, _c.c_int, VP]
        lib.blz_gemm_fp8_block.restype = _c.c_int
        lib.blz_gemm_fp8_block.argtypes = [VP, _c.c_longlong, VP, _c.c_longlong, VP, _c.c_longlong, _c.c_int, _c.c_int, _c.c_int,
                                           VP, _c.c_longlong, VP, VP, _c.c_int, VP]
        lib.blz_quant_fp8_block.restype = _c.c_int
        lib.blz_quant_fp8_block.argtypes = [VP, _c.c_longlong, VP, VP, _c.c_longlong, _c.c_int, _c.c_int, VP]
        # FP8 checkpoints with 128x128 fp32 block scales: "exact" keeps the stored codes and scales and promotes every K block
        # in fp32 (blz_gemm_fp8_block); "mx" re-quantises the weight once to e4m3 with e8m0 scales per 32 elements and runs the
        # hardware block-scaled MMA (faster, but only exact when the stored scales are powers of two)
        self._fp8_block_exact = os.environ.get("BLAZE_FP8_BLOCK", "exact") != "mx"
        lib.blz_gemm_sk_default_ks.restype = _c.c_int
        lib.blz_gemm_sk_default_ks.argtypes = [_c.c_int] * 4
        # decode-sized GEMMs (few output tiles) take the cluster split-K kernel; BLAZE_GEMM_SK=0 keeps them on the
        # one-CTA-per-tile kernel (A/B timing)
        self._sk_ok = os.environ.get("BLAZE_GEMM_SK", "1") != "0"
        self.SK_MAX_ROWS = 512
        self.tuning = None         # optional tune.Tuning: per-shape kernel choices measured on this device
        lib.blz_gemm_wide_ksplit.restype = _c.c_int
        lib.blz_gemm_wide_ksplit.argtypes = [_c.c_int, _c.c_int, _c.c_int]
        self._wide_ok = os.environ.get("BLAZE_GEMM_WIDE", "1") != "0"
        # tile-major weight storage measured no faster than row-major on B200 and keeps a second copy of the weights: opt-in
        self._tiled_ok = os.environ.get("BLAZE_TILED_WEIGHTS", "0") == "1"
        self._wide_ws = self._wide_ctr = None
        lib.blz_embed.argtypes = [VP, VP, VP, _c.c_int, _c.c_int, _c.c_int, VP]
        lib.blz_rmsnorm.argtypes = [VP, VP, VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_float, _c.c_int, _c.c_int, _c.c_int, VP]
        lib.blz_swiglu.argtypes = [VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int, _c.c_int, VP]
        lib.blz_attn_prep.argtypes = [VP, VP, VP, VP, VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                      _c.c_float, _c.c_float, _c.c_int, _c.c_int, _c.c_float, _c.c_float, _c.c_longlong,
                                      _c.c_longlong, _c.c_int, _c.c_longlong, _c.c_int, _c.c_int, VP]
        lib.blz_attn_tc.argtypes = [VP, VP, VP, VP, VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                    _c.c_longlong, _c.c_longlong, _c.c_float, _c.c_float, _c.c_float, _c.c_int, VP, VP, _c.c_int, VP]
        lib.blz_attn_decode_tree.argtypes = [VP, VP, VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                             _c.c_longlong, _c.c_longlong, _c.c_float, _c.c_float, _c.c_float, _c.c_int, _c.c_int, _c.c_int,
                                             _c.c_int, _c.c_int, VP, VP, _c.c_int, VP, VP, VP]
        lib.blz_kv_move_rows.argtypes = [VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int, _c.c_longlong, _c.c_longlong, VP]
        lib.blz_mul_sigmoid.argtypes = [VP, VP, _c.c_longlong, VP]
        lib.blz_add.argtypes = [VP, VP, VP, _c.c_longlong, VP]
        lib.blz_add_sigmoid_scaled.argtypes = [VP, VP, VP, VP, _c.c_int, _c.c_int, VP]
        lib.blz_gather_rows.argtypes = [VP, VP, VP, _c.c_int, _c.c_int, VP]
        lib.blz_argmax.argtypes = [VP, VP, VP, _c.c_int, _c.c_int, _c.c_longlong, _c.c_int, VP]
        lib.blz_moe_route.argtypes = [VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, VP]
        lib.blz_moe_plan.argtypes = [VP, VP, VP, VP, VP, _c.c_int, _c.c_int, VP]
        lib.blz_moe_gemm.restype = _c.c_int
        lib.blz_moe_gemm.argtypes = [_c.c_int, VP, _c.c_longlong, VP, _c.c_longlong, VP, _c.c_longlong, _c.c_int, _c.c_int, _c.c_int,
                                     _c.c_int, VP, VP, VP, VP, VP, VP, _c.c_int, VP]
        lib.blz_gemm_narrow.restype = _c.c_int
        lib.blz_gemm_narrow.argtypes = [_c.c_int, VP, _c.c_longlong, VP, _c.c_longlong, VP, _c.c_longlong, _c.c_int, _c.c_int, _c.c_int,
                                        VP, VP, VP, VP, VP, _c.c_int, _c.c_int, VP]
        # dense layers with few rows (single-user decoding, verify steps) and a large weight take the features-on-lanes kernel
        # with the K range split over a cluster (blz_gemm_narrow).  Measured on B200, NVFP4, captured-graph timing, against the
        # one-CTA-per-tile kernel: 1-32 rows 24576x4096 21 -> 16 us, 4096x12288 19 -> 16 us, 17408x5120 18 -> 16 us, 6144x4096
        # equal, 4096x4096 11.3 -> 12.0 us (loses); at 64 rows only the 24576-wide layer still wins, at 128 rows none does: both
        # kernels sit on a floor of about 10 us (launch, set-up, first load, reduction) at these sizes.  0 = never.
        self.NARROW_ROWS = int(os.environ.get("BLAZE_GEMM_NARROW_ROWS", "64"))
        self.NARROW_ALWAYS = os.environ.get("BLAZE_GEMM_NARROW_ALWAYS", "0") == "1"
        lib.blz_swiglu_live.argtypes = [VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int, _c.c_int, VP, VP]
        # routed rows per expert below this: the expert GEMMs put the features on the tensor-core lanes and only the live rows
        # on its columns (blz_moe_gemm); above it the 128-row tiles of the grouped GEMM are full enough (BLAZE_MOE_NARROW=0: never)
        self.MOE_NARROW_ROWS = 48 if os.environ.get("BLAZE_MOE_NARROW", "1") != "0" else 0
        lib.blz_moe_scatter.argtypes = [_c.c_int, VP, VP, VP, VP, VP, VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                        _c.c_int, VP]
        lib.blz_moe_combine.argtypes = [VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int, VP]
        self._route_counts = None
        lib.blz_gdn_conv.argtypes = [VP, _c.c_longlong, VP, VP, VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int, VP]
        lib.blz_gdn_recurrent.argtypes = [VP, VP, VP, _c.c_longlong, VP, VP, VP, VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int,
                                          _c.c_int, _c.c_int, VP]
        lib.blz_gdn_conv_runs.argtypes = [VP, _c.c_longlong, VP, VP, VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int, _c.c_int, VP]
        lib.blz_gdn_recurrent_upto.argtypes = [VP, VP, VP, _c.c_longlong, VP, VP, VP, VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int,
                                               _c.c_int, _c.c_int, _c.c_int, VP]
        lib.blz_gdn_chunk.argtypes = [VP, VP, VP, _c.c_longlong, VP, VP, VP, VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int,
                                      _c.c_int, _c.c_int, _c.c_int, VP]
        # Gated DeltaNet: sequences with at least this many new tokens in a step take the chunked tensor-core kernel (0 = never)
        self.GDN_CHUNK_MIN = int(os.environ.get("BLAZE_GDN_CHUNK_MIN", "64"))
        lib.blz_gdn_chunk_split.argtypes = [VP, VP, VP, _c.c_longlong, VP, VP, VP, VP, VP, VP, VP, VP, _c.c_int, _c.c_int, _c.c_int,
                                            _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, VP, VP]
        lib.blz_gdn_chunk_ws_bytes.restype = _c.c_longlong
        lib.blz_gdn_chunk_ws_bytes.argtypes = [_c.c_int, _c.c_int]
        # chunk-parallel preparation + sequential scan (two kernels) instead of the one fused kernel; 0 keeps the fused one
        self.GDN_SPLIT = os.environ.get("BLAZE_GDN_SPLIT", "1") != "0"
        self.GDN_SPLIT_MAX_WS = 4 << 30
        lib.blz_gated_rmsnorm.argtypes = [VP, VP, _c.c_longlong, VP, VP, _c.c_int, _c.c_int, _c.c_int, _c.c_float, _c.c_int, VP]
        lib.blz_status_take.restype = _c.c_int
        lib.blz_status_peek_async.restype = _c.c_int
        lib.blz_status_peek_async.argtypes = [VP, VP]

    # ------------------------------------------------------------------ plumbing
    def _stream(self) -> VP:
        s = self._held_stream
        return s if s is not None else VP(torch.cuda.current_stream(self.device).cuda_stream)

    def hold_stream(self) -> None:
        """Look the current stream up once for the launches that follow (a step of the engine issues hundreds, and the
        look-up costs more host time than the launch itself); ``release_stream`` ends it.  Calls nest."""
        if self._held_depth == 0:
            self._held_stream = VP(torch.cuda.current_stream(self.device).cuda_stream)
        self._held_depth += 1

    def release_stream(self) -> None:
        self._held_depth = max(self._held_depth - 1, 0)
        if self._held_depth == 0:
            self._held_stream = None

    def _check(self, code: int, what: str) -> None:
        self.launches += 1
        if code != 0:
            raise CudaError(f"{what} failed with cudaError {code}")

    def take_status(self) -> int:
        """Read and clear the device status word (non-zero = a bounded device wait ran out)."""
        return int(self.lib.blz_status_take())

    def status_peek(self, host_word: torch.Tensor) -> None:
        """Queue a copy of the status word into ``host_word`` (pinned int32) behind the work already on the stream."""
        rc = self.lib.blz_status_peek_async(VP(host_word.data_ptr()), self._stream())
        if rc != 0:
            raise CudaError(f"blz_status_peek_async failed: {rc}")

    def _buf(self, key: str, nbytes: int) -> torch.Tensor:
        """Scratch that only grows.  A buffer that is outgrown is kept alive: captured graphs of smaller steps still hold
        its address, and handing that memory back to the allocator would let other tensors land under their writes."""
        b = self._scratch.get(key)
        if b is None or b.numel() < nbytes:
            if b is not None:
                self._retired.append(b)
            b = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=self.device)
            self._scratch[key] = b
        return b

    # ------------------------------------------------------------------ weights → kernel layouts
    @staticmethod
    def tile_major(w: torch.Tensor) -> Tuple[torch.Tensor, int]:
        """Row-major weight bytes [N, row bytes] -> [ceil(N/128), kt, 128, 128] (zero padded): every 128-row x 128-byte
        operand tile becomes one contiguous 16 KB run, so a CTA streaming a weight tile reads DRAM pages end to end
        instead of touching a new page for every 128 bytes."""
        b = w.contiguous().view(torch.uint8).view(w.shape[0], -1)
        N, KB = b.shape
        NP, KP = (N + 127) // 128 * 128, (KB + 127) // 128 * 128
        if (NP, KP) != (N, KB):
            pad = torch.zeros(NP, KP, dtype=torch.uint8, device=b.device)
            pad[:N, :KB] = b
            b = pad
        kt = KP // 128
        t = b.view(NP // 128, 128, kt, 128).permute(0, 2, 1, 3).contiguous()
        # store each tile as the 128-byte-swizzled shared-memory image the tensor core reads (16-byte chunk c of row r
        # sits at chunk c ^ (r % 8)), so that the kernel fetches a whole 16 KB tile with ONE bulk copy
        v = t.view(NP // 128, kt, 16, 8, 8, 16)
        r = torch.arange(8, device=b.device).view(8, 1)
        c = torch.arange(8, device=b.device).view(1, 8)
        src = (c ^ r).view(1, 1, 1, 8, 8, 1).expand(NP // 128, kt, 16, 8, 8, 16)
        return torch.gather(v, 4, src).contiguous().view(NP // 128, kt, 128, 128), kt

    @staticmethod
    def swiglu_order(n_rows: int) -> torch.Tensor:
        """Row order that turns stacked ``[gate (I rows); up (I rows)]`` into groups of 16 gate rows followed by the 16 up
        rows of the same features, so that one 32-column group of the GEMM output holds both halves of 16 activations."""
        I = n_rows // 2
        g = torch.arange(I).view(I // 16, 16)
        return torch.cat([g, g + I], dim=1).reshape(-1)

    def pack(self, lin: Linear, tiled: Optional[bool] = None, swiglu: bool = False, exact_fp8: bool = True):
        """``tiled`` (default: off unless BLAZE_TILED_WEIGHTS=1): store the weight tile-major (see ``tile_major``); the grouped
        expert GEMM asks for row-major.  ``swiglu``: interleave the gate and up rows for the GEMM's SwiGLU epilogue (the
        packed weight is then only valid for ``linear_swiglu``)."""
        if lin.cuda_pack is not None:
            if bool(lin.cuda_pack.get("swiglu")) != bool(swiglu):
                raise CudaError("this weight was packed for the other epilogue (plain / SwiGLU)")
            return lin.cuda_pack
        pk = self._pack(lin, self.swiglu_order(lin.N).to(self.device) if swiglu else None, exact_fp8=exact_fp8)
        pk["swiglu"] = bool(swiglu)
        if tiled is None:
            tiled = self._tiled_ok
        pk["kt"] = 0
        if tiled:
            pk["w"], pk["kt"] = self.tile_major(pk["w"])
        lin.cuda_pack = pk
        return pk

    def _pack(self, lin: Linear, order: Optional[torch.Tensor] = None, exact_fp8: bool = True):
        """``order``: optional permutation of the output rows applied to the weight, its scales, alpha and bias.
        ``exact_fp8`` = False: an FP8 block-scale weight is re-expressed in MXFP8 (what the grouped expert GEMM consumes)."""
        dev = self.device

        def perm(t):
            return t if (order is None or t is None) else t.to(dev)[order]

        if lin.fmt == Format.DENSE:
            pk = {"kind": 0, "w": perm(lin.w.to(dev, torch.bfloat16)).contiguous(), "sf": None, "alpha": None}
        elif lin.fmt == Format.NVFP4:
            rows = (lin.N + 255) // 256 * 256
            sf = torch.zeros(rows, lin.K // 16, dtype=torch.uint8, device=dev)
            sf[:lin.N] = perm(lin.sf.to(dev).view(torch.uint8))
            pk = {"kind": 1, "w": perm(lin.w.to(dev)).contiguous(), "sf": quant.swizzle_sf_128x4(sf),
                  "alpha": perm(lin.alpha.to(dev, torch.float32)).contiguous()}
        elif lin.fmt == Format.FP8_BLOCK and self._fp8_block_exact and exact_fp8 and order is None and tuple(lin.block) == (128, 128) \
                and lin.K % 128 == 0 and tuple(lin.sf.shape) == ((lin.N + 127) // 128, lin.K // 128):
            pk = {"kind": 4, "w": lin.w.to(dev).view(torch.uint8).contiguous(), "sf": lin.sf.to(dev, torch.float32).contiguous(),
                  "alpha": None}
        elif lin.fmt in (Format.MXFP8, Format.FP8_BLOCK):
            if lin.fmt == Format.FP8_BLOCK:
                # 128x128 fp32 block scales have no native MMA mode: re-express the weight as e4m3 with one e8m0
                # scale per 32 elements (exact when the block scales are powers of two).
                q, e8 = quant.mxfp8_quantize(lin.dequant().to(dev))
            else:
                q, e8 = lin.w.to(dev), lin.sf.to(dev)
            rows = (lin.N + 255) // 256 * 256
            sf = torch.full((rows, lin.K // 32), 127, dtype=torch.uint8, device=dev)
            sf[:lin.N] = perm(e8.view(torch.uint8))
            alpha = None if lin.fmt == Format.FP8_BLOCK else perm(lin.alpha.to(dev, torch.float32)).contiguous()
            pk = {"kind": 2, "w": perm(q.view(torch.uint8)).contiguous(), "sf": quant.swizzle_sf_128x4(sf), "alpha": alpha}
        else:  # per-channel / per-tensor FP8
            pk = {"kind": 3, "w": perm(lin.w.to(dev).view(torch.uint8)).contiguous(), "sf": None,
                  "alpha": perm(lin.alpha.to(dev, torch.float32)).contiguous()}
        pk["bias"] = None if lin.bias is None else perm(lin.bias.to(dev, torch.bfloat16)).contiguous()
        return pk

    # ------------------------------------------------------------------ activation quantisation
    def _alloc_qact(self, fmt: Format, T: int, K: int) -> QuantAct:
        dev = self.device
        if fmt == Format.NVFP4:
            data = torch.empty(T, K // 2, dtype=torch.uint8, device=dev)
            sf = torch.empty(((T + 127) // 128) * ((K + 63) // 64) * 512, dtype=torch.uint8, device=dev)
            rs = torch.empty(T, dtype=torch.float32, device=dev)
        else:
            data = torch.empty(T, K, dtype=torch.uint8, device=dev)
            sf = torch.empty(((T + 127) // 128) * ((K + 127) // 128) * 512, dtype=torch.uint8, device=dev)
            rs = None
        return QuantAct(fmt, data, sf, rs, T, K)

    def _qmode(self, lin: Optional[Linear]) -> int:
        """Activation format the producer's epilogue should emit for ``lin``: 0 bf16, 1 NVFP4, 2 MXFP8.  (The exact FP8
        block-scale GEMM quantises its bf16 input itself, to e4m3 with one fp32 scale per 1x128 group.)"""
        if lin is None or not lin.act_quant:
            return 0
        if lin.fmt == Format.NVFP4:
            return 1
        if lin.fmt == Format.MXFP8:
            return 2
        if lin.fmt == Format.FP8_BLOCK:
            pk = lin.cuda_pack
            return 0 if (pk["kind"] == 4 if pk is not None else self._fp8_block_exact) else 2
        return 0

    def quantize_fp8_block(self, x: torch.Tensor):
        """bf16 ``[T, K]`` -> (e4m3 codes ``[T, K]``, fp32 scales ``[K / 128, T4]``) with one scale per row and 128 columns."""
        T, K = x.shape
        ld = (T + 3) // 4 * 4
        q = torch.empty(T, K, dtype=torch.uint8, device=self.device)
        sc = torch.empty(K // 128, ld, dtype=torch.float32, device=self.device)
        if x.stride(1) != 1:
            x = x.contiguous()
        self._check(self.lib.blz_quant_fp8_block(_ptr(x), x.stride(0), _ptr(q), _ptr(sc), ld, T, K, self._stream()), "quant_fp8_block")
        return q, sc

    def quantize_rows(self, x: torch.Tensor, lin: Linear) -> QuantAct:
        """bf16 ``[T, K]`` → the activation format ``lin`` consumes."""
        mode = self._qmode(lin)
        T, K = x.shape
        qa = self._alloc_qact(Format.NVFP4 if mode == 1 else Format.MXFP8, T, K)
        self._check(self.lib.blz_swiglu(_ptr(x), VP(0), _ptr(qa.data), _ptr(qa.sf), _ptr(qa.row_scale), T, K, mode, 1,
                                        self._stream()), "quantize_rows")
        return qa

    # ------------------------------------------------------------------ basics
    def embed(self, table, tokens):
        T, H = tokens.numel(), table.shape[1]
        out = torch.empty(T, H, dtype=torch.bfloat16, device=self.device)
        self._check(self.lib.blz_embed(_ptr(table), _ptr(tokens), _ptr(out), T, H, table.shape[0], self._stream()), "embed")
        return out

    def norm(self, x, residual, w, eps, zero_centered=False, quant_for: Optional[Linear] = None, zero_src: bool = False):
        T, H = x.shape
        mode = self._qmode(quant_for)
        new_res = residual if residual is not None else x
        if mode == 0:
            out = torch.empty_like(x)
            self._check(self.lib.blz_rmsnorm(_ptr(x), _ptr(residual), _ptr(w), _ptr(out), VP(0), VP(0), VP(0), T, H, eps,
                                             int(zero_centered), 0, int(zero_src), self._stream()), "rmsnorm")
            return out, new_res
        qa = self._alloc_qact(Format.NVFP4 if mode == 1 else Format.MXFP8, T, H)
        self._check(self.lib.blz_rmsnorm(_ptr(x), _ptr(residual), _ptr(w), VP(0), _ptr(qa.data), _ptr(qa.sf),
                                         _ptr(qa.row_scale), T, H, eps, int(zero_centered), mode, int(zero_src), self._stream()), "rmsnorm_q")
        return qa, new_res

    WIDE_WS_BYTES = 40 << 20

    def linear_swiglu(self, lin: Linear, x, quant_for: Optional[Linear] = None):
        """``silu(x @ Wg^T) * (x @ Wu^T)`` for a stacked ``[gate; up]`` weight with the activation computed in the GEMM's
        epilogue (the ``[T, 2I]`` intermediate never reaches memory); quantised for ``quant_for`` when that GEMM wants it."""
        exact8 = lin.fmt == Format.FP8_BLOCK and (lin.cuda_pack["kind"] == 4 if lin.cuda_pack is not None else self._fp8_block_exact)
        if lin.N % 32 or (lin.N // 2) % 8 or exact8:
            return self.silu_mul(self.linear(lin, x), quant_for=quant_for)
        act = self.linear(lin, x, swiglu=True)
        return self.quantize_rows(act, quant_for) if self._qmode(quant_for) else act

    def linear_argmax(self, lin: Linear, x, index_offset: int = 0, want_values: bool = False):
        """``argmax(x @ W^T)`` per row without writing the logits: the GEMM epilogue keeps the best (value, column) of each
        128-column tile and a small kernel merges the tiles (ties to the lower column, like ``argmax``)."""
        M = x.rows if isinstance(x, QuantAct) else x.shape[0]
        tiles = (lin.N + 127) // 128
        val = self._buf("amax_val", tiles * max(M, 1) * 4).view(torch.float32)
        idx = self._buf("amax_idx", tiles * max(M, 1) * 4).view(torch.int32)
        out = torch.empty(M, dtype=torch.int64, device=self.device)
        vals = torch.empty(M, dtype=torch.float32, device=self.device) if want_values else None
        if M == 0:
            return (out, vals) if want_values else out
        self.linear(lin, x, out_dtype=torch.float32, wide=False, argmax_parts=(val, idx))
        self._check(self.lib.blz_argmax_parts(_ptr(val), _ptr(idx), tiles, M, _ptr(out), _ptr(vals), index_offset,
                                              self._stream()), "argmax_parts")
        return (out, vals) if want_values else out

    def _linear_fp8_block(self, lin, pk, x, f32, out, swiglu, argmax_parts, wide, sk):
        if swiglu or argmax_parts is not None or wide or (sk is not None and sk is not False):
            raise CudaError("the FP8 block-scale GEMM has the plain epilogue only (bf16 / fp32 output, optional bias)")
        q = sc = None
        if isinstance(x, QuantAct):
            if x.wait is not None:
                raise CudaError("an activation with a pending peer wait cannot feed the FP8 block-scale GEMM")
            if x.fmt == Format.FP8_BLOCK:
                q, sc = x.data, x.sf              # already in 1x128 groups (quantize_fp8_block)
            else:
                x = x.dense
        M = q.shape[0] if q is not None else x.shape[0]
        if out is None:
            out = torch.empty(M, lin.N, dtype=torch.float32 if f32 else torch.bfloat16, device=self.device)
        if M == 0:
            return out
        if q is None:
            q, sc = self.quantize_fp8_block(x)
        self._check(self.lib.blz_gemm_fp8_block(_ptr(q), lin.K, _ptr(pk["w"]), lin.K, _ptr(out), out.stride(0), M, lin.N, lin.K,
                                                _ptr(sc), sc.stride(0), _ptr(pk["sf"]), _ptr(pk["bias"]), int(f32), self._stream()),
                    "gemm_fp8_block")
        return out

    def linear(self, lin: Linear, x, out_dtype=None, out: Optional[torch.Tensor] = None, bn: int = 0, max_ctas: int = 0,
               wide: Optional[bool] = None, ksplit: int = 0, swiglu: bool = False, argmax_parts=None, sk=None):
        """``wide``: None = choose; False = the 128-column kernel (needed by the fused all-reduce epilogue); True = insist on
        the wide-N kernel (raises when the shape is not covered).  ``sk``: None = choose; False = never; True or a K-slice
        count 1..8 = the cluster split-K kernel (bf16 output, row-major weights)."""
        pk = self.pack(lin, swiglu=swiglu)
        kind = pk["kind"]
        f32 = out_dtype == torch.float32
        n_out = lin.N // 2 if swiglu else lin.N
        sfa = rs = None
        if kind == 4:
            return self._linear_fp8_block(lin, pk, x, f32, out, swiglu, argmax_parts, wide, sk)
        if kind in (1, 2):
            if not isinstance(x, QuantAct):
                x = self.quantize_rows(x.contiguous(), lin)
            a, sfa, rs, M = x.data, x.sf, x.row_scale, x.rows
            lda = a.shape[1]
        elif kind == 3:
            xt = x.dense if isinstance(x, QuantAct) else x
            q, s = quant.fp8_rowwise_quantize(xt)
            a, rs, M = q.view(torch.uint8).contiguous(), s.float().contiguous(), xt.shape[0]
            lda = a.shape[1]
        else:
            a = x.contiguous()
            M, lda = a.shape[0], a.shape[1] * 2
        if argmax_parts is not None:
            out = argmax_parts[0]            # the logits are not written; any valid pointer will do
            ld_out = n_out
        elif out is None:
            out = torch.empty(M, n_out, dtype=torch.float32 if f32 else torch.bfloat16, device=self.device)
        if argmax_parts is None:
            ld_out = out.stride(0)
        if M == 0:
            return out
        w = pk["w"]
        kt = pk.get("kt", 0)
        ldb = 128 if kt else w.shape[1] * w.element_size()
        pending = getattr(x, "wait", None) if isinstance(x, QuantAct) else None
        if pending is not None:
            # the peers may still be writing these rows: the 128-column kernel waits for their flags after it has sent
            # its first weight tiles
            if wide:
                raise CudaError("an activation with a pending peer wait needs the 128-column GEMM")
            wide = False
            rc = self.lib.blz_gemm_wait_flags(VP(pending[0]), VP(pending[1]), pending[2], pending[3])
            if rc != 0:
                raise CudaError(f"blz_gemm_wait_flags failed: {rc}")
            x.wait = None
        big = self.NARROW_ALWAYS or (lin.N * lin.K >= 6144 * 4096 if M <= 32 else lin.N >= 16384)
        narrow = (M <= self.NARROW_ROWS and big and kind in (0, 1, 2) and lin.N % 128 == 0 and not f32 and argmax_parts is None
                  and pending is None and not kt and wide is None and bn == 0 and (sk is None or sk is False)
                  and (not swiglu or ld_out % 8 == 0) and (sfa is None or sfa.numel() >= 512))
        if narrow:
            self._check(self.lib.blz_gemm_narrow(kind, _ptr(a), lda, _ptr(w), ldb, _ptr(out), ld_out, M, lin.N, lin.K, _ptr(rs),
                                                 _ptr(pk["alpha"]), _ptr(pk["bias"]), _ptr(sfa), _ptr(pk["sf"]), 0, int(swiglu),
                                                 self._stream()), f"gemm_narrow kind {kind}")
            return out
        sk_able = not f32 and argmax_parts is None and pending is None and not kt
        if sk is None:
            sk = False
            if self._sk_ok and sk_able and wide is None and bn == 0 and M <= self.SK_MAX_ROWS:
                # Measured on B200 (NVFP4, 256 rows, captured-graph timing): splitting K over a cluster pays when the K range
                # is long and the tiles are few (4096 x 12288: 23.7 -> 22.2 us); for the other decode shapes the exchange of
                # fp32 partials through distributed shared memory (about 5 us per 64 KB tile) costs what the split saves.
                # A tuning table measured on this device (tune.tune_linear) overrides the rule.
                tiles = ((M + 127) // 128) * ((lin.N + 127) // 128)
                sk = lin.K >= 8192 and tiles <= 2 * self._sm // 2
                if self.tuning is not None:
                    from ..tune import bucket
                    hit = self.tuning.get(f"gemm{kind}", lin.N, lin.K, bucket(M))
                    if hit is not None:
                        sk = False if hit.get("kernel") != "sk" else (hit.get("ks") or True)
        if sk is not False and sk is not None:
            if not sk_able:
                raise CudaError("the split-K GEMM writes bf16 from row-major weights and has no arg-max / peer-wait epilogue")
            ks = 0 if sk is True else int(sk)
            self._check(self.lib.blz_gemm_sk(kind, _ptr(a), lda, _ptr(w), ldb, _ptr(out), ld_out, M, lin.N, lin.K,
                                             _ptr(rs), _ptr(pk["alpha"]), _ptr(pk["bias"]), _ptr(sfa), _ptr(pk["sf"]),
                                             ks, int(swiglu), self._stream()), f"gemm_sk kind {kind}")
            return out
        if wide is None:
            # Measured on B200 (Qwen3-8B shapes, captured-graph timing): 256-feature tiles win for block-scaled prefill GEMMs
            # (NVFP4 2048x24576x4096: 156 -> 119 us); the swapped orientation wins for the very wide bf16 head
            # (256x151936x4096: 346 -> 315 us) but not for the per-layer decode GEMMs, which stay on the 128-column kernel.
            wide = self._wide_ok and bn == 0 and ((M <= 256 and kind == 0 and lin.N >= 32768 and not swiglu)
                                                  or (kind in (1, 2) and lin.N % 256 == 0 and M > 256))
        if wide:
            swap = M <= 256
            ks, ws, ctr = 1, None, None
            if swap:
                tok = 64 if M <= 64 else (128 if M <= 128 else 256)
                tiles = (lin.N + 127) // 128
                k_tiles = (lin.K + (64 if kind == 0 else 256 if kind == 1 else 128) - 1) // (64 if kind == 0 else 256 if kind == 1 else 128)
                ks = ksplit or 1          # the split along K is opt-in: its workspace round trip costs more than it saves so far
                while ks > 1 and tiles * ks * 128 * tok * 4 > self.WIDE_WS_BYTES:
                    ks -= 1
                if ks > 1:
                    if self._wide_ws is None:
                        self._wide_ws = torch.empty(self.WIDE_WS_BYTES, dtype=torch.uint8, device=self.device)
                        self._wide_ctr = torch.zeros(8192, dtype=torch.int32, device=self.device)
                    if tiles > self._wide_ctr.numel():
                        ks = 1
                    ws, ctr = self._wide_ws, self._wide_ctr
            self._check(self.lib.blz_gemm_wide(kind, _ptr(a), lda, _ptr(w), ldb, _ptr(out), out.stride(0), M, lin.N, lin.K,
                                               _ptr(rs), _ptr(pk["alpha"]), _ptr(pk["bias"]), _ptr(sfa), _ptr(pk["sf"]),
                                               int(f32), int(swap), ks, _ptr(ws), self.WIDE_WS_BYTES if ws is not None else 0,
                                               _ptr(ctr), max_ctas, kt, int(swiglu), self._stream()), f"gemm_wide kind {kind}")
            return out
        if argmax_parts is not None:
            rc = self.lib.blz_gemm_argmax_parts(_ptr(argmax_parts[0]), _ptr(argmax_parts[1]))
            if rc != 0:
                raise CudaError(f"blz_gemm_argmax_parts failed: {rc}")
        self._check(self.lib.blz_gemm_tc(kind, _ptr(a), lda, _ptr(w), ldb, _ptr(out), ld_out, M, lin.N, lin.K,
                                         _ptr(rs), _ptr(pk["alpha"]), _ptr(pk["bias"]), _ptr(sfa), _ptr(pk["sf"]),
                                         int(f32), bn, max_ctas, VP(0), 0, kt, int(swiglu), self._stream()), f"gemm kind {kind}")
        return out

    def silu_mul(self, gu, quant_for: Optional[Linear] = None):
        T, I2 = gu.shape
        I = I2 // 2
        mode = self._qmode(quant_for)
        if mode == 0:
            out = torch.empty(T, I, dtype=torch.bfloat16, device=self.device)
            self._check(self.lib.blz_swiglu(_ptr(gu), _ptr(out), VP(0), VP(0), VP(0), T, I, 0, 0, self._stream()), "swiglu")
            return out
        qa = self._alloc_qact(Format.NVFP4 if mode == 1 else Format.MXFP8, T, I)
        self._check(self.lib.blz_swiglu(_ptr(gu), VP(0), _ptr(qa.data), _ptr(qa.sf), _ptr(qa.row_scale), T, I, mode, 0,
                                        self._stream()), "swiglu_q")
        return qa

    def mul_sigmoid(self, x, gate):
        x = x.contiguous()
        self._check(self.lib.blz_mul_sigmoid(_ptr(x), _ptr(gate.contiguous()), x.numel(), self._stream()), "mul_sigmoid")
        return x

    def add(self, a, b):
        out = torch.empty_like(a)
        self._check(self.lib.blz_add(_ptr(a), _ptr(b), _ptr(out), a.numel(), self._stream()), "add")
        return out

    def add_sigmoid_scaled(self, a, b, gate_logit):
        out = torch.empty_like(a)
        self._check(self.lib.blz_add_sigmoid_scaled(_ptr(a), _ptr(b), _ptr(gate_logit.contiguous()), _ptr(out), a.shape[0],
                                                    a.shape[1], self._stream()), "add_sigmoid_scaled")
        return out

    def gather_rows(self, x, rows):
        R, H = rows.numel(), x.shape[1]
        out = torch.empty(R, H, dtype=x.dtype, device=self.device)
        self._check(self.lib.blz_gather_rows(_ptr(x), _ptr(rows), _ptr(out), R, H, self._stream()), "gather_rows")
        return out

    def all_reduce(self, x, group=None):
        if group is None or group.world == 1:
            return x
        return group.all_reduce(x)

    # ------------------------------------------------------------------ attention
    def rope_tables(self, model, batch):
        return None   # angles are computed inside the prep kernel

    def attn_prep_store(self, qkv, attn, model, batch, kv, layer_idx, rope):
        cfg = model.cfg
        T = qkv.shape[0]
        D = cfg.head_dim
        if kv.layout != "umma":
            raise CudaError("the CUDA attention path needs the FP8 'umma' KV layout (kv_dtype='fp8')")
        q = torch.empty(T, attn.heads, D, dtype=torch.bfloat16, device=self.device)
        gate = torch.empty(T, attn.heads, D, dtype=torch.bfloat16, device=self.device) if cfg.attn_output_gate else None
        # M-RoPE: three position streams [3, T]; frequency i reads stream 0 / 1 / 2 by the model's section sizes
        pos, pos_stride, m0, m1 = batch.positions, 0, 0, 0
        sec = cfg.rope.mrope_section
        if getattr(batch, "positions3", None) is not None:
            pos, pos_stride = batch.positions3, batch.positions3.stride(0)
            if sec:
                m0, m1 = int(sec[0]), int(sec[0]) + int(sec[1])
            else:
                m0 = m1 = cfg.rotary_dim // 2          # no sections: every frequency follows the first stream
        self._check(self.lib.blz_attn_prep(_ptr(qkv), _ptr(q), _ptr(gate), _ptr(kv.kv[layer_idx]), _ptr(pos),
                                           _ptr(batch.slot_mapping), _ptr(model.inv_freq), _ptr(attn.q_norm), _ptr(attn.k_norm),
                                           T, attn.heads, attn.kv_heads, D, cfg.rotary_dim, cfg.rms_norm_eps,
                                           model.rope_scale, int(cfg.attn_output_gate), int(cfg.zero_centered_norm),
                                           1.0, 1.0, kv.kv[layer_idx].stride(0), kv.kv[layer_idx].stride(1),
                                           int(getattr(model, "kv_rotate", False)), pos_stride, m0, m1, self._stream()),
                    "attn_prep")
        return q, gate

    def kv_move_rows(self, pool, src, dst, seg, D):
        """Move KV rows between flat slots of one layer's pool (kernel page layout); ``seg`` = per-sequence move ranges."""
        self._check(self.lib.blz_kv_move_rows(_ptr(pool), _ptr(src), _ptr(dst), _ptr(seg), seg.numel() - 1, pool.shape[1], D,
                                              pool.stride(0), pool.stride(1), self._stream()), "kv_move_rows")

    def attention(self, q, model, batch, kv, layer_idx, scale, splits: int = 0, max_ctas: int = 0, allowed=None):
        """Sequences with few query rows (decode, verify) go to the decode kernel, the rest to the row-block kernel."""
        if allowed is not None:
            # a sparse selection (a context beyond an indexer's budget): the kernels read every key of a sequence, so these
            # steps take the masked torch attention over the pages on this device (correct, not fast)
            from . import ref
            kl, vl = kv.logical_kv(layer_idx)
            o = ref.paged_attention(q, kl, vl, kv.block_table, batch.h_slots, batch.h_q_start, batch.h_ctx_len, scale,
                                    tree_mask=getattr(batch, "tree_mask", None), allowed=allowed)
            return o.reshape(q.shape[0], -1).contiguous()
        T, Hq, D = q.shape
        Hkv = kv.kv_heads
        group = Hq // Hkv
        out = torch.empty(T, Hq, D, dtype=torch.bfloat16, device=self.device)
        B = batch.slots.numel()
        tiles = max((batch.max_ctx + 127) // 128, 1)
        # the decode kernel runs once per row tier: plain decode rows (<= 8 rows per kv head) take its two-CTAs-per-SM
        # configuration, short multi-token sequences (verify rows, prompt tails) the wider one
        tiers = []
        if D != 128:
            # the decode kernel is built for head_dim 128: every sequence is a row-block item here (engine.attn_all_items)
            if batch.item_seq is None or batch.tiny_rows_max or batch.small_rows_max:
                raise CudaError(f"head_dim {D}: the batch must send every sequence to the row-block attention kernel")
            if getattr(batch, "tree_mask", None) is not None:
                raise CudaError(f"head_dim {D}: draft trees are verified by the decode kernel, which covers head_dim 128 only")
        if batch.tiny_rows_max:
            tiers.append((1, batch.tiny_rows_max, batch.num_tiny))
        if batch.small_rows_max:
            tiers.append((batch.tiny_rows_max + 1 if batch.tiny_rows_max else 1, batch.small_rows_max, batch.num_small))
        if not tiers and not batch.num_large and D == 128:
            tiers.append((1, group * batch.max_q_len, B))
        for lo, hi, count in tiers:
            nmax = 16
            rb = (hi + nmax - 1) // nmax
            work = max(count, 1) * Hkv * rb
            sp = splits if splits > 0 else (1 if work >= 3 * self._sm else max(1, min(8, tiles, (3 * self._sm) // max(work, 1))))
            po = pm = None
            if sp > 1:
                n = B * Hkv * rb * sp * nmax
                po = self._buf("attn_part_o", n * D * 4).view(torch.float32)
                pm = self._buf("attn_part_ml", n * 2 * 4).view(torch.float32)
            self._check(self.lib.blz_attn_decode_tree(_ptr(q), _ptr(out), _ptr(kv.kv[layer_idx]), _ptr(kv.block_table),
                                                 _ptr(batch.slots), _ptr(batch.q_start), _ptr(batch.ctx_len), B, Hq, Hkv, D,
                                                 kv.block_table.stride(0), kv.kv[layer_idx].stride(0), kv.kv[layer_idx].stride(1),
                                                 scale, 1.0, 1.0, nmax, rb, lo, hi, sp,
                                                 _ptr(po), _ptr(pm), max_ctas, _ptr(self.attn_prof),
                                                 _ptr(getattr(batch, "tree_mask", None)), self._stream()), "attn_decode")
            if sp > 1:
                self.launches += 1
        if batch.item_seq is not None:
            n_items = batch.item_seq.numel()
            work = n_items * Hkv
            sp = splits if splits > 0 else (1 if work >= self._sm else max(1, min(8, tiles, self._sm // max(work, 1))))
            po = pm = None
            if sp > 1:
                n = work * sp * 128
                po = self._buf("attn_part_o2", n * D * 4).view(torch.float32)
                pm = self._buf("attn_part_ml2", n * 2 * 4).view(torch.float32)
            self._check(self.lib.blz_attn_tc(_ptr(q), _ptr(out), _ptr(kv.kv[layer_idx]), _ptr(kv.block_table),
                                             _ptr(batch.slots), _ptr(batch.q_start), _ptr(batch.ctx_len), _ptr(batch.item_seq),
                                             _ptr(batch.item_q0), n_items, Hq, Hkv, D, kv.block_table.stride(0), kv.kv[layer_idx].stride(0),
                                             kv.kv[layer_idx].stride(1), scale, 1.0,
                                             1.0, sp, _ptr(po), _ptr(pm), max_ctas, self._stream()), "attn_prefill")
            if sp > 1:
                self.launches += 1
        return out.view(T, Hq * D)

    # ------------------------------------------------------------------ head
    def argmax(self, logits, index_offset: int = 0, want_values: bool = False):
        R, V = logits.shape
        out = torch.empty(R, dtype=torch.int64, device=self.device)
        vals = torch.empty(R, dtype=torch.float32, device=self.device) if want_values else None
        self._check(self.lib.blz_argmax(_ptr(logits), _ptr(out), _ptr(vals), R, V, logits.stride(0), index_offset,
                                        self._stream()), "argmax")
        return (out, vals) if want_values else out

    # ------------------------------------------------------------------ mixture of experts
    def router_topk(self, logits, k, renorm=True, first: int = 0, local_n: int = -1):
        """Softmax → top-k → renormalise on the device; also counts the routed rows of each local expert."""
        T, E = logits.shape
        local_n = E if local_n < 0 else local_n
        w = torch.empty(T, k, dtype=torch.float32, device=self.device)
        ids = torch.empty(T, k, dtype=torch.int32, device=self.device)
        counts = torch.empty(max(local_n, 1), dtype=torch.int32, device=self.device)
        self._check(self.lib.blz_moe_route(_ptr(logits.contiguous()), _ptr(w), _ptr(ids), _ptr(counts), T, E, k, int(renorm),
                                           first, local_n, self._stream()), "moe_route")
        self._route_counts = (counts, first, local_n)
        return w, ids

    def pack_experts(self, ex):
        """Stack the local experts' weights into two grouped-GEMM operands (gate_up and down)."""
        if ex.cuda_pack is not None:
            return ex.cuda_pack

        def stack(lins):
            pk0 = self.pack(lins[0], tiled=False, exact_fp8=False)
            kind = pk0["kind"]
            w = torch.cat([self.pack(l, tiled=False, exact_fp8=False)["w"] for l in lins])
            alpha = torch.cat([self.pack(l, tiled=False, exact_fp8=False)["alpha"] for l in lins]) if pk0["alpha"] is not None else None
            sf = None
            if kind in (1, 2):
                l0 = lins[0]
                if l0.N % 128:
                    raise CudaError("grouped GEMM needs expert output dims that are multiples of 128")
                per = l0.K // (16 if kind == 1 else 32)
                if kind == 1:
                    raw = torch.cat([l.sf.to(self.device).view(torch.uint8) for l in lins])
                else:
                    raw = torch.cat([quant.unswizzle_sf_128x4(self.pack(l, tiled=False, exact_fp8=False)["sf"], (l.N + 255) // 256 * 256, per)[:l.N] for l in lins])
                rows = (raw.shape[0] + 255) // 256 * 256
                buf = torch.zeros(rows, per, dtype=torch.uint8, device=self.device)
                buf[:raw.shape[0]] = raw
                sf = quant.swizzle_sf_128x4(buf)
            for l in lins:
                l.cuda_pack = None          # the stacked copy replaces the per-expert ones
            return {"kind": kind, "w": w.contiguous(), "sf": sf, "alpha": alpha, "N": lins[0].N, "K": lins[0].K,
                    "fmt": lins[0].fmt, "act_quant": lins[0].act_quant}
        ex.cuda_pack = {"gate_up": stack(ex.gate_up), "down": stack(ex.down)}
        return ex.cuda_pack

    def _grouped_gemm(self, pk, a, M_pad, tile_expert, n_exp, out):
        kind = pk["kind"]
        if kind in (1, 2):
            data, sfa, rs = a.data, a.sf, a.row_scale
            lda = data.shape[1]
        else:
            data, sfa, rs = a, None, None
            lda = a.shape[1] * 2
        w = pk["w"]
        self._check(self.lib.blz_gemm_tc(kind, _ptr(data), lda, _ptr(w), w.shape[1] * w.element_size(), _ptr(out), out.stride(0),
                                         M_pad, pk["N"], pk["K"], _ptr(rs), _ptr(pk["alpha"]), VP(0), _ptr(sfa), _ptr(pk["sf"]),
                                         0, 128, 0, _ptr(tile_expert), n_exp, 0, 0, self._stream()), "grouped gemm")
        return out

    def moe(self, x, topk_w, topk_id, experts):
        """Routed experts held by this rank: scatter rows by expert → grouped gate_up GEMM → SwiGLU → grouped down GEMM →
        weighted combine.  ``x`` is bf16 ``[T, H]``.  Under expert parallelism the result is a partial sum."""
        pk = self.pack_experts(experts)
        gu, dn = pk["gate_up"], pk["down"]
        T, H = x.shape
        k = topk_id.shape[1]
        n_exp, first = experts.count, experts.first
        counts, cf, cn = getattr(self, "_route_counts", (None, -1, -1))
        if counts is None or cf != first or cn != n_exp:
            # routing was computed elsewhere: rebuild the histogram of local experts
            le = (topk_id.long() - first).flatten()
            ok = (le >= 0) & (le < n_exp)
            counts = torch.bincount(le[ok], minlength=n_exp).to(torch.int32)
        max_tiles = (T * k + 127) // 128 + n_exp
        M_pad = max_tiles * 128
        dev = self.device
        offsets = torch.empty(n_exp, dtype=torch.int32, device=dev)
        fill = torch.empty(n_exp, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=dev)
        tile_rows = torch.empty(max_tiles, dtype=torch.int32, device=dev)
        row_map = torch.empty(T, k, dtype=torch.int32, device=dev)
        self._check(self.lib.blz_moe_plan(_ptr(counts), _ptr(offsets), _ptr(fill), _ptr(tile_expert), _ptr(tile_rows), n_exp,
                                          max_tiles, self._stream()), "moe_plan")
        narrow = T * k <= self.MOE_NARROW_ROWS * n_exp and gu["kind"] in (0, 1, 2) and gu["N"] % 128 == 0 and dn["N"] % 128 == 0
        mode = 1 if (gu["fmt"] == Format.NVFP4 and gu["act_quant"]) else (2 if gu["kind"] == 2 else 0)
        if mode:
            proxy = Linear(gu["fmt"], gu["N"], gu["K"])
            proxy.act_quant = True
            xq = self.quantize_rows(x.contiguous(), proxy)
            a = self._alloc_qact(Format.NVFP4 if mode == 1 else Format.MXFP8, M_pad, H)
            self._check(self.lib.blz_moe_scatter(mode, _ptr(xq.data), _ptr(xq.sf), _ptr(xq.row_scale), _ptr(a.data), _ptr(a.sf),
                                                 _ptr(a.row_scale), _ptr(topk_id), _ptr(offsets), _ptr(fill), _ptr(row_map), T, H, k,
                                                 first, n_exp, self._stream()), "moe_scatter")
        else:
            a = torch.empty(M_pad, H, dtype=torch.bfloat16, device=dev)
            self._check(self.lib.blz_moe_scatter(0, _ptr(x.contiguous()), VP(0), VP(0), _ptr(a), VP(0), VP(0), _ptr(topk_id),
                                                 _ptr(offsets), _ptr(fill), _ptr(row_map), T, H, k, first, n_exp, self._stream()),
                        "moe_scatter")
        g = torch.empty(M_pad, gu["N"], dtype=torch.bfloat16, device=dev)
        proxy_d = Linear(dn["fmt"], dn["N"], dn["K"])
        proxy_d.act_quant = dn["act_quant"]
        y = torch.empty(M_pad, dn["N"], dtype=torch.bfloat16, device=dev)
        if narrow:
            self._moe_gemm(gu, a, max_tiles, tile_expert, tile_rows, n_exp, g)
            act = self._silu_mul_live(g, proxy_d if dn["kind"] in (1, 2) else None, row_map)
            self._moe_gemm(dn, act, max_tiles, tile_expert, tile_rows, n_exp, y)
        else:
            self._grouped_gemm(gu, a, M_pad, tile_expert, n_exp, g)
            # only the routed rows: the padded row space is up to (1 + experts * 128 / routed rows) times larger
            act = self._silu_mul_live(g, proxy_d if dn["kind"] in (1, 2) else None, row_map)
            self._grouped_gemm(dn, act, M_pad, tile_expert, n_exp, y)
        out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        self._check(self.lib.blz_moe_combine(_ptr(y), _ptr(topk_w.contiguous()), _ptr(row_map), _ptr(out), T, H, k, self._stream()),
                    "moe_combine")
        self._route_counts = None
        return out

    def _moe_gemm(self, pk, a, row_tiles, tile_expert, tile_rows, n_exp, out):
        """Expert GEMM over the padded row space with the features on the MMA lanes and only each tile's live rows on its columns."""
        kind = pk["kind"]
        if isinstance(a, QuantAct):
            data, sfa, rs = a.data, a.sf, a.row_scale
            lda = data.shape[1]
        else:
            data, sfa, rs = a, None, None
            lda = a.shape[1] * 2
        w = pk["w"]
        self._check(self.lib.blz_moe_gemm(kind, _ptr(data), lda, _ptr(w), w.shape[1] * w.element_size(), _ptr(out), out.stride(0),
                                          row_tiles, pk["N"], pk["K"], n_exp, _ptr(rs), _ptr(pk["alpha"]), _ptr(sfa), _ptr(pk["sf"]),
                                          _ptr(tile_expert), _ptr(tile_rows), 0, self._stream()), f"moe_gemm kind {kind}")

    def _silu_mul_live(self, gu, quant_for, row_list):
        """``silu_mul`` over the padded row space of the routed rows: only the rows named in ``row_list`` (-1 = none) are
        touched, one CTA each."""
        T, I2 = gu.shape
        I = I2 // 2
        n = row_list.numel()
        mode = self._qmode(quant_for)
        if mode == 0:
            out = torch.empty(T, I, dtype=torch.bfloat16, device=self.device)
            self._check(self.lib.blz_swiglu_live(_ptr(gu), _ptr(out), VP(0), VP(0), VP(0), n, I, 0, 0, _ptr(row_list), self._stream()),
                        "swiglu_live")
            return out
        qa = self._alloc_qact(Format.NVFP4 if mode == 1 else Format.MXFP8, T, I)
        self._check(self.lib.blz_swiglu_live(_ptr(gu), VP(0), _ptr(qa.data), _ptr(qa.sf), _ptr(qa.row_scale), n, I, mode, 0,
                                             _ptr(row_list), self._stream()), "swiglu_live_q")
        return qa

    # ------------------------------------------------------------------ Gated DeltaNet
    def gdn(self, mixed_qkv, z, b, a, gdn, model, batch, kv, layer_idx, state_only: bool = False):
        """Causal conv + SiLU → gated delta rule (gates computed in the kernel) → gated RMSNorm.  Sequences flagged in
        ``batch.gdn_defer`` leave their state untouched; ``state_only`` advances the states and returns nothing."""
        cfg = model.cfg
        dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        hk, hv = gdn.k_heads, gdn.v_heads
        T = mixed_qkv.shape[0]
        C = 2 * hk * dk + hv * dv
        B = batch.slots.numel()
        conv = torch.empty(T, C, dtype=torch.bfloat16, device=self.device)
        self._check(self.lib.blz_gdn_conv_runs(_ptr(mixed_qkv), mixed_qkv.stride(0), _ptr(conv), _ptr(kv.conv_state[layer_idx]),
                                               _ptr(gdn.conv_w), _ptr(batch.slots), _ptr(batch.q_start), _ptr(batch.ctx_len),
                                               _ptr(batch.gdn_defer), B, C, gdn.conv_w.shape[1], int(batch.max_q_len),
                                               self._stream()), "gdn_conv")
        o = None if state_only else torch.empty(T, hv, dv, dtype=torch.bfloat16, device=self.device)
        # long token runs (prompt chunks) go through the chunked tensor-core kernel, short ones (decode, verify, replay)
        # through the token-by-token kernel; both walk the same batch and each takes its own sequences
        chunked = (self.GDN_CHUNK_MIN > 0 and not state_only and dk == 128 and dv == 128 and batch.max_q_len >= self.GDN_CHUNK_MIN)
        n_chunks = T // 128 + B                    # upper bound of the sum over sequences of ceil(new tokens / 128)
        ws_bytes = int(self.lib.blz_gdn_chunk_ws_bytes(n_chunks, hv)) if chunked and self.GDN_SPLIT else 0
        if chunked and self.GDN_SPLIT and ws_bytes <= self.GDN_SPLIT_MAX_WS:
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=self.device)
            self._check(self.lib.blz_gdn_chunk_split(_ptr(conv), _ptr(a), _ptr(b), a.stride(0), _ptr(gdn.A_log), _ptr(gdn.dt_bias),
                                                     _ptr(kv.rec_state[layer_idx]), _ptr(o), _ptr(batch.slots), _ptr(batch.q_start),
                                                     _ptr(batch.ctx_len), _ptr(batch.gdn_defer), B, hk, hv, dk, dv, self.GDN_CHUNK_MIN,
                                                     int(batch.max_q_len), n_chunks, _ptr(ws), self._stream()), "gdn_chunk_split")
            self.launches += 1                     # two kernels behind the one call
        elif chunked:
            self._check(self.lib.blz_gdn_chunk(_ptr(conv), _ptr(a), _ptr(b), a.stride(0), _ptr(gdn.A_log), _ptr(gdn.dt_bias),
                                               _ptr(kv.rec_state[layer_idx]), _ptr(o), _ptr(batch.slots), _ptr(batch.q_start),
                                               _ptr(batch.ctx_len), _ptr(batch.gdn_defer), B, hk, hv, dk, dv, self.GDN_CHUNK_MIN,
                                               self._stream()), "gdn_chunk")
        if not chunked or batch.num_rows > batch.max_q_len or B > 1:
            self._check(self.lib.blz_gdn_recurrent_upto(_ptr(conv), _ptr(a), _ptr(b), a.stride(0), _ptr(gdn.A_log), _ptr(gdn.dt_bias),
                                                        _ptr(kv.rec_state[layer_idx]), _ptr(o), _ptr(batch.slots), _ptr(batch.q_start),
                                                        _ptr(batch.ctx_len), _ptr(batch.gdn_defer), B, hk, hv, dk, dv,
                                                        self.GDN_CHUNK_MIN - 1 if chunked else 0x7fffffff, self._stream()),
                        "gdn_recurrent")
        if state_only:
            return None
        y = torch.empty(T, hv * dv, dtype=torch.bfloat16, device=self.device)
        self._check(self.lib.blz_gated_rmsnorm(_ptr(o), _ptr(z), z.stride(0), _ptr(gdn.norm_w), _ptr(y), T, hv, dv,
                                               cfg.rms_norm_eps, 2 if cfg.gdn_output_gate == "sigmoid" else 0, self._stream()),
                    "gated_rmsnorm")
        return y
