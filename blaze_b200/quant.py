"""Weight/activation number formats: detection from a checkpoint and torch reference (de)quantisers.

The format resolver mirrors what the reference accepts (``crates/blaze/src/quant.rs:22-226``):
compressed-tensors NVFP4 (``weight_packed`` + ``weight_scale`` + ``weight_global_scale``), ModelOpt
NVFP4 (U8 ``weight`` + ``weight_scale`` + ``weight_scale_2``), MXFP8 (E4M3 + E8M0 per 32), FP8
with 2-D block scales, FP8 per-channel / per-tensor, and dense 16/32-bit.

The reference quantisers here are the oracle for the CUDA quantise kernels and GEMM tests.
NVFP4 follows ``kernels/include/blaze/nvfp4.h:1-100``: 16-element blocks, E2M1 codes with the
even element in the low nibble, E4M3 block scale, fp32 global scale, optional "four-over-six"
block-scale search.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
FP8_MAX = 448.0
FP4_MAX = 6.0
NVFP4_BLOCK = 16
MXFP8_BLOCK = 32


class Format(enum.Enum):
    DENSE = "dense"            # bf16 / f16 / f32
    NVFP4 = "nvfp4"
    MXFP8 = "mxfp8"
    FP8_BLOCK = "fp8_block"    # 2-D block scale (usually 128x128)
    FP8_CHANNEL = "fp8_channel"
    FP8_TENSOR = "fp8_tensor"


class ActQuant(enum.Enum):
    NONE = "none"       # activations stay 16-bit
    DYNAMIC = "dynamic"  # quantise per row at run time
    STATIC = "static"


@dataclass
class QuantConfig:
    """What ``quantization_config`` / ``hf_quant_config.json`` says (may be empty)."""
    method: str = ""                    # "compressed-tensors" | "modelopt" | "fp8" | ""
    default_format: Optional[Format] = None
    block_size: Tuple[int, int] = (128, 128)
    act: ActQuant = ActQuant.NONE
    ignore: Tuple[str, ...] = ()

    @classmethod
    def from_model_config(cls, qc: Optional[Dict[str, Any]]) -> "QuantConfig":
        if not qc:
            return cls()
        if "hf_quant_config" in qc:  # ModelOpt sidecar file
            q = qc["hf_quant_config"].get("quantization", {})
            algo = str(q.get("quant_algo", "")).upper()
            fmt = Format.NVFP4 if "NVFP4" in algo else Format.FP8_TENSOR if "FP8" in algo else None
            return cls(method="modelopt", default_format=fmt, act=ActQuant.DYNAMIC,
                       ignore=tuple(q.get("exclude_modules", []) or []))
        method = str(qc.get("quant_method", "")).lower()
        if "quant_algo" in qc or method == "modelopt":
            algo = str(qc.get("quant_algo", "")).upper()
            fmt = Format.NVFP4 if "NVFP4" in algo else Format.FP8_TENSOR if "FP8" in algo else None
            return cls(method="modelopt", default_format=fmt, act=ActQuant.DYNAMIC,
                       ignore=tuple(qc.get("ignore", qc.get("exclude_modules", [])) or []))
        if method == "compressed-tensors":
            fmt = None
            act = ActQuant.NONE
            for grp in (qc.get("config_groups") or {}).values():
                w = grp.get("weights") or {}
                bits, typ = w.get("num_bits"), w.get("type")
                if bits == 4 and typ == "float":
                    fmt = Format.NVFP4
                elif bits == 8 and typ == "float":
                    strat = w.get("strategy", "tensor")
                    fmt = {"block": Format.FP8_BLOCK, "channel": Format.FP8_CHANNEL}.get(strat, Format.FP8_TENSOR)
                    if w.get("block_structure"):
                        bs = w["block_structure"]
                if grp.get("input_activations"):
                    act = ActQuant.DYNAMIC if grp["input_activations"].get("dynamic", True) else ActQuant.STATIC
            return cls(method=method, default_format=fmt, act=act, ignore=tuple(qc.get("ignore", []) or []))
        if method in ("fp8", "mxfp8"):
            bs = qc.get("weight_block_size")
            if method == "mxfp8":
                return cls(method=method, default_format=Format.MXFP8)
            if bs:
                return cls(method=method, default_format=Format.FP8_BLOCK, block_size=(int(bs[0]), int(bs[1])),
                           act=ActQuant.DYNAMIC)
            return cls(method=method, default_format=Format.FP8_TENSOR, act=ActQuant.DYNAMIC)
        return cls(method=method)


def resolve_format(names: Dict[str, Tuple[str, Tuple[int, ...]]], module: str) -> Format:
    """Decide a linear module's format from the tensors present in the checkpoint.

    ``names`` maps tensor name → (dtype string, shape).  Rules as in ``quant.rs:171-226``.
    """
    def has(s):
        return f"{module}.{s}" in names

    if has("weight_packed") and has("weight_global_scale"):
        return Format.NVFP4
    if has("weight") and has("weight_scale_2"):
        return Format.NVFP4
    if has("weight"):
        dt, shape = names[f"{module}.weight"]
        if dt in ("F8_E4M3", "float8_e4m3fn"):
            for sname in ("weight_scale", "weight_scale_inv"):
                if has(sname):
                    sdt, sshape = names[f"{module}.{sname}"]
                    if sdt in ("U8", "uint8", "F8_E8M0", "float8_e8m0fnu"):
                        return Format.MXFP8
                    # a block-scale grid is [ceil(N / bn), ceil(K / bk)]: more than one column, or fewer rows than the weight
                    # has (a per-channel scale is [N] or [N, 1]); a module of one block row still has its columns
                    if len(sshape) == 2 and (sshape[1] > 1 or 1 < sshape[0] < shape[0]):
                        return Format.FP8_BLOCK
                    if len(sshape) >= 1 and max(sshape) > 1:
                        return Format.FP8_CHANNEL
                    return Format.FP8_TENSOR
            return Format.FP8_TENSOR
        return Format.DENSE
    raise KeyError(f"no weight tensors for module {module}")


# ------------------------------------------------------------------------------- E2M1 helpers
def _e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    """Round fp32 values (already divided by their scale) to E2M1 codes 0..15 (sign in bit 3).

    Round-to-nearest, ties to even code, saturating at ±6.
    """
    a = x.abs().clamp_(max=FP4_MAX)
    # decision thresholds between grid points with ties-to-even (even mantissa code)
    # grid: 0, .5, 1, 1.5, 2, 3, 4, 6 ; midpoints .25 .75 1.25 1.75 2.5 3.5 5
    code = torch.zeros_like(a, dtype=torch.int32)
    code += (a > 0.25).int()      # 0 | 0.5   tie .25 -> 0 (even)
    code += (a >= 0.75).int()     # 0.5 | 1   tie .75 -> 1.0 (code 2, even)
    code += (a > 1.25).int()      # 1 | 1.5   tie -> 1.0 (code 2)
    code += (a >= 1.75).int()     # 1.5 | 2   tie -> 2.0 (code 4)
    code += (a > 2.5).int()       # 2 | 3     tie -> 2.0 (code 4)
    code += (a >= 3.5).int()      # 3 | 4     tie -> 4.0 (code 6)
    code += (a > 5.0).int()       # 4 | 6     tie -> 4.0 (code 6)
    sign = (x < 0) | ((x == 0) & (torch.signbit(x)))
    return (code | (sign.int() << 3)).to(torch.uint8)


def _e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    lut = torch.tensor(E2M1_VALUES + tuple(-v for v in E2M1_VALUES), dtype=torch.float32, device=codes.device)
    return lut[codes.long()]


def pack_fp4(codes: torch.Tensor) -> torch.Tensor:
    """[..., K] codes → [..., K/2] bytes; even element in the low nibble."""
    lo, hi = codes[..., 0::2], codes[..., 1::2]
    return (lo | (hi << 4)).to(torch.uint8)


def unpack_fp4(packed: torch.Tensor) -> torch.Tensor:
    lo, hi = packed & 0xF, packed >> 4
    return torch.stack([lo, hi], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def to_e4m3(x: torch.Tensor) -> torch.Tensor:
    return x.clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)


# ------------------------------------------------------------------------------- NVFP4
def nvfp4_quantize(x: torch.Tensor, global_scale: Optional[torch.Tensor] = None, per_row: bool = False,
                   four_over_six: bool = False):
    """Quantise ``x [rows, K]`` (K % 16 == 0) to NVFP4.

    Returns ``(packed uint8 [rows, K/2], block_scale float8_e4m3fn [rows, K/16], global fp32)``.
    ``global`` is a scalar tensor, or ``[rows]`` with ``per_row=True`` (dynamic activation
    quantisation as in ``kernels/src/cuda/nvfp4_gemm.cu:33``).  Dequantised value =
    e2m1 * block_scale * global.
    """
    xf = x.float()
    rows, K = xf.shape
    assert K % NVFP4_BLOCK == 0
    if global_scale is None:
        amax = xf.abs().amax(dim=1) if per_row else xf.abs().amax()
        global_scale = (amax / (FP4_MAX * FP8_MAX)).clamp_min(1e-30)
    g = global_scale.float()
    gb = g.view(-1, 1, 1) if g.dim() == 1 else g
    xb = xf.view(rows, K // NVFP4_BLOCK, NVFP4_BLOCK)
    bmax = xb.abs().amax(dim=2, keepdim=True)

    def attempt(divisor):
        sf = to_e4m3(bmax / divisor / gb)
        sff = sf.float()
        denom = (sff * gb)
        q = torch.where(denom > 0, xb / denom.clamp_min(1e-30), torch.zeros_like(xb))
        codes = _e2m1_codes(q)
        deq = _e2m1_decode(codes) * denom
        err = ((deq - xb) ** 2).sum(dim=2, keepdim=True)
        return sf, codes, err

    sf, codes, err = attempt(FP4_MAX)
    if four_over_six:
        sf4, codes4, err4 = attempt(4.0)
        better = err4 < err
        sf = torch.where(better, sf4.float(), sf.float()).to(torch.float8_e4m3fn)
        codes = torch.where(better, codes4, codes)
    packed = pack_fp4(codes.view(rows, K))
    return packed, sf.view(rows, K // NVFP4_BLOCK), g


def nvfp4_dequantize(packed: torch.Tensor, block_scale: torch.Tensor, global_scale: torch.Tensor) -> torch.Tensor:
    rows = packed.shape[0]
    vals = _e2m1_decode(unpack_fp4(packed)).view(rows, -1, NVFP4_BLOCK)
    g = global_scale.float()
    g = g.view(-1, 1, 1) if g.dim() == 1 else g
    return (vals * block_scale.float().unsqueeze(-1) * g).view(rows, -1)


def nvfp4_kv_quantize(x: torch.Tensor, g: float = 1.0, search: bool = False) -> torch.Tensor:
    """Rows of a KV cache in NVFP4: ``x [..., D]`` (D % 16 == 0) -> uint8 ``[..., D/2 + D/16]``, the packed E2M1 codes of a row
    followed by its E4M3 block scales (one per 16 elements); value = e2m1 * scale * g.

    The block scale is the E4M3 rounding of ``amax / (6 g)``.  With ``search`` ("four over six") the candidates are that
    scale, the rounding of ``amax / (4 g)``, and the E4M3 codes -1 .. +5 steps from the first; the one with the lowest
    squared error of the block is kept, earlier candidates winning ties (reference: ``kv_store_kernel``,
    kernels/src/cuda/nvfp4_kv.cu:62-113, ``kScaleSearchFirst`` / ``Last`` in kernels/include/blaze/nvfp4.h:28)."""
    D = x.shape[-1]
    assert D % NVFP4_BLOCK == 0
    xb = x.float().reshape(-1, D // NVFP4_BLOCK, NVFP4_BLOCK)
    amax = xb.abs().amax(dim=2)

    def code_of(v):
        return v.clamp(max=FP8_MAX).to(torch.float8_e4m3fn).view(torch.uint8).to(torch.int32)

    def attempt(code):
        t = code.clamp(0, 0x7E).to(torch.uint8).view(torch.float8_e4m3fn).float() * g          # [rows, blocks]
        inv = torch.where(t > 0, 1.0 / t.clamp_min(1e-30), torch.zeros_like(t))
        codes = _e2m1_codes(xb * inv[..., None])
        err = ((_e2m1_decode(codes) * t[..., None] - xb) ** 2).sum(dim=2)
        return codes, err

    lo = code_of(amax / (6.0 * g))
    best_code = lo.clone()
    best, best_err = attempt(lo)
    if search:
        cands = [code_of(amax / (4.0 * g))] + [lo + s for s in range(-1, 6) if s != 0]
        for c in cands:
            valid = (c >= 0) & (c <= 0x7E)
            codes, err = attempt(c)
            take = valid & (err < best_err)
            best = torch.where(take[..., None], codes, best)
            best_err = torch.where(take, err, best_err)
            best_code = torch.where(take, c, best_code)
    packed = pack_fp4(best.reshape(-1, D))
    out = torch.cat([packed, best_code.to(torch.uint8)], dim=1)
    return out.reshape(*x.shape[:-1], D // 2 + D // NVFP4_BLOCK)


def nvfp4_kv_dequantize(rows: torch.Tensor, D: int, g: float = 1.0) -> torch.Tensor:
    """Inverse of :func:`nvfp4_kv_quantize`: uint8 ``[..., D/2 + D/16]`` -> fp32 ``[..., D]``."""
    flat = rows.reshape(-1, rows.shape[-1])
    vals = _e2m1_decode(unpack_fp4(flat[:, :D // 2])).view(flat.shape[0], D // NVFP4_BLOCK, NVFP4_BLOCK)
    sc = flat[:, D // 2:].contiguous().view(torch.float8_e4m3fn).float() * g
    return (vals * sc[..., None]).reshape(*rows.shape[:-1], D)


# ------------------------------------------------------------------------------- MXFP8
def mxfp8_quantize(x: torch.Tensor):
    """``x [rows, K]`` → (e4m3 [rows, K], e8m0 exponent bytes uint8 [rows, K/32])."""
    xf = x.float()
    rows, K = xf.shape
    assert K % MXFP8_BLOCK == 0
    xb = xf.view(rows, K // MXFP8_BLOCK, MXFP8_BLOCK)
    bmax = xb.abs().amax(dim=2, keepdim=True).clamp_min(2.0 ** -127)
    exp = torch.ceil(torch.log2(bmax / FP8_MAX)).clamp(-127, 127)
    scale = torch.exp2(exp)
    q = to_e4m3(xb / scale).view(rows, K)
    e8 = (exp + 127).to(torch.uint8).view(rows, K // MXFP8_BLOCK)
    return q, e8


def mxfp8_dequantize(q: torch.Tensor, e8: torch.Tensor) -> torch.Tensor:
    rows, K = q.shape
    scale = torch.exp2(e8.float() - 127.0).unsqueeze(-1)
    return (q.float().view(rows, -1, MXFP8_BLOCK) * scale).view(rows, K)


# ------------------------------------------------------------------------------- FP8 block / channel
def fp8_block_quantize(w: torch.Tensor, block: Tuple[int, int] = (128, 128)):
    """``w [N, K]`` → (e4m3 [N, K], fp32 dequant scale [ceil(N/bn), ceil(K/bk)])."""
    wf = w.float()
    N, K = wf.shape
    bn, bk = block
    nb, kb = (N + bn - 1) // bn, (K + bk - 1) // bk
    pad = torch.zeros(nb * bn, kb * bk, dtype=torch.float32, device=w.device)
    pad[:N, :K] = wf
    blocks = pad.view(nb, bn, kb, bk)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = to_e4m3(blocks / scale.view(nb, 1, kb, 1)).view(nb * bn, kb * bk)[:N, :K].contiguous()
    return q, scale


def fp8_block_dequantize(q: torch.Tensor, scale: torch.Tensor, block: Tuple[int, int] = (128, 128)) -> torch.Tensor:
    N, K = q.shape
    bn, bk = block
    s = scale.float().repeat_interleave(bn, dim=0)[:N].repeat_interleave(bk, dim=1)[:, :K]
    return q.float() * s


def fp8_channel_quantize(w: torch.Tensor):
    wf = w.float()
    scale = (wf.abs().amax(dim=1, keepdim=True) / FP8_MAX).clamp_min(1e-12)
    return to_e4m3(wf / scale), scale


def fp8_rowwise_quantize(x: torch.Tensor):
    """Dynamic per-row activation quantisation to e4m3."""
    xf = x.float()
    scale = (xf.abs().amax(dim=1, keepdim=True) / FP8_MAX).clamp_min(1e-12)
    return to_e4m3(xf / scale), scale.squeeze(1)


# ------------------------------------------------------------------------------- scale-factor swizzle
def swizzle_sf_128x4(sf: torch.Tensor) -> torch.Tensor:
    """Re-order a ``[rows, cols]`` 1-byte scale-factor matrix into 128×4 tiles of 512 bytes.

    Inside a tile, the byte of (row r, column c) sits at ``(r % 32) * 16 + (r // 32) * 4 + c``.
    This is the layout the tcgen05 block-scaled MMA reads scale factors in after a
    ``tcgen05.cp 32x128b.warpx4`` copy into tensor memory; tiles are ordered row-tile major.
    Rows are padded to a multiple of 128 and columns to a multiple of 4 with zeros.
    """
    rows, cols = sf.shape
    R, C = (rows + 127) // 128 * 128, (cols + 3) // 4 * 4
    buf = torch.zeros(R, C, dtype=torch.uint8, device=sf.device)
    buf[:rows, :cols] = sf.view(torch.uint8)
    t = buf.view(R // 128, 4, 32, C // 4, 4)          # [rt, r//32, r%32, ct, c]
    return t.permute(0, 3, 2, 1, 4).contiguous().view(-1)  # [rt, ct, r%32, r//32, c]


def unswizzle_sf_128x4(flat: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    R, C = (rows + 127) // 128 * 128, (cols + 3) // 4 * 4
    t = flat.view(R // 128, C // 4, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(R, C)
    return t[:rows, :cols].contiguous()
