"""Linear layers in every stored format, with tensor-parallel cuts and the GEMM router.

Counterpart of the reference's ``crates/blaze/src/linear.rs`` (``Cut`` :15, ``Store`` :23,
``Linear::load`` :237 which stacks modules sharing an input, ``run`` :535 which picks a kernel by
row count).  Here every format runs on one tcgen05 GEMM family (bf16, NVFP4 block-scaled,
MXFP8 block-scaled, FP8 with 128x128 scales); there is no dequantise-then-library path.
On CPU (and as the oracle) the layer multiplies by the dequantised weight in fp32 and, when the
format quantises activations, applies the same activation quantiser first so that both paths
compute the same function.
"""
from __future__ import annotations

import enum
from typing import List, Optional, Sequence

import torch

from . import quant
from .quant import Format


class Cut(enum.Enum):
    ALL = 0    # replicated
    ROWS = 1   # output features split (q/k/v, gate/up, vocab)
    COLS = 2   # input features split (o_proj, down_proj) → partial sums need a reduction


def part(n: int, rank: int, world: int):
    """Even contiguous range of ``n`` items for ``rank`` (``model.rs:39``)."""
    assert n % world == 0, f"{n} does not divide over {world} ranks"
    s = n // world
    return rank * s, (rank + 1) * s


class QuantAct:
    """A quantised activation matrix handed from a producer epilogue to the next GEMM."""
    __slots__ = ("fmt", "data", "sf", "row_scale", "rows", "cols", "dense", "wait")

    def __init__(self, fmt, data, sf, row_scale, rows, cols, dense=None):
        self.fmt, self.data, self.sf, self.row_scale = fmt, data, sf, row_scale
        self.rows, self.cols, self.dense = rows, cols, dense
        # (arrival counters ptr, expected-count ptr, world, timeout ms) while peers may still be writing this buffer: the first
        # GEMM that consumes it waits for the flags inside its producer warp
        self.wait = None


class Linear:
    """``y = x @ W^T`` with W ``[N, K]`` held in one of the storage formats."""

    def __init__(self, fmt: Format, N: int, K: int):
        self.fmt, self.N, self.K = fmt, N, K
        self.w: Optional[torch.Tensor] = None        # dense [N,K] | packed fp4 [N,K/2] | e4m3 [N,K]
        self.sf: Optional[torch.Tensor] = None       # block scales (logical layout)
        self.alpha: Optional[torch.Tensor] = None    # fp32 [N] per-output multiplier (global / channel scale)
        self.block = (128, 128)
        self.bias: Optional[torch.Tensor] = None
        self.act_quant = False                       # quantise activations to the weight's format (W4A4 / W8A8)
        self.cut = Cut.ALL
        self.cuda_pack = None                        # kernel-side layouts, built by ops.cuda on first use
        self.name = ""

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_dense(cls, w: torch.Tensor, fmt: Format = Format.DENSE, act_quant: Optional[bool] = None,
                   dtype: torch.dtype = torch.bfloat16, segments: Optional[Sequence[int]] = None,
                   four_over_six: bool = False) -> "Linear":
        """Quantise a dense weight.  ``segments`` = row counts of stacked modules that each get their
        own global scale (as separately quantised checkpoint modules would)."""
        N, K = w.shape
        lin = cls(fmt, N, K)
        segs = list(segments) if segments else [N]
        if fmt == Format.DENSE:
            lin.w = w.to(dtype).contiguous()
            lin.act_quant = False
        elif fmt == Format.NVFP4:
            ws, sfs, als = [], [], []
            r = 0
            for n in segs:
                p, sf, g = quant.nvfp4_quantize(w[r:r + n], four_over_six=four_over_six)
                ws.append(p); sfs.append(sf); als.append(g.reshape(1).expand(n))
                r += n
            lin.w, lin.sf, lin.alpha = torch.cat(ws), torch.cat(sfs), torch.cat(als).float().contiguous()
            lin.act_quant = True if act_quant is None else act_quant
        elif fmt == Format.MXFP8:
            lin.w, lin.sf = quant.mxfp8_quantize(w)
            lin.alpha = torch.ones(N, dtype=torch.float32, device=w.device)
            lin.act_quant = True if act_quant is None else act_quant
        elif fmt == Format.FP8_BLOCK:
            lin.w, lin.sf = quant.fp8_block_quantize(w, lin.block)
            lin.alpha = torch.ones(N, dtype=torch.float32, device=w.device)
            lin.act_quant = True if act_quant is None else act_quant
        elif fmt in (Format.FP8_CHANNEL, Format.FP8_TENSOR):
            q, s = quant.fp8_channel_quantize(w)
            lin.w, lin.alpha = q, s.squeeze(1).float().contiguous()
            lin.fmt = Format.FP8_CHANNEL
            lin.act_quant = True if act_quant is None else act_quant
        else:
            raise ValueError(fmt)
        return lin

    @classmethod
    def load(cls, ckpt, modules: Sequence[str], cut: Cut = Cut.ALL, rank: int = 0, world: int = 1,
             dtype: torch.dtype = torch.bfloat16, device="cpu", act_quant: Optional[bool] = None,
             row_groups: Optional[Sequence[Sequence[int]]] = None) -> "Linear":
        """Load and stack checkpoint modules that share an input (qkv, gate_up).

        ``row_groups[i]`` optionally gives, for module i, the unit (e.g. head_dim) so that ROWS cuts
        fall on unit boundaries; each module is cut on its own and the cuts are concatenated.
        """
        meta = ckpt.meta()
        fmts = {quant.resolve_format(meta, m) for m in modules}
        if len(fmts) != 1:
            raise ValueError(f"modules {modules} mix formats {fmts}")
        fmt = fmts.pop()
        parts = [cls._load_one(ckpt, m, fmt, cut, rank, world, dtype) for m in modules]
        lin = parts[0] if len(parts) == 1 else cls._stack(parts)
        lin.cut = cut
        lin.name = "+".join(modules)
        if act_quant is not None:
            lin.act_quant = act_quant and fmt != Format.DENSE
        return lin.to(device)

    @staticmethod
    def _rows(t: torch.Tensor, cut: Cut, rank: int, world: int, unit: int = 1) -> torch.Tensor:
        if cut != Cut.ROWS or world == 1:
            return t
        a, b = part(t.shape[0] // unit, rank, world)
        return t[a * unit:b * unit]

    @staticmethod
    def _cols(t: torch.Tensor, cut: Cut, rank: int, world: int, per: int = 1) -> torch.Tensor:
        """Slice the K axis; ``per`` = K elements per stored column (2 for packed fp4; 16/32/128 for scales)."""
        if cut != Cut.COLS or world == 1:
            return t
        a, b = part(t.shape[1], rank, world)
        return t[:, a:b]

    @classmethod
    def _load_one(cls, ckpt, m: str, fmt: Format, cut: Cut, rank: int, world: int, dtype) -> "Linear":
        def cutw(t):
            return cls._cols(cls._rows(t, cut, rank, world), cut, rank, world)

        if fmt == Format.DENSE:
            w = cutw(ckpt.get(f"{m}.weight")).to(dtype)
            lin = cls(fmt, w.shape[0], w.shape[1])
            lin.w = w.contiguous()
        elif fmt == Format.NVFP4:
            if f"{m}.weight_packed" in ckpt:   # compressed-tensors: dequant divides by the global scale
                packed = ckpt.get(f"{m}.weight_packed")
                g = 1.0 / ckpt.get(f"{m}.weight_global_scale").float().reshape(-1)[0]
            else:                               # ModelOpt: dequant multiplies by weight_scale_2
                packed = ckpt.get(f"{m}.weight")
                g = ckpt.get(f"{m}.weight_scale_2").float().reshape(-1)[0]
            sf = ckpt.get(f"{m}.weight_scale")
            if sf.dtype != torch.float8_e4m3fn:
                sf = sf.view(torch.float8_e4m3fn)
            packed, sf = cutw(packed.view(torch.uint8)), cutw(sf)
            lin = cls(fmt, packed.shape[0], packed.shape[1] * 2)
            lin.w, lin.sf = packed.contiguous(), sf.contiguous()
            lin.alpha = torch.full((lin.N,), float(g), dtype=torch.float32)
            lin.act_quant = True
            if f"{m}.input_global_scale" in ckpt or f"{m}.input_scale" in ckpt:
                pass  # static activation scales are ignored: activations are quantised per row at run time
        elif fmt == Format.MXFP8:
            q = cutw(ckpt.get(f"{m}.weight"))
            sname = f"{m}.weight_scale" if f"{m}.weight_scale" in ckpt else f"{m}.weight_scale_inv"
            sf = cutw(ckpt.get(sname).view(torch.uint8))
            lin = cls(fmt, q.shape[0], q.shape[1])
            lin.w, lin.sf = q.contiguous(), sf.contiguous()
            lin.alpha = torch.ones(lin.N, dtype=torch.float32)
            lin.act_quant = True
        elif fmt == Format.FP8_BLOCK:
            q = ckpt.get(f"{m}.weight")
            sname = f"{m}.weight_scale_inv" if f"{m}.weight_scale_inv" in ckpt else f"{m}.weight_scale"
            s = ckpt.get(sname).float()
            bn = -(-q.shape[0] // s.shape[0])
            bk = -(-q.shape[1] // s.shape[1])
            lin_block = (bn, bk)
            if cut == Cut.ROWS and world > 1:
                a, b = part(q.shape[0], rank, world)
                assert a % bn == 0, "FP8 block rows must cut on block boundaries"
                q, s = q[a:b], s[a // bn:-(-b // bn)]
            elif cut == Cut.COLS and world > 1:
                a, b = part(q.shape[1], rank, world)
                assert a % bk == 0, "FP8 block columns must cut on block boundaries"
                q, s = q[:, a:b], s[:, a // bk:-(-b // bk)]
            lin = cls(fmt, q.shape[0], q.shape[1])
            lin.block = lin_block
            lin.w, lin.sf = q.contiguous(), s.contiguous()
            lin.alpha = torch.ones(lin.N, dtype=torch.float32)
            lin.act_quant = True
        else:  # per-channel / per-tensor FP8
            q = ckpt.get(f"{m}.weight")
            sname = f"{m}.weight_scale" if f"{m}.weight_scale" in ckpt else f"{m}.weight_scale_inv"
            s = ckpt.get(sname).float().reshape(-1) if sname in ckpt else torch.ones(1)
            s = s.expand(q.shape[0]) if s.numel() == 1 else s
            if cut == Cut.ROWS and world > 1:
                a, b = part(q.shape[0], rank, world)
                q, s = q[a:b], s[a:b]
            q = cls._cols(q, cut, rank, world)
            lin = cls(Format.FP8_CHANNEL, q.shape[0], q.shape[1])
            lin.w, lin.alpha = q.contiguous(), s.float().contiguous()
            lin.act_quant = True
        b = ckpt.get_opt(f"{m}.bias")
        if b is not None:
            lin.bias = cls._rows(b, cut, rank, world).to(dtype)
        return lin

    @classmethod
    def _stack(cls, parts: List["Linear"]) -> "Linear":
        p0 = parts[0]
        lin = cls(p0.fmt, sum(p.N for p in parts), p0.K)
        lin.block, lin.act_quant = p0.block, p0.act_quant
        lin.w = torch.cat([p.w for p in parts])
        if p0.sf is not None:
            lin.sf = torch.cat([p.sf for p in parts])
        if p0.alpha is not None:
            lin.alpha = torch.cat([p.alpha for p in parts])
        if p0.bias is not None:
            lin.bias = torch.cat([p.bias for p in parts])
        return lin

    def to(self, device) -> "Linear":
        for a in ("w", "sf", "alpha", "bias"):
            t = getattr(self, a)
            if t is not None:
                setattr(self, a, t.to(device))
        return self

    @property
    def device(self):
        return self.w.device

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w, self.sf, self.alpha, self.bias) if t is not None)

    # ------------------------------------------------------------------ reference math
    def dequant(self) -> torch.Tensor:
        """fp32 ``[N, K]`` weight as the kernels see it."""
        if self.fmt == Format.DENSE:
            return self.w.float()
        if self.fmt == Format.NVFP4:
            return quant.nvfp4_dequantize(self.w, self.sf, self.alpha)
        if self.fmt == Format.MXFP8:
            return quant.mxfp8_dequantize(self.w, self.sf) * self.alpha.unsqueeze(1)
        if self.fmt == Format.FP8_BLOCK:
            return quant.fp8_block_dequantize(self.w, self.sf, self.block) * self.alpha.unsqueeze(1)
        return self.w.float() * self.alpha.unsqueeze(1)

    def quant_act_ref(self, x: torch.Tensor) -> torch.Tensor:
        """Apply (quantise → dequantise) of this layer's activation format to ``x`` in fp32."""
        if not self.act_quant:
            return x.float()
        x2 = x.reshape(-1, x.shape[-1])
        if self.fmt == Format.NVFP4:
            p, sf, g = quant.nvfp4_quantize(x2, per_row=True)
            return quant.nvfp4_dequantize(p, sf, g).view(x.shape)
        if self.fmt == Format.MXFP8:
            q, e = quant.mxfp8_quantize(x2)
            return quant.mxfp8_dequantize(q, e).view(x.shape)
        if self.fmt == Format.FP8_BLOCK:
            # 1 x 128 activation groups
            bk = self.block[1]
            K = x2.shape[1]
            pad = (-K) % bk
            xp = torch.nn.functional.pad(x2.float(), (0, pad)).view(x2.shape[0], -1, bk)
            s = (xp.abs().amax(-1, keepdim=True) / quant.FP8_MAX).clamp_min(1e-12)
            d = (quant.to_e4m3(xp / s).float() * s).view(x2.shape[0], -1)[:, :K]
            return d.view(x.shape)
        q, s = quant.fp8_rowwise_quantize(x2)
        return (q.float() * s.unsqueeze(1)).view(x.shape)

    def ref(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        xd = x.dense if isinstance(x, QuantAct) else x
        y = self.quant_act_ref(xd) @ self.dequant().t()
        if self.bias is not None:
            y = y + self.bias.float()
        return y.to(out_dtype or xd.dtype)

    def __call__(self, x, ops=None, **kw):
        if ops is None or not ops.is_cuda:
            return self.ref(x, **{k: v for k, v in kw.items() if k == "out_dtype"})
        return ops.linear(self, x, **kw)
