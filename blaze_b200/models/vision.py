"""Vision tower: image preprocessing, the ViT encoder (CUDA path and CPU path) and the patch merger.

The encoder is a pre-LayerNorm ViT with 2-D rotary attention inside each image and a tanh-GELU MLP; a merger joins
``merge x merge`` neighbouring patch tokens into one language-model embedding.  On a GPU the four projections of each
block run on the bf16 tcgen05 GEMM (bias in the epilogue) and the rest on ``csrc/kernels/vision.cu``; on the CPU the
same math runs in fp32 torch, and the C++ tower of the host runtime (``blz_vit_forward_cpu``) is the oracle for both.

Reference: ``crates/blaze/src/vision.rs`` (``VisionConfig::load`` :39, smart resize :250-299, bicubic resize :352,
``preprocess`` :410, GPU tower ``encode_batch`` :611, CPU tower :747-793) and ``kernels/src/cuda/vision.cu``.
"""
from __future__ import annotations

import ctypes
import json
import math
import os
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..linear import Linear
from ..quant import Format

VP = ctypes.c_void_p
IMAGE_MEAN = (0.48145466, 0.4578275, 0.40821073)
IMAGE_STD = (0.26862954, 0.26130258, 0.27577711)


@dataclass
class VisionConfig:
    hidden_size: int = 1152
    num_heads: int = 16
    intermediate_size: int = 4304
    depth: int = 27
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    in_channels: int = 3
    out_hidden_size: int = 4096
    num_position_embeddings: int = 2304          # side² of the learned position grid
    eps: float = 1e-6
    min_pixels: int = 56 * 56
    max_pixels: int = 1280 * 28 * 28

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @classmethod
    def load(cls, model_dir: str) -> Optional["VisionConfig"]:
        with open(os.path.join(model_dir, "config.json")) as f:
            raw = json.load(f)
        v = raw.get("vision_config")
        if not v:
            return None
        c = cls()
        for key, name in (("hidden_size", "hidden_size"), ("num_heads", "num_heads"), ("intermediate_size", "intermediate_size"),
                          ("depth", "depth"), ("patch_size", "patch_size"), ("temporal_patch_size", "temporal_patch_size"),
                          ("spatial_merge_size", "spatial_merge_size"), ("in_channels", "in_channels"),
                          ("out_hidden_size", "out_hidden_size"), ("num_position_embeddings", "num_position_embeddings")):
            if key in v:
                setattr(c, name, int(v[key]))
        return c


# ------------------------------------------------------------------------------------------ preprocessing
def smart_resize(height: int, width: int, factor: int, min_pixels: int, max_pixels: int) -> Tuple[int, int]:
    """Round both sides to multiples of ``factor`` while keeping the pixel count inside [min, max] and the aspect ratio
    close (``vision.rs:250-299``)."""
    if min(height, width) <= 0:
        raise ValueError("empty image")
    if max(height, width) / min(height, width) > 200:
        raise ValueError("aspect ratio above 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def preprocess(image: torch.Tensor, cfg: VisionConfig) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
    """``image``: uint8 or float ``[H, W, 3]`` (RGB).  Returns patches ``[T, patch_dim]`` fp32 in merge-block order
    (the ``merge x merge`` patches of one output token are consecutive) and the grid ``(t, h, w)`` in patches."""
    x = image.float()
    if image.dtype == torch.uint8:
        x = x / 255.0
    H, W, C = x.shape
    f = cfg.patch_size * cfg.spatial_merge_size
    nh, nw = smart_resize(H, W, f, cfg.min_pixels, cfg.max_pixels)
    x = x.permute(2, 0, 1).unsqueeze(0)
    if (nh, nw) != (H, W):
        x = F.interpolate(x, size=(nh, nw), mode="bicubic", align_corners=False, antialias=True).clamp(0.0, 1.0)
    mean = torch.tensor(IMAGE_MEAN).view(1, 3, 1, 1)
    std = torch.tensor(IMAGE_STD).view(1, 3, 1, 1)
    x = (x - mean) / std
    x = x.repeat(cfg.temporal_patch_size, 1, 1, 1)                      # a still image fills the temporal patch
    p, m = cfg.patch_size, cfg.spatial_merge_size
    gh, gw = nh // p, nw // p
    # [tp, C, gh/m, m, p, gw/m, m, p] -> [gh/m, gw/m, m, m, C, tp, p, p]
    x = x.view(cfg.temporal_patch_size, C, gh // m, m, p, gw // m, m, p).permute(2, 5, 3, 6, 1, 0, 4, 7).contiguous()
    return x.view(gh * gw, cfg.patch_dim), (1, gh, gw)


def rope_tables(grid: Tuple[int, int, int], cfg: VisionConfig) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin ``[T, head_dim/2]`` for the merge-block token order: the first half of the pairs rotates with the row
    index, the second half with the column index (theta 10000)."""
    t, gh, gw = grid
    m = cfg.spatial_merge_size
    hh = torch.arange(gh).view(gh // m, 1, m, 1).expand(gh // m, gw // m, m, m).reshape(-1)
    ww = torch.arange(gw).view(1, gw // m, 1, m).expand(gh // m, gw // m, m, m).reshape(-1)
    quarter = cfg.head_dim // 4
    inv = 1.0 / (10000.0 ** (torch.arange(quarter, dtype=torch.float32) / quarter))
    ang = torch.cat([hh.float()[:, None] * inv[None], ww.float()[:, None] * inv[None]], dim=1)   # [T, head_dim/2]
    ang = ang.repeat(t, 1)
    return ang.cos().contiguous(), ang.sin().contiguous()


# ------------------------------------------------------------------------------------------ the tower
class Block:
    __slots__ = ("ln1_w", "ln1_b", "qkv", "proj", "ln2_w", "ln2_b", "fc1", "fc2")


class VisionTower:
    def __init__(self, cfg: VisionConfig, device, dtype=torch.bfloat16):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.blocks: List[Block] = []
        self.patch: Optional[Linear] = None
        self.pos: Optional[torch.Tensor] = None            # [side*side, hidden] learned grid
        self.merge_ln_w = self.merge_ln_b = None
        self.merge_fc1: Optional[Linear] = None
        self.merge_fc2: Optional[Linear] = None
        self._ops = None
        self._lib = None

    # -------------------------------------------------------------- construction
    @classmethod
    def random_init(cls, cfg: VisionConfig, device, dtype=torch.bfloat16, seed: int = 0) -> "VisionTower":
        g = torch.Generator().manual_seed(seed)
        vt = cls(cfg, device, dtype)

        def lin(n, k, scale=None):
            w = torch.randn(n, k, generator=g) * (scale or 1.0 / math.sqrt(k))
            l = Linear.from_dense(w.to(vt.device), Format.DENSE, dtype=dtype)
            l.bias = (torch.randn(n, generator=g) * 0.02).to(vt.device, dtype)
            return l

        def vec(n, base):
            return (base + 0.05 * torch.randn(n, generator=g)).to(vt.device, dtype)

        H = cfg.hidden_size
        vt.patch = lin(H, cfg.patch_dim)
        vt.pos = (torch.randn(cfg.num_position_embeddings, H, generator=g) * 0.02).to(vt.device, dtype)
        for _ in range(cfg.depth):
            b = Block()
            b.ln1_w, b.ln1_b, b.ln2_w, b.ln2_b = vec(H, 1.0), vec(H, 0.0), vec(H, 1.0), vec(H, 0.0)
            b.qkv, b.proj, b.fc1, b.fc2 = lin(3 * H, H), lin(H, H), lin(cfg.intermediate_size, H), lin(H, cfg.intermediate_size)
            vt.blocks.append(b)
        mm = H * cfg.spatial_merge_size ** 2
        vt.merge_ln_w, vt.merge_ln_b = vec(H, 1.0), vec(H, 0.0)
        vt.merge_fc1, vt.merge_fc2 = lin(mm, mm), lin(cfg.out_hidden_size, mm)
        return vt

    @classmethod
    def load(cls, model_dir: str, device, dtype=torch.bfloat16) -> Optional["VisionTower"]:
        """Load ``visual.*`` tensors of a Qwen-VL style checkpoint (``vision.rs:550``)."""
        cfg = VisionConfig.load(model_dir)
        if cfg is None:
            return None
        from ..weights import Checkpoint
        ck = Checkpoint.open(model_dir)
        pre = "model.visual." if "model.visual.patch_embed.proj.weight" in ck else "visual."
        vt = cls(cfg, device, dtype)

        def lin(name):
            l = Linear.from_dense(ck.get(pre + name + ".weight").float().reshape(ck.get(pre + name + ".weight").shape[0], -1).to(vt.device),
                                  Format.DENSE, dtype=dtype)
            if (pre + name + ".bias") in ck:
                l.bias = ck.get(pre + name + ".bias").to(vt.device, dtype)
            return l

        def vec(name):
            return ck.get(pre + name).to(vt.device, dtype) if (pre + name) in ck else None

        vt.patch = lin("patch_embed.proj")
        vt.pos = vec("pos_embed.weight")
        for i in range(cfg.depth):
            p = f"blocks.{i}."
            b = Block()
            b.ln1_w, b.ln1_b, b.ln2_w, b.ln2_b = vec(p + "norm1.weight"), vec(p + "norm1.bias"), vec(p + "norm2.weight"), vec(p + "norm2.bias")
            b.qkv, b.proj = lin(p + "attn.qkv"), lin(p + "attn.proj")
            b.fc1, b.fc2 = lin(p + "mlp.linear_fc1"), lin(p + "mlp.linear_fc2")
            vt.blocks.append(b)
        vt.merge_ln_w, vt.merge_ln_b = vec("merger.norm.weight"), vec("merger.norm.bias")
        vt.merge_fc1, vt.merge_fc2 = lin("merger.linear_fc1"), lin("merger.linear_fc2")
        return vt

    # -------------------------------------------------------------- pieces
    def _cuda(self) -> bool:
        if self.device.type != "cuda":
            return False
        if self._ops is None:
            from ..ops import get_ops
            self._ops = get_ops(self.device)
            lib = self._ops.lib
            lib.blz_vit_layernorm.argtypes = [VP, VP, VP, VP, ctypes.c_int, ctypes.c_int, ctypes.c_float, VP]
            lib.blz_vit_gelu.argtypes = [VP, ctypes.c_longlong, VP]
            lib.blz_vit_rope.argtypes = [VP, VP, VP, ctypes.c_int, ctypes.c_int, ctypes.c_int, VP]
            lib.blz_vit_attention.argtypes = [VP, VP, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, VP]
            self._lib = lib
        return self._ops.is_cuda

    def _stream(self):
        return VP(torch.cuda.current_stream(self.device).cuda_stream)

    def _check(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed: cuda error {rc}")
        self._ops.launches += 1

    def _linear(self, lin: Linear, x: torch.Tensor) -> torch.Tensor:
        if self._cuda():
            return self._ops.linear(lin, x.contiguous())
        y = x.float() @ lin.w.float().t()
        return (y + lin.bias.float()).to(x.dtype) if lin.bias is not None else y.to(x.dtype)

    def _layernorm(self, x, w, b):
        if self._cuda():
            y = torch.empty_like(x)
            self._check(self._lib.blz_vit_layernorm(VP(x.data_ptr()), VP(w.data_ptr()), VP(b.data_ptr() if b is not None else 0),
                                                    VP(y.data_ptr()), x.shape[0], x.shape[1], self.cfg.eps, self._stream()), "vit_layernorm")
            return y
        return F.layer_norm(x.float(), (x.shape[1],), w.float(), b.float() if b is not None else None, self.cfg.eps).to(x.dtype)

    def _gelu(self, x):
        if self._cuda():
            self._check(self._lib.blz_vit_gelu(VP(x.data_ptr()), x.numel(), self._stream()), "vit_gelu")
            return x
        return F.gelu(x.float(), approximate="tanh").to(x.dtype)

    def _attention(self, qkv: torch.Tensor, cos, sin, segments: Sequence[Tuple[int, int]]) -> torch.Tensor:
        T, H3 = qkv.shape
        H, NH = H3 // 3, self.cfg.num_heads
        D = H // NH
        if self._cuda():
            qkv = qkv.contiguous()
            out = torch.empty(T, H, dtype=qkv.dtype, device=qkv.device)
            self._check(self._lib.blz_vit_rope(VP(qkv.data_ptr()), VP(cos.data_ptr()), VP(sin.data_ptr()), T, H, NH, self._stream()), "vit_rope")
            for t0, t1 in segments:
                self._check(self._lib.blz_vit_attention(VP(qkv.data_ptr()), VP(out.data_ptr()), t0, t1, H, NH, self._stream()), "vit_attention")
            return out
        q, k, v = qkv.float().view(T, 3, NH, D).unbind(1)
        half = D // 2

        def rot(x):
            a, b = x[..., :half], x[..., half:]
            c, s = cos[:, None, :], sin[:, None, :]
            return torch.cat([a * c - b * s, b * c + a * s], -1)
        q, k = rot(q), rot(k)
        out = torch.empty(T, NH, D)
        for t0, t1 in segments:
            s = torch.einsum("qhd,khd->hqk", q[t0:t1], k[t0:t1]) / math.sqrt(D)
            out[t0:t1] = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v[t0:t1])
        return out.view(T, H).to(qkv.dtype)

    def pos_embed(self, grid: Tuple[int, int, int]) -> torch.Tensor:
        """The learned ``side x side`` position grid resampled (bilinear) to ``gh x gw``, in merge-block order."""
        t, gh, gw = grid
        side = int(round(math.sqrt(self.pos.shape[0])))
        p = self.pos.float().view(1, side, side, -1).permute(0, 3, 1, 2)
        p = F.interpolate(p, size=(gh, gw), mode="bilinear", align_corners=True)[0].permute(1, 2, 0)      # [gh, gw, H]
        m = self.cfg.spatial_merge_size
        p = p.view(gh // m, m, gw // m, m, -1).permute(0, 2, 1, 3, 4).reshape(gh * gw, -1)
        return p.repeat(t, 1).to(self.dtype)

    # -------------------------------------------------------------- forward
    def encode(self, patches: torch.Tensor, grids: Sequence[Tuple[int, int, int]], merge: bool = True) -> torch.Tensor:
        """``patches`` ``[T, patch_dim]`` of one or more images (concatenated), ``grids`` their (t, h, w).  Returns the
        language-model embeddings ``[T / merge², out_hidden]`` (or the encoder output ``[T, hidden]`` with ``merge=False``)."""
        cfg = self.cfg
        dev = self.device
        x = self._linear(self.patch, patches.to(dev, self.dtype))
        pos, cs, sn, segs, t0 = [], [], [], [], 0
        for g in grids:
            n = g[0] * g[1] * g[2]
            pos.append(self.pos_embed(g))
            c, s = rope_tables(g, cfg)
            cs.append(c)
            sn.append(s)
            per = g[1] * g[2]
            for f in range(g[0]):                     # attention stays inside one frame of one image
                segs.append((t0 + f * per, t0 + (f + 1) * per))
            t0 += n
        x = (x.float() + torch.cat(pos).to(dev).float()).to(self.dtype)
        cos, sin = torch.cat(cs).to(dev), torch.cat(sn).to(dev)
        for b in self.blocks:
            h = self._layernorm(x, b.ln1_w, b.ln1_b)
            a = self._attention(self._linear(b.qkv, h), cos, sin, segs)
            x = x + self._linear(b.proj, a)
            h = self._layernorm(x, b.ln2_w, b.ln2_b)
            x = x + self._linear(b.fc2, self._gelu(self._linear(b.fc1, h)))
        if not merge:
            return x
        m2 = cfg.spatial_merge_size ** 2
        h = self._layernorm(x, self.merge_ln_w, self.merge_ln_b).view(x.shape[0] // m2, m2 * cfg.hidden_size)
        return self._linear(self.merge_fc2, self._gelu(self._linear(self.merge_fc1, h)))

    # -------------------------------------------------------------- the C++ CPU tower as oracle
    def encode_cpu_oracle(self, patches: torch.Tensor, grid: Tuple[int, int, int], threads: int = 8) -> torch.Tensor:
        """fp32 encoder output ``[T, hidden]`` (before the merger) of ONE image through ``blz_vit_forward_cpu``."""
        from .. import runtime
        lib = runtime.lib()
        cfg = self.cfg
        keep = []

        def fp(t):
            t = t.detach().float().cpu().contiguous()
            keep.append(t)
            return ctypes.cast(t.data_ptr(), ctypes.POINTER(ctypes.c_float))

        class Blk(ctypes.Structure):
            _fields_ = [(n, ctypes.POINTER(ctypes.c_float)) for n in
                        ("ln1_w", "ln1_b", "qkv_w", "qkv_b", "proj_w", "proj_b", "ln2_w", "ln2_b", "fc1_w", "fc1_b", "fc2_w", "fc2_b")]

        class Wts(ctypes.Structure):
            _fields_ = [("hidden", ctypes.c_int), ("heads", ctypes.c_int), ("mlp", ctypes.c_int), ("depth", ctypes.c_int),
                        ("patch_dim", ctypes.c_int), ("eps", ctypes.c_float),
                        ("patch_w", ctypes.POINTER(ctypes.c_float)), ("patch_b", ctypes.POINTER(ctypes.c_float)),
                        ("pos", ctypes.POINTER(ctypes.c_float)), ("rope_cos", ctypes.POINTER(ctypes.c_float)),
                        ("rope_sin", ctypes.POINTER(ctypes.c_float)), ("blocks", ctypes.POINTER(Blk)),
                        ("ln_f_w", ctypes.POINTER(ctypes.c_float)), ("ln_f_b", ctypes.POINTER(ctypes.c_float))]

        blks = (Blk * cfg.depth)()
        for i, b in enumerate(self.blocks):
            blks[i] = Blk(fp(b.ln1_w), fp(b.ln1_b), fp(b.qkv.w), fp(b.qkv.bias), fp(b.proj.w), fp(b.proj.bias), fp(b.ln2_w),
                          fp(b.ln2_b), fp(b.fc1.w), fp(b.fc1.bias), fp(b.fc2.w), fp(b.fc2.bias))
        cos, sin = rope_tables(grid, cfg)
        null = ctypes.POINTER(ctypes.c_float)()
        w = Wts(cfg.hidden_size, cfg.num_heads, cfg.intermediate_size, cfg.depth, cfg.patch_dim, cfg.eps, fp(self.patch.w),
                fp(self.patch.bias), fp(self.pos_embed(grid)), fp(cos), fp(sin), blks, null, null)
        T = patches.shape[0]
        x = patches.detach().float().cpu().contiguous()
        out = torch.empty(T, cfg.hidden_size, dtype=torch.float32)
        lib.blz_vit_forward_cpu(VP(x.data_ptr()), T, ctypes.byref(w), VP(out.data_ptr()), threads)
        return out


class Vision:
    """What the server holds: the tower plus the ids it needs to splice image embeddings into a prompt
    (``vision.rs:88`` ``Vision::load``)."""

    def __init__(self, tower: VisionTower, image_pad_id: int):
        self.tower, self.image_pad_id = tower, image_pad_id
        self.cfg = tower.cfg

    @classmethod
    def load(cls, model_dir: str, device) -> Optional["Vision"]:
        tower = VisionTower.load(model_dir, device)
        if tower is None:
            return None
        with open(os.path.join(model_dir, "config.json")) as f:
            raw = json.load(f)
        pad = raw.get("image_token_id", raw.get("vision_config", {}).get("image_token_id", -1))
        return cls(tower, int(pad))

    def encode(self, image, min_pixels: Optional[int] = None, max_pixels: Optional[int] = None) -> Tuple[torch.Tensor, Tuple[int, int]]:
        """One decoded RGB image (``[H, W, 3]`` uint8) -> (embeddings ``[tokens, out_hidden]``, merged (h, w) grid).
        ``min_pixels`` / ``max_pixels`` replace the processor's resize limits for this image."""
        cfg = self.cfg
        if min_pixels is not None or max_pixels is not None:
            import dataclasses
            cfg = dataclasses.replace(cfg, min_pixels=min_pixels or cfg.min_pixels, max_pixels=max_pixels or cfg.max_pixels)
        if not isinstance(image, torch.Tensor):
            import numpy as np
            image = torch.from_numpy(np.array(image))      # a decoded PIL image or an array (copied: writable)
        patches, grid = preprocess(image, cfg)
        emb = self.tower.encode(patches, [grid])
        m = self.cfg.spatial_merge_size
        return emb, (grid[1] // m, grid[2] // m)


def check_reference(model_dir: Optional[str], image_path: Optional[str]) -> int:
    """CLI ``vision-check``: run one image through the device tower and the C++ CPU tower and print the difference."""
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    vt = VisionTower.load(model_dir, dev) if model_dir and os.path.isdir(model_dir) else None
    if vt is None:
        vt = VisionTower.random_init(VisionConfig(hidden_size=256, num_heads=4, intermediate_size=512, depth=2, out_hidden_size=256,
                                                  num_position_embeddings=64), dev)
    if image_path:
        from ..server.media import decode_image
        with open(image_path, "rb") as f:
            img = decode_image(f.read())
        import numpy as np
        img = torch.from_numpy(np.array(img))
    else:
        img = (torch.rand(224, 224, 3, generator=torch.Generator().manual_seed(0)) * 255).to(torch.uint8)
    patches, grid = preprocess(img, vt.cfg)
    got = vt.encode(patches, [grid], merge=False).float().cpu()
    want = vt.encode_cpu_oracle(patches, grid)
    err = (got - want).abs().max().item()
    print(json.dumps({"tokens": patches.shape[0], "grid": grid, "max_abs_err": err, "mean_abs_ref": want.abs().mean().item(),
                      "device": dev}))
    return 0 if err < 0.1 * max(1.0, want.abs().max().item()) else 1
