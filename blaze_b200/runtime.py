"""ctypes bindings of the host runtime library (``libblaze_runtime.so``): safetensors reader, scale-factor repack,
page allocator, CPU expert oracle, CPU vision tower, log bridge."""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import log
from ._native import runtime as _load

VP = ctypes.c_void_p
_lib = None
_log_cb = None


def lib():
    global _lib, _log_cb
    if _lib is None:
        l = _load()
        l.blz_st_open.restype = VP
        l.blz_st_open.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int]
        l.blz_st_close.argtypes = [VP]
        l.blz_st_count.argtypes = [VP]
        l.blz_st_info.argtypes = [VP, ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int,
                                  ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]
        l.blz_st_find.argtypes = [VP, ctypes.c_char_p]
        l.blz_st_read.argtypes = [VP, ctypes.c_int, VP, ctypes.c_int64, ctypes.c_int]
        l.blz_swizzle_sf.argtypes = [VP, ctypes.c_int64, ctypes.c_int64, VP]
        l.blz_swizzle_sf_bytes.restype = ctypes.c_int64
        l.blz_swizzle_sf_bytes.argtypes = [ctypes.c_int64, ctypes.c_int64]
        l.blz_pages_create.restype = VP
        l.blz_pages_create.argtypes = [ctypes.c_int]
        l.blz_pages_destroy.argtypes = [VP]
        l.blz_pages_free_count.argtypes = [VP]
        l.blz_pages_alloc.argtypes = [VP, ctypes.c_int, VP]
        l.blz_pages_retain.argtypes = [VP, VP, ctypes.c_int]
        l.blz_pages_release.argtypes = [VP, VP, ctypes.c_int]
        l.blz_cpu_expert_nvfp4.argtypes = [VP, ctypes.c_int, ctypes.c_int, ctypes.c_int, VP, VP, VP, VP, VP, VP, VP, ctypes.c_int]
        l.blz_vit_forward_cpu.argtypes = [VP, ctypes.c_int, VP, VP, ctypes.c_int]
        cb_t = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_char_p)
        levels = {0: "debug", 1: "info", 2: "warn", 3: "error"}

        def _cb(level, msg):
            log.event(levels.get(level, "info"), "native", message=msg.decode("utf-8", "replace"))
        _log_cb = cb_t(_cb)
        l.blz_log_set(_log_cb)
        _lib = l
    return _lib


_ST_DTYPES = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64,
              "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
              "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2, "F8_E8M0": torch.uint8}


class NativeCheckpoint:
    """Safetensors directory through the C++ reader: tensors are pread (several threads) into pinned host memory."""

    def __init__(self, model_dir: str, threads: int = 8):
        err = ctypes.create_string_buffer(512)
        self.h = lib().blz_st_open(model_dir.encode(), err, 512)
        if not self.h:
            raise OSError(err.value.decode())
        self.threads = threads
        self.index: Dict[str, Tuple[int, str, Tuple[int, ...], int]] = {}
        name = ctypes.create_string_buffer(1024)
        dt = ctypes.create_string_buffer(32)
        shape = (ctypes.c_int64 * 8)()
        nb = ctypes.c_int64()
        for i in range(lib().blz_st_count(self.h)):
            r = lib().blz_st_info(self.h, i, name, 1024, dt, 32, shape, ctypes.byref(nb))
            self.index[name.value.decode()] = (i, dt.value.decode(), tuple(shape[k] for k in range(r)), nb.value)

    def names(self):
        return self.index.keys()

    def meta(self):
        return {k: (v[1], v[2]) for k, v in self.index.items()}

    def __contains__(self, name):
        return name in self.index

    def get(self, name: str, pin: bool = False) -> torch.Tensor:
        i, dt, shape, nb = self.index[name]
        buf = torch.empty(max(nb, 1), dtype=torch.uint8, pin_memory=pin and torch.cuda.is_available())
        if nb:
            rc = lib().blz_st_read(self.h, i, VP(buf.data_ptr()), nb, self.threads)
            if rc != 0:
                raise OSError(f"reading {name} failed: {rc}")
        return buf[:nb].view(_ST_DTYPES[dt]).view(shape)

    def close(self):
        if self.h:
            lib().blz_st_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def swizzle_sf(sf: torch.Tensor) -> torch.Tensor:
    """C++ twin of :func:`blaze_b200.quant.swizzle_sf_128x4` for CPU tensors."""
    s = sf.contiguous().view(torch.uint8).cpu()
    rows, cols = s.shape
    out = torch.empty(lib().blz_swizzle_sf_bytes(rows, cols), dtype=torch.uint8)
    lib().blz_swizzle_sf(VP(s.data_ptr()), rows, cols, VP(out.data_ptr()))
    return out


class NativePages:
    """Ref-counted page allocator in C++ (same interface as ``engine.PageAllocator``)."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self.h = lib().blz_pages_create(num_pages)

    @property
    def free_count(self) -> int:
        return lib().blz_pages_free_count(self.h)

    def alloc(self, n: int) -> List[int]:
        from .engine import OutOfPages
        out = (ctypes.c_int32 * max(n, 1))()
        if lib().blz_pages_alloc(self.h, n, out) != 0:
            raise OutOfPages(f"need {n} pages, {self.free_count} free")
        return list(out[:n])

    def retain(self, pages: Sequence[int]) -> None:
        a = (ctypes.c_int32 * max(len(pages), 1))(*pages)
        lib().blz_pages_retain(self.h, a, len(pages))

    def release(self, pages: Sequence[int]) -> None:
        a = (ctypes.c_int32 * max(len(pages), 1))(*pages)
        if lib().blz_pages_release(self.h, a, len(pages)) != 0:
            raise RuntimeError("a page was released twice")

    def __del__(self):
        try:
            lib().blz_pages_destroy(self.h)
        except Exception:
            pass


def cpu_expert_nvfp4(x: torch.Tensor, gate_up, down, threads: int = 8) -> torch.Tensor:
    """fp32 CPU result of one NVFP4 expert; ``gate_up`` / ``down`` are :class:`blaze_b200.linear.Linear` in NVFP4."""
    xf = x.float().cpu().contiguous()
    rows, H = xf.shape
    I = down.K
    y = torch.empty(rows, H, dtype=torch.float32)
    t = [gate_up.w.cpu().contiguous(), gate_up.sf.cpu().view(torch.uint8).contiguous(), gate_up.alpha.cpu().float().contiguous(),
         down.w.cpu().contiguous(), down.sf.cpu().view(torch.uint8).contiguous(), down.alpha.cpu().float().contiguous()]
    lib().blz_cpu_expert_nvfp4(VP(xf.data_ptr()), rows, H, I, *[VP(a.data_ptr()) for a in t], VP(y.data_ptr()), threads)
    return y
