"""Local safetensors checkpoints: reader (mmap), writer (for synthetic test checkpoints).

Same job as the reference's ``crates/blaze/src/weights.rs:83-204`` (mmap every ``*.safetensors``,
validate headers, find the text-model prefix) and of its C++ reader
``kernels/src/runtime/safetensors.cpp``.  When the native runtime library is built, large reads
go through its pread-based reader into pinned staging; otherwise tensors are views of the mmap.
"""
from __future__ import annotations

import glob
import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
    "F8_E4M3": (torch.float8_e4m3fn, 1), "F8_E5M2": (torch.float8_e5m2, 1), "F8_E8M0": (torch.uint8, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items() if k != "F8_E8M0"}


class TensorInfo:
    __slots__ = ("name", "dtype", "shape", "begin", "end", "file")

    def __init__(self, name, dtype, shape, begin, end, file):
        self.name, self.dtype, self.shape, self.begin, self.end, self.file = name, dtype, tuple(shape), begin, end, file


class _File:
    def __init__(self, path: str):
        self.path = path
        self.f = open(path, "rb")
        size = os.fstat(self.f.fileno()).st_size
        if size < 8:
            raise ValueError(f"{path}: too small for a safetensors file")
        (hlen,) = struct.unpack("<Q", self.f.read(8))
        if hlen > size - 8 or hlen > (100 << 20):
            raise ValueError(f"{path}: bad header length {hlen}")
        header = json.loads(self.f.read(hlen))
        self.data_off = 8 + hlen
        self.mm = mmap.mmap(self.f.fileno(), 0, access=mmap.ACCESS_READ)
        self.tensors: Dict[str, TensorInfo] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            dt = meta["dtype"]
            if dt not in _DTYPES:
                raise ValueError(f"{path}: tensor {name} has unsupported dtype {dt}")
            b, e = meta["data_offsets"]
            n = 1
            for s in meta["shape"]:
                n *= s
            if e - b != n * _DTYPES[dt][1] or self.data_off + e > size:
                raise ValueError(f"{path}: tensor {name} has inconsistent offsets")
            self.tensors[name] = TensorInfo(name, dt, meta["shape"], b, e, self)

    def read(self, info: TensorInfo) -> torch.Tensor:
        tdt, _ = _DTYPES[info.dtype]
        n = info.end - info.begin
        if n == 0:
            return torch.empty(info.shape, dtype=tdt)
        buf = np.frombuffer(self.mm, dtype=np.uint8, count=n, offset=self.data_off + info.begin)
        t = torch.from_numpy(buf)  # read-only view of the mapping; callers copy to the device
        return t.view(tdt).view(info.shape)


class Checkpoint:
    """All ``*.safetensors`` files of a model directory behind one name → tensor map."""

    def __init__(self, model_dir: str):
        self.dir = model_dir
        paths = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
        if not paths:
            raise FileNotFoundError(f"no *.safetensors under {model_dir}")
        self.files = [_File(p) for p in paths]
        # Large tensors are read by the C++ reader of the host runtime library (several pread threads per tensor into
        # pinned staging memory, csrc/runtime/safetensors.cpp) when it is built; small ones are views of the mapping.
        self.native = None
        if os.environ.get("BLAZE_NATIVE_READER", "1") != "0":
            try:
                from .runtime import NativeCheckpoint
                self.native = NativeCheckpoint(model_dir)
            except Exception:
                self.native = None
        self.index: Dict[str, TensorInfo] = {}
        for f in self.files:
            for k, v in f.tensors.items():
                if k in self.index:
                    raise ValueError(f"tensor {k} appears in two shards")
                self.index[k] = v

    NATIVE_MIN_BYTES = 1 << 20

    @classmethod
    def open(cls, model_dir: str) -> "Checkpoint":
        return cls(model_dir)

    def __contains__(self, name: str) -> bool:
        return name in self.index

    def names(self) -> Iterable[str]:
        return self.index.keys()

    def meta(self) -> Dict[str, Tuple[str, Tuple[int, ...]]]:
        return {k: (v.dtype, v.shape) for k, v in self.index.items()}

    def get(self, name: str) -> torch.Tensor:
        info = self.index.get(name)
        if info is None:
            raise KeyError(f"tensor {name} not in checkpoint {self.dir}")
        if self.native is not None and info.end - info.begin >= self.NATIVE_MIN_BYTES and name in self.native:
            t = self.native.get(name, pin=torch.cuda.is_available())
            return t.view(torch.uint8) if info.dtype == "F8_E8M0" else t
        return info.file.read(info)

    def get_opt(self, name: str) -> Optional[torch.Tensor]:
        return self.get(name) if name in self.index else None

    def text_prefix(self) -> str:
        """``model.language_model.`` for multimodal wrappers, else ``model.`` (``weights.rs:155``)."""
        for k in self.index:
            if k.startswith("model.language_model."):
                return "model.language_model."
        return "model."

    def total_bytes(self) -> int:
        return sum(v.end - v.begin for v in self.index.values())


def save_safetensors(path: str, tensors: Dict[str, torch.Tensor], dtype_override: Optional[Dict[str, str]] = None,
                     metadata: Optional[Dict[str, str]] = None) -> None:
    """Write one safetensors file (used to build synthetic checkpoints in every quant format)."""
    header = {}
    if metadata:
        header["__metadata__"] = metadata
    off = 0
    blobs: List[bytes] = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        dt = (dtype_override or {}).get(name) or _NAMES[t.dtype]
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": dt, "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for b in blobs:
            f.write(b)
