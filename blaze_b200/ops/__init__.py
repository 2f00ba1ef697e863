"""Op layer: ``RefOps`` (PyTorch oracle, any device) and ``CudaOps`` (sm_100a kernels).

``get_ops(device)`` returns the kernel-backed implementation for CUDA devices and raises if the
native library is missing there — a GPU run never falls back silently to the oracle.
"""
from __future__ import annotations

import torch

from .ref_ops import RefOps


def get_ops(device, force_ref: bool = False):
    dev = torch.device(device)
    if dev.type != "cuda" or force_ref:
        return RefOps()
    from .cuda_ops import CudaOps  # raises when the extension cannot be loaded
    return CudaOps(dev)
