"""Build and load the native libraries (in-tree, sm_100a only).

``libblaze_kernels.so``  — every ``csrc/kernels/*.cu`` (C ABI ``blz_*`` over raw device pointers and a stream,
                           returning a ``cudaError_t`` code, like the reference's kernel library,
                           ``kernels/CMakeLists.txt:23``).
``libblaze_runtime.so``  — ``csrc/runtime/*.cpp`` host runtime (safetensors reader, weight repack, page
                           allocator, CPU oracles, log bridge).

The reference builds its kernels with CMake and binds them through a Rust FFI crate
(``crates/blaze-sys/build.rs``, ``crates/blaze-sys/src/lib.rs``); here the binding is ctypes over the same kind
of C ABI.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "csrc")
LIBDIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_lib")
KERNELS_SO = os.path.join(LIBDIR, "libblaze_kernels.so")
RUNTIME_SO = os.path.join(LIBDIR, "libblaze_runtime.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-I" + os.path.join(CSRC, "include")]


def _nvcc() -> Optional[str]:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    return None


def _sources(sub: str, ext: str) -> List[str]:
    d = os.path.join(CSRC, sub)
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(ext)) if os.path.isdir(d) else []


def _digest(paths: List[str]) -> str:
    h = hashlib.sha256()
    incs = []
    for dp, _, fs in os.walk(os.path.join(CSRC, "include")):
        incs += [os.path.join(dp, f) for f in fs]
    for p in sorted(paths + incs):
        h.update(p.encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale(so: str, paths: List[str]) -> bool:
    stamp = so + ".sha"
    if not os.path.exists(so) or not os.path.exists(stamp):
        return True
    with open(stamp) as f:
        return f.read().strip() != _digest(paths)


def build(force: bool = False, verbose: bool = False) -> None:
    """Compile everything that is out of date.  Raises on a compiler error."""
    os.makedirs(LIBDIR, exist_ok=True)
    cu = _sources("kernels", ".cu")
    if cu and (force or _stale(KERNELS_SO, cu)):
        nvcc = _nvcc()
        if nvcc is None:
            raise RuntimeError("nvcc not found; cannot build blaze_b200 kernels")
        objdir = os.path.join(LIBDIR, "obj")
        os.makedirs(objdir, exist_ok=True)

        def one(src):
            obj = os.path.join(objdir, os.path.basename(src) + ".o")
            cmd = [nvcc] + NVCC_FLAGS + ["-c", src, "-o", obj]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
            if verbose and r.stderr:
                print(r.stderr, file=sys.stderr)
            return obj

        with ThreadPoolExecutor(max_workers=min(8, len(cu))) as ex:
            objs = list(ex.map(one, cu))
        r = subprocess.run([nvcc, "-shared", "-o", KERNELS_SO] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        with open(KERNELS_SO + ".sha", "w") as f:
            f.write(_digest(cu))
    cpp = _sources("runtime", ".cpp")
    if cpp and (force or _stale(RUNTIME_SO, cpp)):
        cxx = shutil.which("g++") or "g++"
        cmd = [cxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-pthread", "-mavx2", "-mfma", "-ffp-contract=off",
               "-I" + os.path.join(CSRC, "include"), "-o", RUNTIME_SO] + cpp
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"g++ failed:\n{r.stdout}\n{r.stderr}")
        with open(RUNTIME_SO + ".sha", "w") as f:
            f.write(_digest(cpp))


_kernels = None
_runtime = None


def kernels() -> ctypes.CDLL:
    """The CUDA kernel library.  Builds it when missing and nvcc is present; raises otherwise."""
    global _kernels
    if _kernels is None:
        if not os.path.exists(KERNELS_SO) or (os.environ.get("BLAZE_REBUILD") and _stale(KERNELS_SO, _sources("kernels", ".cu"))):
            build()
        if not os.path.exists(KERNELS_SO):
            raise RuntimeError(f"{KERNELS_SO} is missing: run `python -c 'import __graft_entry__ as g; g.build()'`")
        # BLAZE_KERNELS_SO: load another build of the kernel library (A/B timing of kernel variants in one process set-up)
        _kernels = ctypes.CDLL(os.environ.get("BLAZE_KERNELS_SO") or KERNELS_SO)
    return _kernels


def runtime() -> ctypes.CDLL:
    global _runtime
    if _runtime is None:
        if not os.path.exists(RUNTIME_SO):
            build()
        _runtime = ctypes.CDLL(RUNTIME_SO)
    return _runtime


def have_runtime() -> bool:
    try:
        runtime()
        return True
    except Exception:
        return False
