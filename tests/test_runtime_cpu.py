"""Host runtime library (C++): safetensors reader, scale-factor repack, page allocator, CPU expert oracle."""
import os

import pytest
import torch

from blaze_b200 import quant, runtime
from blaze_b200.linear import Linear
from blaze_b200.ops import ref
from blaze_b200.quant import Format
from blaze_b200.weights import Checkpoint, save_safetensors


def test_native_safetensors_matches_python_reader(tmp_path):
    g = torch.Generator().manual_seed(0)
    tensors = {"a.weight": torch.randn(33, 17, generator=g).bfloat16(), "b": torch.randint(0, 255, (5, 4, 3), generator=g, dtype=torch.uint8),
               "c.scale": torch.randn(7, generator=g), "d.e4m3": torch.randn(8, 16, generator=g).to(torch.float8_e4m3fn)}
    save_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), {k: tensors[k] for k in ("a.weight", "b")})
    save_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), {k: tensors[k] for k in ("c.scale", "d.e4m3")})
    py = Checkpoint.open(str(tmp_path))
    nat = runtime.NativeCheckpoint(str(tmp_path))
    assert set(nat.names()) == set(py.names()) == set(tensors)
    for k, t in tensors.items():
        got = nat.get(k)
        assert got.dtype == t.dtype and tuple(got.shape) == tuple(t.shape)
        assert torch.equal(got.view(torch.uint8), t.view(torch.uint8))
        assert torch.equal(py.get(k).view(torch.uint8), t.view(torch.uint8))
    with open(tmp_path / "bad.safetensors", "wb") as f:
        f.write(b"\xff" * 16)
    with pytest.raises(OSError):
        runtime.NativeCheckpoint(str(tmp_path))
    with pytest.raises(ValueError):
        Checkpoint.open(str(tmp_path))


def test_swizzle_twin_and_pages():
    sf = torch.randint(0, 255, (200, 10), dtype=torch.uint8)
    assert torch.equal(runtime.swizzle_sf(sf), quant.swizzle_sf_128x4(sf))
    assert torch.equal(quant.unswizzle_sf_128x4(quant.swizzle_sf_128x4(sf), 200, 10), sf)
    p = runtime.NativePages(10)
    a = p.alloc(4)
    assert len(set(a)) == 4 and 0 not in a and p.free_count == 5
    p.retain(a[:2])
    p.release(a)
    assert p.free_count == 7
    p.release(a[:2])
    assert p.free_count == 9
    with pytest.raises(RuntimeError):
        p.release(a[:1])
    from blaze_b200.engine import OutOfPages
    with pytest.raises(OutOfPages):
        p.alloc(10)


def test_cpu_expert_oracle_matches_torch_reference():
    g = torch.Generator().manual_seed(1)
    H, I = 128, 64
    gu = Linear.from_dense(torch.randn(2 * I, H, generator=g) * 0.1, Format.NVFP4, act_quant=False, segments=[I, I])
    dn = Linear.from_dense(torch.randn(H, I, generator=g) * 0.1, Format.NVFP4, act_quant=False)
    x = torch.randn(9, H, generator=g)
    want = ref.silu_mul(x @ gu.dequant().t()) @ dn.dequant().t()
    got = runtime.cpu_expert_nvfp4(x, gu, dn, threads=3)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)
