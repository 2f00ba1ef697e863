"""CUDA vision tower (tcgen05 GEMMs + vision.cu kernels) against the C++ CPU tower."""
import pytest
import torch

from blaze_b200.models.vision import VisionConfig, VisionTower, preprocess

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("hidden,heads", [(128, 4), (288, 4), (256, 4)])
def test_cuda_tower_matches_cpu_tower(hidden, heads):
    cfg = VisionConfig(hidden_size=hidden, num_heads=heads, intermediate_size=2 * hidden, depth=2, patch_size=8,
                       out_hidden_size=192, num_position_embeddings=64, min_pixels=32 * 32, max_pixels=256 * 256)
    vt = VisionTower.random_init(cfg, "cuda", seed=5)
    img = (torch.rand(120, 168, 3, generator=torch.Generator().manual_seed(6)) * 255).to(torch.uint8)
    patches, grid = preprocess(img, cfg)
    got = vt.encode(patches, [grid], merge=False).float().cpu()
    torch.cuda.synchronize()
    assert vt._ops.take_status() == 0 and vt._ops.launches > 0
    want = vt.encode_cpu_oracle(patches, grid)
    err = (got - want).abs()
    scale = want.abs().mean().item()
    print(f"[vision {hidden}/{heads}] tokens={patches.shape[0]} mean|ref|={scale:.3f} mean err={err.mean().item():.4f} max err={err.max().item():.4f}")
    assert err.mean().item() < 0.03 * scale + 0.02
    assert err.max().item() < 0.25 * max(1.0, want.abs().max().item())
    merged = vt.encode(patches, [grid])
    assert merged.shape == (patches.shape[0] // 4, cfg.out_hidden_size) and torch.isfinite(merged.float()).all()
    two = vt.encode(torch.cat([patches, patches]), [grid, grid])
    assert torch.equal(two[:merged.shape[0]], merged) and torch.equal(two[merged.shape[0]:], merged)
