"""Vision tower on CPU: preprocessing shapes, and the torch fp32 path against the C++ tower of the host runtime."""
import torch

from blaze_b200.models.vision import VisionConfig, VisionTower, preprocess, rope_tables, smart_resize

CFG = VisionConfig(hidden_size=64, num_heads=4, intermediate_size=96, depth=2, patch_size=8, out_hidden_size=48,
                   num_position_embeddings=36, min_pixels=16 * 16, max_pixels=96 * 96)


def test_smart_resize_rules():
    assert smart_resize(100, 100, 16, 16 * 16, 1 << 20) == (96, 96)
    h, w = smart_resize(4000, 3000, 32, 56 * 56, 1280 * 28 * 28)
    assert h % 32 == 0 and w % 32 == 0 and h * w <= 1280 * 28 * 28 and abs(h / w - 4 / 3) < 0.05
    h, w = smart_resize(10, 12, 16, 64 * 64, 1 << 20)
    assert h * w >= 64 * 64


def test_preprocess_patch_order_and_grid():
    img = (torch.rand(50, 70, 3, generator=torch.Generator().manual_seed(1)) * 255).to(torch.uint8)
    patches, grid = preprocess(img, CFG)
    t, gh, gw = grid
    assert t == 1 and gh % CFG.spatial_merge_size == 0 and gw % CFG.spatial_merge_size == 0
    assert patches.shape == (gh * gw, CFG.patch_dim)
    cos, sin = rope_tables(grid, CFG)
    assert cos.shape == (gh * gw, CFG.head_dim // 2)
    # the four patches of one merge block are consecutive tokens: rows differ by < merge, columns too
    assert torch.allclose(cos[0], torch.ones(CFG.head_dim // 2))


def test_torch_tower_matches_cpp_tower():
    vt = VisionTower.random_init(CFG, "cpu", dtype=torch.float32, seed=3)
    img = (torch.rand(48, 64, 3, generator=torch.Generator().manual_seed(2)) * 255).to(torch.uint8)
    patches, grid = preprocess(img, CFG)
    got = vt.encode(patches, [grid], merge=False)
    want = vt.encode_cpu_oracle(patches, grid, threads=2)
    assert got.shape == want.shape
    assert (got - want).abs().max().item() < 2e-3 * max(1.0, want.abs().max().item())
    merged = vt.encode(patches, [grid])
    assert merged.shape == (patches.shape[0] // 4, CFG.out_hidden_size)
    # two images in one call give the same rows as two calls
    both = vt.encode(torch.cat([patches, patches]), [grid, grid])
    assert torch.allclose(both[:merged.shape[0]], merged, atol=1e-5) and torch.allclose(both[merged.shape[0]:], merged, atol=1e-5)
