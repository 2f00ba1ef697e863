"""The allocation-free decode-attention entry point (``blz_attn_decode_noalloc``), called through its exported C symbol.

Callers that must not allocate device memory (code running under someone else's stream capture, host callbacks, processes
with a frozen memory pool) use it for split-KV decode attention: its scratch is a fixed array inside the library.  The
test runs it twice in a row and checks both results against the regular entry point, which takes caller-owned scratch.
This file sorts last so that a failure here cannot hide any other test's result.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
VP = ctypes.c_void_p


def _p(t):
    return VP(0) if t is None else VP(t.data_ptr())


def test_noalloc_matches_regular_entry_point_twice():
    from blaze_b200._native import kernels
    from blaze_b200.batch import SeqChunk, build_batch
    from blaze_b200.config import ModelConfig, RopeConfig
    from blaze_b200.kv import KVCache
    lib = kernels()
    fn = lib.blz_attn_decode_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [VP, VP, VP, VP, VP, VP, VP, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_longlong, ctypes.c_longlong, ctypes.c_float,
                   ctypes.c_float, ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, VP]
    lib.blz_attn_decode_noalloc_error.restype = ctypes.c_char_p
    lib.blz_attn_decode_noalloc_bytes.restype = ctypes.c_longlong
    lib.blz_attn_decode_noalloc_bytes.argtypes = [ctypes.c_int] * 4
    lib.blz_attn_decode_noalloc_status.restype = ctypes.c_int
    ref = lib.blz_attn_decode
    ref.restype = ctypes.c_int
    ref.argtypes = [VP, VP, VP, VP, VP, VP, VP, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                    ctypes.c_longlong, ctypes.c_longlong, ctypes.c_float,
                    ctypes.c_float, ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, VP, VP,
                    ctypes.c_int, VP, VP]
    dev = "cuda"
    Hq, Hkv, D, splits = 8, 2, 128, 4
    ctxs = [1500, 700, 130]
    B = len(ctxs)
    cfg = ModelConfig(hidden_size=Hq * D, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, num_layers=1, rope=RopeConfig(theta=1e6))
    cfg.layer_types = ["full_attention"]
    pages = (max(ctxs) + 15) // 16 + 1
    kv = KVCache(cfg, 1 + B * pages, B, pages, "fp8", dev, "umma")
    g = torch.Generator(device=dev).manual_seed(3)
    perm = torch.randperm(B * pages, generator=torch.Generator().manual_seed(3)).tolist()
    for b in range(B):
        kv.set_pages(b, [1 + p for p in perm[b * pages:(b + 1) * pages]])
    kv.kv[0].copy_(torch.randint(0, 96, kv.kv[0].shape, dtype=torch.uint8, device=dev, generator=g))   # finite e4m3 codes
    batch = build_batch([SeqChunk(b, [0], c - 1) for b, c in enumerate(ctxs)], kv.block_table_host, dev)
    stream = VP(torch.cuda.current_stream().cuda_stream)
    scale = D ** -0.5 * 0.02
    group = Hq // Hkv
    assert lib.blz_attn_decode_noalloc_bytes(B, Hkv, 1, splits) == B * Hkv * splits * 16 * 130 * 4
    for call in range(2):
        q = torch.randn(B, Hq, D, device=dev, generator=g).bfloat16()
        want = torch.zeros(B, Hq, D, dtype=torch.bfloat16, device=dev)
        n = B * Hkv * splits * 16
        po = torch.empty(n * D, dtype=torch.float32, device=dev)
        pm = torch.empty(n * 2, dtype=torch.float32, device=dev)
        rc = ref(_p(q), _p(want), _p(kv.kv[0]), _p(kv.block_table), _p(batch.slots), _p(batch.q_start), _p(batch.ctx_len), B, Hq, Hkv, D,
                 kv.block_table.stride(0), kv.kv[0].stride(0), kv.kv[0].stride(1), scale, 1.0, 1.0, 16, 1, 1, group, splits, _p(po), _p(pm), 0, VP(0), stream)
        assert rc == 0
        got = torch.zeros_like(want)
        rc = fn(_p(q), _p(got), _p(kv.kv[0]), _p(kv.block_table), _p(batch.slots), _p(batch.q_start), _p(batch.ctx_len), B, Hq, Hkv, D,
                kv.block_table.stride(0), kv.kv[0].stride(0), kv.kv[0].stride(1), scale, 1.0, 1.0, 1, 1, group, splits, 0, stream)
        assert rc == 0, lib.blz_attn_decode_noalloc_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        # both entry points launch the same kernel with the same split count: the results agree bit for bit
        assert torch.equal(got, want), f"call {call}: max abs err {(got.float() - want.float()).abs().max().item()}"
        assert lib.blz_attn_decode_noalloc_status() == 0      # no bounded wait ran out inside the kernel
    # a problem whose partials cannot fit the built-in array is refused with a message, not attempted
    rc = fn(_p(q), _p(got), _p(kv.kv[0]), _p(kv.block_table), _p(batch.slots), _p(batch.q_start), _p(batch.ctx_len), 4096, Hq, Hkv, D,
            kv.block_table.stride(0), kv.kv[0].stride(0), kv.kv[0].stride(1), scale, 1.0, 1.0, 1, 1, group, 8, 0, stream)
    assert rc != 0 and b"exceeds the built-in" in lib.blz_attn_decode_noalloc_error()
    # row blocks that do not cover the declared rows per kv head are refused as well (rows would be skipped silently)
    rc = fn(_p(q), _p(got), _p(kv.kv[0]), _p(kv.block_table), _p(batch.slots), _p(batch.q_start), _p(batch.ctx_len), B, Hq, Hkv, D,
            kv.block_table.stride(0), kv.kv[0].stride(0), kv.kv[0].stride(1), scale, 1.0, 1.0, 1, 1, 40, splits, 0, stream)
    assert rc != 0 and b"do not cover" in lib.blz_attn_decode_noalloc_error()
