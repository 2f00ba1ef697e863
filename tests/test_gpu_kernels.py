"""sm_100a kernels against plain PyTorch fp32 references of the same ops (run on a B200)."""
import math

import pytest
import torch

from blaze_b200 import quant
from blaze_b200.kv import KVCache
from blaze_b200.linear import Linear
from blaze_b200.ops import ref
from blaze_b200.quant import Format

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from blaze_b200.ops import get_ops
    return get_ops(DEV)


def _report(name, got, want):
    err = (got.float() - want.float()).abs()
    denom = want.float().abs().mean().item() + 1e-9
    print(f"[{name}] max_abs={err.max().item():.4g} mean_abs={err.mean().item():.4g} ref_mean_abs={denom:.4g}")
    return err.max().item(), err.mean().item() / denom


@pytest.mark.parametrize("M,N,K,bn", [(256, 512, 512, 128), (100, 384, 320, 128), (300, 1024, 1024, 256),
                                       (1, 4096, 4096, 128), (2048, 6144, 4096, 0)])
def test_gemm_bf16(ops, M, N, K, bn):
    g = torch.Generator(device=DEV).manual_seed(1)
    x = (torch.randn(M, K, generator=g, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g, device=DEV) * 0.05).bfloat16()
    lin = Linear.from_dense(w.float(), Format.DENSE)
    y = ops.linear(lin, x, bn=bn)
    want = x.float() @ w.float().t()
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    mx, rel = _report(f"gemm_bf16 {M}x{N}x{K} bn{bn}", y, want)
    assert rel < 0.01
    y32 = ops.linear(lin, x, out_dtype=torch.float32, bn=bn)
    assert torch.allclose(y32, want, atol=2e-3 * math.sqrt(K), rtol=1e-2)


@pytest.mark.parametrize("M,N,K,bn", [(128, 256, 256, 128), (256, 512, 1024, 128), (77, 384, 320, 128),
                                       (512, 1024, 4096, 256), (256, 6144, 4096, 0)])
def test_gemm_nvfp4(ops, M, N, K, bn):
    g = torch.Generator(device=DEV).manual_seed(2)
    x = (torch.randn(M, K, generator=g, device=DEV)).bfloat16()
    w = torch.randn(N, K, generator=g, device=DEV) * 0.02
    lin = Linear.from_dense(w, Format.NVFP4, segments=[N // 2, N - N // 2])
    y = ops.linear(lin, x, bn=bn)
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    want = lin.ref(x, torch.float32)
    mx, rel = _report(f"gemm_nvfp4 {M}x{N}x{K} bn{bn}", y, want)
    # the kernel's activation quantiser may round a few ties differently from the reference: compare to the
    # reference computed from the kernel's own quantised activations as well
    qa = ops.quantize_rows(x, lin)
    sfx = quant.unswizzle_sf_128x4(qa.sf, M, K // 16).view(torch.float8_e4m3fn)
    xd = quant.nvfp4_dequantize(qa.data, sfx, qa.row_scale)
    want2 = xd @ lin.dequant().t()
    mx2, rel2 = _report(f"gemm_nvfp4(kernel acts) {M}x{N}x{K}", y, want2)
    assert rel2 < 0.01
    assert rel < 0.05


@pytest.mark.parametrize("M,N,K,bn", [(128, 256, 256, 128), (200, 512, 1024, 128), (512, 1024, 2048, 256)])
def test_gemm_mxfp8(ops, M, N, K, bn):
    g = torch.Generator(device=DEV).manual_seed(3)
    x = (torch.randn(M, K, generator=g, device=DEV)).bfloat16()
    w = torch.randn(N, K, generator=g, device=DEV) * 0.02
    lin = Linear.from_dense(w, Format.MXFP8)
    y = ops.linear(lin, x, bn=bn)
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    want = lin.ref(x, torch.float32)
    mx, rel = _report(f"gemm_mxfp8 {M}x{N}x{K} bn{bn}", y, want)
    assert rel < 0.02


@pytest.mark.parametrize("fmt,M,N,K,ksplit", [
    ("nvfp4", 256, 4096, 4096, 4), ("nvfp4", 256, 6144, 4096, 3), ("nvfp4", 200, 1024, 12288, 8), ("nvfp4", 77, 512, 1024, 1),
    ("nvfp4", 1, 384, 512, 2), ("nvfp4", 128, 256, 256, 0), ("nvfp4", 1024, 1024, 4096, 0), ("nvfp4", 333, 512, 1024, 0),
    ("mxfp8", 256, 1024, 2048, 4), ("mxfp8", 40, 384, 1024, 1), ("mxfp8", 700, 512, 2048, 0),
    ("bf16", 256, 1000, 1024, 2), ("bf16", 19, 131, 320, 1), ("fp8", 192, 384, 512, 2)])
def test_gemm_wide(ops, fmt, M, N, K, ksplit):
    """Wide-N kernel: swapped orientation (M <= 256, optional split along K) and 256-feature tiles (M > 256)."""
    g = torch.Generator(device=DEV).manual_seed(21)
    x = (torch.randn(M, K, generator=g, device=DEV)).bfloat16()
    w = torch.randn(N, K, generator=g, device=DEV) * 0.02
    f = {"nvfp4": Format.NVFP4, "mxfp8": Format.MXFP8, "bf16": Format.DENSE, "fp8": Format.FP8_CHANNEL}[fmt]
    lin = Linear.from_dense(w, f)
    if fmt == "bf16":
        lin.bias = (torch.randn(N, generator=g, device=DEV) * 0.1).bfloat16()
        lin.cuda_pack = None
    y = ops.linear(lin, x, wide=True, ksplit=ksplit)
    y_tc = ops.linear(lin, x, wide=False)
    y32 = ops.linear(lin, x, out_dtype=torch.float32, wide=True, ksplit=ksplit)
    again = ops.linear(lin, x, wide=True, ksplit=ksplit)
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    assert torch.equal(y, again), "the split-K sum must be deterministic"
    mx, rel = _report(f"gemm_wide {fmt} {M}x{N}x{K} ks{ksplit} vs 128-column kernel", y, y_tc.float())
    assert rel < 2e-3
    mx, rel = _report(f"gemm_wide {fmt} fp32 out", y32, y_tc.float())
    assert rel < 4e-3
    want = lin.ref(x, torch.float32)
    mx, rel = _report(f"gemm_wide {fmt} vs oracle", y, want)
    assert rel < 0.05


@pytest.mark.parametrize("fmt,M,N,K,ks", [
    ("nvfp4", 256, 6144, 4096, 0), ("nvfp4", 256, 4096, 4096, 4), ("nvfp4", 256, 768, 4096, 8), ("nvfp4", 256, 4096, 512, 2),
    ("nvfp4", 200, 1024, 12288, 3), ("nvfp4", 77, 520, 1024, 4), ("nvfp4", 1, 384, 512, 2), ("nvfp4", 130, 256, 320, 5),
    ("nvfp4", 384, 1000, 2048, 6), ("mxfp8", 256, 1024, 2048, 4), ("mxfp8", 40, 384, 1024, 7), ("mxfp8", 300, 512, 2048, 1),
    ("bf16", 256, 1000, 1024, 2), ("bf16", 19, 131, 320, 3), ("fp8", 192, 384, 512, 2), ("fp8", 64, 256, 4096, 8)])
def test_gemm_cluster_split_k(ops, fmt, M, N, K, ks):
    """Decode GEMM whose K range is split over a thread-block cluster and reduced through distributed shared memory."""
    g = torch.Generator(device=DEV).manual_seed(31)
    x = (torch.randn(M, K, generator=g, device=DEV)).bfloat16()
    w = torch.randn(N, K, generator=g, device=DEV) * 0.02
    f = {"nvfp4": Format.NVFP4, "mxfp8": Format.MXFP8, "bf16": Format.DENSE, "fp8": Format.FP8_CHANNEL}[fmt]
    lin = Linear.from_dense(w, f)
    if fmt == "bf16":
        lin.bias = (torch.randn(N, generator=g, device=DEV) * 0.1).bfloat16()
        lin.cuda_pack = None
    xin = ops.quantize_rows(x, lin) if ops._qmode(lin) else x
    guard = torch.full((M + 2, N + 8), 7.0, dtype=torch.bfloat16, device=DEV)     # poison around the output
    out = guard[1:M + 1, :N]
    l0 = ops.launches
    y = ops.linear(lin, xin, sk=ks if ks else True, out=out)
    assert ops.launches == l0 + 1
    y_tc = ops.linear(lin, xin, wide=False, sk=False)
    again = ops.linear(lin, xin, sk=ks if ks else True)
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    assert torch.equal(y, again), "the cluster reduction must be deterministic"
    assert (guard[0] == 7).all() and (guard[M + 1] == 7).all() and (guard[:, N:] == 7).all(), "wrote outside the output"
    _, rel = _report(f"gemm_sk {fmt} {M}x{N}x{K} ks{ks} vs 128-column kernel", y, y_tc.float())
    assert rel < 2e-3
    want = lin.ref(x, torch.float32)
    _, rel = _report(f"gemm_sk {fmt} vs oracle", y, want)
    assert rel < 0.05


@pytest.mark.parametrize("M,N,K", [(256, 1024, 2048), (1, 384, 512), (77, 448, 1024), (300, 520, 384), (130, 256, 128),
                                   (1000, 2048, 5120)])
def test_gemm_fp8_block_scale_exact(ops, M, N, K):
    """FP8 weights with 128x128 fp32 block scales that are NOT powers of two and 1x128 activation groups: every K block is
    promoted in fp32 with its own (row, block) scale, so the result matches the fp32 oracle on the stored codes to bf16
    rounding, and the activation quantiser reproduces the oracle's codes and scales."""
    from blaze_b200 import quant
    g = torch.Generator(device=DEV).manual_seed(41)
    x = (torch.randn(M, K, generator=g, device=DEV) * (1 + 3 * torch.rand(M, 1, generator=g, device=DEV))).bfloat16()
    w = torch.randn(N, K, generator=g, device=DEV) * 0.02
    w = w * (0.3 + 2 * torch.rand((N + 127) // 128, 1, K // 128, 1, generator=g, device=DEV)).expand(-1, 128, -1, 128) \
        .reshape(-1, K)[:N]                                                  # very different magnitudes per block
    lin = Linear.from_dense(w, Format.FP8_BLOCK)
    lin.bias = (torch.randn(N, generator=g, device=DEV) * 0.1).bfloat16()
    assert ops.pack(lin)["kind"] == 4 and ops._qmode(lin) == 0
    # the quantiser against the oracle's 1x128 groups
    q, sc = ops.quantize_fp8_block(x)
    xg = x.float().view(M, K // 128, 128)
    s_want = (xg.abs().amax(-1) / quant.FP8_MAX).clamp_min(1e-12)
    s_got = sc[:, :M].t().contiguous()
    assert torch.allclose(s_got, s_want, rtol=1e-6, atol=0)          # (a division by 448 against a multiplication by 1/448)
    q_want = quant.to_e4m3(xg / s_got.unsqueeze(-1)).view(M, K)
    assert torch.equal(q.view(torch.float8_e4m3fn).float(), q_want.float())
    guard = torch.full((M + 2, N + 8), 7.0, dtype=torch.bfloat16, device=DEV)
    out = guard[1:M + 1, :N]
    y = ops.linear(lin, x, out=out)
    y32 = ops.linear(lin, x, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    assert (guard[0] == 7).all() and (guard[M + 1] == 7).all() and (guard[:, N:] == 7).all(), "wrote outside the output"
    want = (q_want.float().view(M, K // 128, 128) * s_got.unsqueeze(-1)).view(M, K) @ lin.dequant().t() + lin.bias.float()
    _, rel = _report(f"gemm_fp8_block {M}x{N}x{K} fp32 out vs oracle", y32, want)
    assert rel < 1e-5
    _, rel = _report(f"gemm_fp8_block {M}x{N}x{K} bf16 out vs oracle", y, want)
    assert rel < 4e-3
    # the re-expressed (MXFP8) path of the same layer loses the stored scales' mantissas: the exact path must be closer
    lin2 = Linear.from_dense(w, Format.FP8_BLOCK)
    lin2.bias = lin.bias
    old, ops._fp8_block_exact = ops._fp8_block_exact, False
    try:
        y_mx = ops.linear(lin2, x, out_dtype=torch.float32)
    finally:
        ops._fp8_block_exact = old
    dense = x.float() @ lin.dequant().t() + lin.bias.float()
    e_exact = ((y32 - dense).norm() / dense.norm()).item()
    e_mx = ((y_mx - dense).norm() / dense.norm()).item()
    print(f"[gemm_fp8_block] error against unquantised activations: exact path {e_exact:.4f}, MXFP8 re-expression {e_mx:.4f}")
    assert e_exact <= e_mx * 1.05


@pytest.mark.parametrize("fmt,M,N,K,ks", [
    ("nvfp4", 1, 6144, 4096, 0), ("nvfp4", 2, 4096, 12288, 8), ("nvfp4", 32, 1024, 2048, 4), ("nvfp4", 33, 512, 1024, 2),
    ("nvfp4", 64, 768, 4096, 0), ("nvfp4", 100, 256, 512, 2), ("nvfp4", 128, 1280, 2048, 3), ("mxfp8", 5, 1024, 2048, 0),
    ("mxfp8", 48, 384, 1024, 8), ("bf16", 7, 1024, 1024, 0), ("bf16", 96, 256, 320, 5), ("bf16", 16, 2048, 512, 1)])
def test_gemm_narrow_small_batch(ops, fmt, M, N, K, ks):
    """Dense layer at small batch: features on the tensor-core lanes, rows as 32..128 MMA columns, K split over a cluster
    and reduced through distributed shared memory.  Against the one-CTA-per-tile kernel and the oracle."""
    import ctypes
    g = torch.Generator(device=DEV).manual_seed(51)
    x = (torch.randn(M, K, generator=g, device=DEV)).bfloat16()
    w = torch.randn(N, K, generator=g, device=DEV) * 0.02
    f = {"nvfp4": Format.NVFP4, "mxfp8": Format.MXFP8, "bf16": Format.DENSE}[fmt]
    lin = Linear.from_dense(w, f)
    lin.bias = (torch.randn(N, generator=g, device=DEV) * 0.1).bfloat16()
    xin = ops.quantize_rows(x, lin) if ops._qmode(lin) else x
    pk = ops.pack(lin)
    guard = torch.full((M + 2, N + 8), 7.0, dtype=torch.bfloat16, device=DEV)
    out = guard[1:M + 1, :N]
    VP = ctypes.c_void_p
    ptr = lambda t: VP(0) if t is None else VP(t.data_ptr())      # noqa: E731
    if isinstance(xin, torch.Tensor):
        a, lda, sfa, rs = xin, K * 2, None, None
    else:
        a, lda, sfa, rs = xin.data, xin.data.shape[1], xin.sf, xin.row_scale
    wt = pk["w"]
    for _ in range(2):
        rc = ops.lib.blz_gemm_narrow(pk["kind"], ptr(a), lda, ptr(wt), wt.shape[1] * wt.element_size(), ptr(out), out.stride(0), M, N, K,
                                     ptr(rs), ptr(pk["alpha"]), ptr(pk["bias"]), ptr(sfa), ptr(pk["sf"]), ks, 0,
                                     VP(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
    y_tc = ops.linear(lin, xin, wide=False, sk=False)
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    assert (guard[0] == 7).all() and (guard[M + 1] == 7).all() and (guard[:, N:] == 7).all(), "wrote outside the output"
    _, rel = _report(f"gemm_narrow {fmt} {M}x{N}x{K} ks{ks} vs 128-column kernel", out, y_tc.float())
    assert rel < 2e-3
    want = lin.ref(x, torch.float32)
    _, rel = _report(f"gemm_narrow {fmt} vs oracle", out, want)
    assert rel < 0.05
    if M <= ops.NARROW_ROWS:
        l0 = ops.launches
        ops.NARROW_ALWAYS = True
        try:
            y = ops.linear(lin, xin)                    # the router's own call of the kernel (K slices chosen by the launcher)
        finally:
            ops.NARROW_ALWAYS = False
        assert ops.launches == l0 + 1
        assert (y.float() - out.float()).abs().max().item() <= 0.02 * out.float().abs().max().item()


def test_gemm_narrow_swiglu_epilogue(ops):
    g = torch.Generator(device=DEV).manual_seed(52)
    M, I, K = 24, 768, 1024
    x = torch.randn(M, K, generator=g, device=DEV).bfloat16()
    lin = Linear.from_dense(torch.randn(2 * I, K, generator=g, device=DEV) * 0.03, Format.NVFP4, segments=[I, I])
    ops.NARROW_ALWAYS = True
    try:
        y = ops.linear_swiglu(lin, x)
    finally:
        ops.NARROW_ALWAYS = False
    want = ref.silu_mul(lin.ref(x, torch.float32).bfloat16()).float()
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    _, rel = _report("gemm_narrow SwiGLU epilogue vs oracle", y, want)
    assert y.shape == (M, I) and rel < 0.05


@pytest.mark.parametrize("fmt,M,N,K", [("nvfp4", 300, 512, 1024), ("nvfp4", 64, 384, 576 * 2), ("bf16", 100, 200, 320),
                                       ("mxfp8", 130, 256, 640)])
def test_gemm_tile_major_weights(ops, fmt, M, N, K):
    """The tile-major weight repack gives the same result as row-major storage, through both GEMM kernels."""
    g = torch.Generator(device=DEV).manual_seed(22)
    x = (torch.randn(M, K, generator=g, device=DEV)).bfloat16()
    w = torch.randn(N, K, generator=g, device=DEV) * 0.02
    f = {"nvfp4": Format.NVFP4, "mxfp8": Format.MXFP8, "bf16": Format.DENSE}[fmt]
    lin = Linear.from_dense(w, f)
    want = ops.linear(lin, x, wide=False)
    lin.cuda_pack = None
    pk = ops.pack(lin, tiled=True)
    assert pk["kt"] > 0 and pk["w"].dim() == 4
    got = ops.linear(lin, x, wide=False)
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    assert torch.equal(got, want)
    if M <= 256 or (N % 256 == 0 and fmt != "bf16"):
        got_w = ops.linear(lin, x, wide=True)
        torch.cuda.synchronize()
        _, rel = _report(f"tile-major {fmt} wide", got_w, want.float())
        assert rel < 2e-3


@pytest.mark.parametrize("fmt,M,I,K", [("nvfp4", 300, 512, 1024), ("nvfp4", 77, 384, 512), ("nvfp4", 256, 1024, 1024),
                                       ("mxfp8", 600, 256, 1024), ("bf16", 90, 160, 320)])
def test_gemm_swiglu_epilogue(ops, fmt, M, I, K):
    """SwiGLU computed in the GEMM epilogue (interleaved gate / up rows) equals GEMM followed by the SwiGLU kernel."""
    g = torch.Generator(device=DEV).manual_seed(23)
    x = (torch.randn(M, K, generator=g, device=DEV)).bfloat16()
    w = torch.randn(2 * I, K, generator=g, device=DEV) * 0.05
    f = {"nvfp4": Format.NVFP4, "mxfp8": Format.MXFP8, "bf16": Format.DENSE}[fmt]
    lin = Linear.from_dense(w, f, segments=[I, I])
    down = Linear.from_dense(torch.randn(64, I, generator=g, device=DEV) * 0.05, f)
    want = ops.silu_mul(ops.linear(lin, x))
    lin.cuda_pack = None
    got = ops.linear_swiglu(lin, x)
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    assert got.shape == (M, I)
    d = (got.float() - want.float()).abs()
    print(f"[swiglu epilogue {fmt} {M}x{I}x{K}] max diff {d.max().item():.3g} mean |ref| {want.float().abs().mean().item():.3g}")
    assert d.max().item() <= 0.02 * max(1.0, want.float().abs().max().item())
    assert (d > 0).float().mean().item() < 0.02
    if fmt != "bf16":
        qa = ops.linear_swiglu(lin, x, quant_for=down)
        qb = ops.quantize_rows(got, down)
        per = 16 if fmt == "nvfp4" else 32
        sa = quant.unswizzle_sf_128x4(qa.sf, M, I // per)
        sb = quant.unswizzle_sf_128x4(qb.sf, M, I // per)
        assert torch.equal(qa.data, qb.data) and torch.equal(sa, sb)
    with pytest.raises(Exception):
        ops.linear(lin, x)          # packed for the SwiGLU epilogue: the plain GEMM must refuse it


def test_gemm_fp8_channel(ops):
    g = torch.Generator(device=DEV).manual_seed(4)
    x = (torch.randn(192, 512, generator=g, device=DEV)).bfloat16()
    w = torch.randn(384, 512, generator=g, device=DEV) * 0.02
    lin = Linear.from_dense(w, Format.FP8_CHANNEL)
    y = ops.linear(lin, x)
    torch.cuda.synchronize()
    want = lin.ref(x, torch.float32)
    mx, rel = _report("gemm_fp8_channel", y, want)
    assert rel < 0.02


def test_rmsnorm_and_quant(ops):
    g = torch.Generator(device=DEV).manual_seed(5)
    T, H = 67, 4096
    x = torch.randn(T, H, generator=g, device=DEV).bfloat16()
    res = torch.randn(T, H, generator=g, device=DEV).bfloat16()
    w = (1 + 0.1 * torch.randn(H, generator=g, device=DEV)).bfloat16()
    want, want_res = ref.rmsnorm(x, w, 1e-6, res)
    r2 = res.clone()
    y, nr = ops.norm(x, r2, w, 1e-6)
    assert torch.equal(nr, want_res)
    assert (y.float() - want.float()).abs().max().item() <= 0.03
    # quantised output feeds an NVFP4 GEMM
    lin = Linear.from_dense(torch.randn(256, H, generator=g, device=DEV) * 0.02, Format.NVFP4)
    r3 = res.clone()
    qa, _ = ops.norm(x, r3, w, 1e-6, quant_for=lin)
    sfx = quant.unswizzle_sf_128x4(qa.sf, T, H // 16).view(torch.float8_e4m3fn)
    xd = quant.nvfp4_dequantize(qa.data, sfx, qa.row_scale)
    p, sf, gs = quant.nvfp4_quantize(want, per_row=True)
    xr = quant.nvfp4_dequantize(p, sf, gs)
    # the kernel's normed row can differ from the oracle's by one bf16 ulp, which moves the row scale; what must
    # hold is that the kernel's quantisation error is no worse than the reference quantiser's
    err_k = (xd - want.float()).abs().mean().item()
    err_r = (xr - want.float()).abs().mean().item()
    print(f"[rmsnorm_quant] mean abs quantisation error: kernel {err_k:.5f} reference {err_r:.5f}")
    assert err_k < 1.05 * err_r + 1e-4


def test_swiglu(ops):
    g = torch.Generator(device=DEV).manual_seed(6)
    gu = torch.randn(33, 2 * 1536, generator=g, device=DEV).bfloat16()
    y = ops.silu_mul(gu)
    want = ref.silu_mul(gu)
    assert (y.float() - want.float()).abs().max().item() < 0.02
    lin = Linear.from_dense(torch.randn(128, 1536, generator=g, device=DEV) * 0.02, Format.MXFP8)
    qa = ops.silu_mul(gu, quant_for=lin)
    sfx = quant.unswizzle_sf_128x4(qa.sf, 33, 1536 // 32)
    xd = quant.mxfp8_dequantize(qa.data.view(torch.float8_e4m3fn), sfx)
    assert (xd - want.float()).abs().mean().item() < 0.03


def test_argmax_embed(ops):
    g = torch.Generator(device=DEV).manual_seed(7)
    logits = torch.randn(9, 151936, generator=g, device=DEV)
    logits[3, 100] = logits[3, 5000] = 50.0
    ids = ops.argmax(logits)
    assert torch.equal(ids.cpu(), ref.argmax_lowest(logits).cpu())
    table = torch.randn(1000, 256, generator=g, device=DEV).bfloat16()
    toks = torch.randint(0, 1000, (40,), generator=g, device=DEV, dtype=torch.int32)
    assert torch.equal(ops.embed(table, toks), table[toks.long()])


class _A:
    pass


def _attention_case(ops, Hq, Hkv, ctxs, qlens, seed=8, rotate=False, parents=None, D=128, splits=0):
    """Write random K/V through the prep kernel, then compare attention with the oracle over the same FP8 cache."""
    from blaze_b200.batch import SeqChunk, build_batch
    from blaze_b200.config import ModelConfig, RopeConfig, inv_freq
    cfg = ModelConfig(hidden_size=Hq * D, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, num_layers=1, rope=RopeConfig(theta=1e6))
    cfg.layer_types = ["full_attention"]
    g = torch.Generator(device=DEV).manual_seed(seed)
    B = len(ctxs)
    max_pages = (max(ctxs) + 15) // 16 + 1
    kv = KVCache(cfg, 1 + B * max_pages, B, max_pages, "fp8", DEV, "umma")
    perm = torch.randperm(B * max_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    for b in range(B):
        kv.set_pages(b, [1 + p for p in perm[b * max_pages:(b + 1) * max_pages]])
    model = _A()
    model.cfg = cfg
    model.inv_freq = torch.tensor(inv_freq(cfg), dtype=torch.float32, device=DEV)
    model.rope_scale = 1.0
    model.kv_rotate = rotate
    attn = _A()
    attn.heads, attn.kv_heads = Hq, Hkv
    attn.q_norm = (1 + 0.1 * torch.randn(D, generator=g, device=DEV)).bfloat16()
    attn.k_norm = (1 + 0.1 * torch.randn(D, generator=g, device=DEV)).bfloat16()
    tpb = 128 // (Hq // Hkv)
    # step 1: prefill everything but the last qlen tokens (fills the cache); step 2: the rows under test
    outs = {}
    for phase in (0, 1):
        chunks = []
        for b in range(B):
            pre = ctxs[b] - qlens[b]
            if phase == 0 and pre > 0:
                chunks.append(SeqChunk(b, [0] * pre, 0))
            elif phase == 1:
                chunks.append(SeqChunk(b, [0] * qlens[b], pre, parents=parents[b] if parents else None))
        if not chunks:
            continue
        batch = build_batch(chunks, kv.block_table_host, DEV, attn_group=Hq // Hkv, all_items=D != 128)
        T = batch.num_rows
        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, generator=g, device=DEV).bfloat16()
        q, _ = ops.attn_prep_store(qkv, attn, model, batch, kv, 0, None)
        # oracle prep on the same inputs
        cos, sin = ref.rope_cos_sin(batch.positions, model.inv_freq)
        qr, kr, vr, _ = ref.attn_prep(qkv, Hq, Hkv, D, attn.q_norm, attn.k_norm, 1e-6, cos, sin, rotate=rotate)
        assert (q.float() - qr.float()).abs().max().item() < 0.07
        if phase == 1:
            o = ops.attention(q, model, batch, kv, 0, D ** -0.5, splits=splits)
            torch.cuda.synchronize()
            assert ops.take_status() == 0
            kl, vl = kv.logical_kv(0)
            want = ref.paged_attention(qr, kl, vl, kv.block_table, batch.h_slots, batch.h_q_start, batch.h_ctx_len, D ** -0.5,
                                       tree_mask=batch.tree_mask)
            outs = (o.view(T, Hq, D), want)
            # the cache itself: the newest token of sequence 0 must round-trip
            s0 = chunks[0]
            pos = s0.start_pos + len(s0.tokens) - 1
            page = kv.block_table_host[s0.slot, pos // 16]
            row = batch.h_q_start[1] - 1
            kc = kl[page, :, pos % 16].float()
            assert (kc - kr[row].float()).abs().max().item() <= 0.07 * kr[row].float().abs().max().item() + 0.02
    return outs


@pytest.mark.parametrize("Hq,Hkv,ctxs,qlens", [
    (8, 2, [40], [1]),
    (32, 8, [1024, 300, 129, 17], [1, 1, 1, 1]),
    (16, 2, [513, 100, 31], [1, 1, 1]),      # plain decode at group 8 (8 rows per KV head)
    (8, 2, [200, 96], [200, 96]),            # pure prefill
    (8, 1, [700, 64, 333], [5, 64, 77]),     # verify rows + chunked prefill with history
    (4, 4, [300], [150]),                    # MHA (group 1)
])
def test_attention(ops, Hq, Hkv, ctxs, qlens):
    o, want = _attention_case(ops, Hq, Hkv, ctxs, qlens)
    mx, rel = _report(f"attention Hq{Hq} Hkv{Hkv} ctx{ctxs} q{qlens}", o, want)
    assert rel < 0.06
    assert torch.isfinite(o.float()).all()


@pytest.mark.parametrize("Hq,Hkv,ctxs,qlens", [
    (16, 2, [513, 100, 31], [1, 1, 1]),      # decode rows through the row-block kernel (group 8)
    (8, 2, [200, 96], [200, 96]),            # pure prefill
    (8, 1, [700, 64, 333], [5, 64, 77]),     # verify rows + chunked prefill with history
    (4, 4, [300], [150]),                    # MHA (group 1): more than one row block per sequence
    (16, 2, [2000, 1500, 40], [1, 1, 1]),    # few items: the KV range is split and merged
])
def test_attention_head_dim_256(ops, Hq, Hkv, ctxs, qlens):
    """head_dim 256 (two accumulator warpgroups, one 256-column output accumulator in tensor memory)."""
    o, want = _attention_case(ops, Hq, Hkv, ctxs, qlens, D=256)
    mx, rel = _report(f"attention D256 Hq{Hq} Hkv{Hkv} ctx{ctxs} q{qlens}", o, want)
    assert rel < 0.06
    assert torch.isfinite(o.float()).all()


@pytest.mark.parametrize("Hq,Hkv,q,splits", [(32, 8, 5, 1), (32, 8, 5, 3), (64, 8, 5, 1), (32, 8, 4, 1), (16, 2, 8, 1), (32, 8, 2, 1),
                                             (32, 8, 1, 1), (32, 8, 1, 2), (32, 8, 1, 3), (32, 8, 1, 5), (32, 8, 1, 8),
                                             (64, 8, 1, 3), (32, 8, 4, 3), (32, 8, 2, 3)])
def test_attention_verify_rows_without_kv_split(ops, Hq, Hkv, q, splits):
    """Chain-verify rows (a few query rows per sequence, several 16-row blocks per KV head) with the KV range in ONE piece,
    as a large batch runs them, and with a forced split: both must match the oracle row by row, later chain rows included."""
    ctxs = [700, 64, 333, 1024, 129, 17, 500, 260, 1030, 1089, 1153, 385]
    o, want = _attention_case(ops, Hq, Hkv, ctxs, [q] * len(ctxs), splits=splits)
    T = o.shape[0]
    err = (o.float() - want.float()).abs().amax(dim=(1, 2)).view(len(ctxs), q)
    print(f"[attention verify rows Hq{Hq} Hkv{Hkv} q{q} splits{splits}] max error by chain row: {err.amax(0).tolist()}")
    mx, rel = _report("attention verify rows", o, want)
    assert rel < 0.06
    ref_mag = want.float().abs().amax().item()
    assert err.max().item() < 0.25 * ref_mag, "a chain row is off by more than rounding"


def test_attention_rotated_keys(ops):
    """With the Hadamard rotation of q and k on, the prep kernel matches the rotated oracle, and the attention output
    stays the output without rotation up to the rounding of the FP8 keys."""
    o, want = _attention_case(ops, 32, 8, [1024, 300, 129, 17], [1, 1, 1, 1], rotate=True)
    _, rel = _report("attention rotated q/k vs rotated oracle", o, want)
    assert rel < 0.06
    plain, _ = _attention_case(ops, 32, 8, [1024, 300, 129, 17], [1, 1, 1, 1], rotate=False)
    _, rel = _report("attention rotated q/k vs unrotated kernel", o, plain)
    assert rel < 0.08


def test_attention_split_kv(ops):
    o, want = _attention_case(ops, 8, 2, [2000, 1500], [1, 1])
    mx, rel = _report("attention split-kv", o, want)
    assert rel < 0.06


def _experts(n, H, I, fmt, seed):
    from blaze_b200.models.qwen3 import Experts
    g = torch.Generator(device=DEV).manual_seed(seed)
    ex = Experts()
    ex.num_experts, ex.first, ex.count = n, 0, n
    for _ in range(n):
        ex.gate_up.append(Linear.from_dense(torch.randn(2 * I, H, generator=g, device=DEV) * 0.05, fmt, segments=[I, I]))
        ex.down.append(Linear.from_dense(torch.randn(H, I, generator=g, device=DEV) * 0.05, fmt))
    return ex


@pytest.mark.parametrize("fmt,T,E,k", [(Format.DENSE, 37, 8, 2), (Format.NVFP4, 200, 16, 4), (Format.MXFP8, 64, 8, 8)])
def test_moe_routed_experts(ops, fmt, T, E, k):
    H, I = 512, 256
    ex = _experts(E, H, I, fmt, 21)
    g = torch.Generator(device=DEV).manual_seed(22)
    x = torch.randn(T, H, generator=g, device=DEV).bfloat16()
    logits = torch.randn(T, E, generator=g, device=DEV)
    w, ids = ops.router_topk(logits, k, True, 0, E)
    wr, idr = ref.router_topk(logits, k, True)
    assert torch.equal(ids.cpu(), idr.cpu())
    assert torch.allclose(w, wr, atol=1e-5)
    y = ops.moe(x, w, ids, ex)
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    want = ref.moe_forward(x, wr, idr, ex.forward_one, E)
    mx, rel = _report(f"moe {fmt.value} T{T} E{E} k{k}", y, want)
    assert rel < (0.02 if fmt == Format.DENSE else 0.08)


@pytest.mark.parametrize("fmt,T,E,k", [(Format.DENSE, 37, 8, 2), (Format.NVFP4, 200, 16, 4), (Format.MXFP8, 64, 8, 8),
                                       (Format.NVFP4, 256, 32, 8), (Format.NVFP4, 3, 16, 4), (Format.NVFP4, 700, 4, 2)])
def test_moe_narrow_expert_gemm(ops, fmt, T, E, k):
    """Decode-sized routing: expert GEMMs with the features on the tensor-core lanes and only the live rows of every 128-row
    tile as columns (32 .. 128), padding rows skipped by the activation kernel.  Same result as the padded grouped GEMM (the
    products are the same, only the tile orientation differs) and as the oracle; experts with no row, with more than 128
    rows (several tiles) and with row counts that are not multiples of 32 all occur."""
    H, I = 512, 256
    ex = _experts(E, H, I, fmt, 23)
    g = torch.Generator(device=DEV).manual_seed(24)
    x = torch.randn(T, H, generator=g, device=DEV).bfloat16()
    logits = torch.randn(T, E, generator=g, device=DEV)
    logits[:, 1] -= 30.0                                   # expert 1 is never chosen
    keep = ops.MOE_NARROW_ROWS
    try:
        ops.MOE_NARROW_ROWS = 0
        w, ids = ops.router_topk(logits, k, True, 0, E)
        wide = ops.moe(x, w, ids, ex)
        ops.MOE_NARROW_ROWS = 1 << 20
        w, ids = ops.router_topk(logits, k, True, 0, E)
        l0 = ops.launches
        narrow = ops.moe(x, w, ids, ex)
        used = ops.launches - l0
    finally:
        ops.MOE_NARROW_ROWS = keep
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    wr, idr = ref.router_topk(logits, k, True)
    want = ref.moe_forward(x, wr, idr, ex.forward_one, E)
    _, rel = _report(f"moe narrow {fmt.value} T{T} E{E} k{k} vs oracle ({used} launches)", narrow, want)
    assert rel < (0.02 if fmt == Format.DENSE else 0.08)
    _, rel = _report("moe narrow vs padded grouped GEMM", narrow, wide)
    assert rel < 5e-3
    assert torch.isfinite(narrow.float()).all()


def test_moe_expert_parallel_partials_sum_to_full(ops):
    H, I, E, k, T = 512, 256, 8, 2, 50
    full = _experts(E, H, I, Format.DENSE, 31)
    g = torch.Generator(device=DEV).manual_seed(32)
    x = torch.randn(T, H, generator=g, device=DEV).bfloat16()
    logits = torch.randn(T, E, generator=g, device=DEV)
    from blaze_b200.models.qwen3 import Experts
    total = torch.zeros(T, H, device=DEV)
    for r in range(2):
        part = Experts()
        part.num_experts, part.first, part.count = E, r * 4, 4
        part.gate_up, part.down = full.gate_up[r * 4:r * 4 + 4], full.down[r * 4:r * 4 + 4]
        w, ids = ops.router_topk(logits, k, True, part.first, part.count)
        total += ops.moe(x, w, ids, part).float()
    wr, idr = ref.router_topk(logits, k, True)
    want = ref.moe_forward(x, wr, idr, full.forward_one, E)
    mx, rel = _report("moe expert-parallel partial sums", total, want)
    assert rel < 0.03


def test_gdn_layer(ops):
    from blaze_b200.batch import SeqChunk, build_batch
    from blaze_b200.config import named_config
    from blaze_b200.ops.ref_ops import RefOps
    cfg = named_config("qwen3-next-80b-a3b")
    cfg.linear_num_key_heads, cfg.linear_num_value_heads = 2, 4
    cfg.num_layers, cfg.layer_types = 1, ["linear_attention"]
    hk, hv, dk, dv = 2, 4, 128, 128
    g = torch.Generator(device=DEV).manual_seed(41)

    class G:
        pass
    gd = G()
    gd.k_heads, gd.v_heads = hk, hv
    C = 2 * hk * dk + hv * dv
    gd.conv_w = (torch.randn(C, 4, generator=g, device=DEV) * 0.3).bfloat16()
    gd.A_log = torch.log(torch.linspace(1, 4, hv, device=DEV))
    gd.dt_bias = torch.randn(hv, generator=g, device=DEV) * 0.1
    gd.norm_w = (1 + 0.1 * torch.randn(dv, generator=g, device=DEV)).bfloat16()

    class M:
        pass
    m = M()
    m.cfg, m.gdn_chunked = cfg, False
    outs = {}
    for name, o in (("cuda", ops), ("ref", RefOps())):
        kv = KVCache(cfg, 4, 4, 8, "bf16", DEV, "logical")
        gi = torch.Generator(device=DEV).manual_seed(42)
        res = []
        for step, lens in enumerate(([40, 7], [1, 1], [3, 1])):       # prefill, decode, verify-like rows
            chunks = []
            for b, n in enumerate(lens):
                done = sum(l[b] for l in ([40, 7], [1, 1], [3, 1])[:step])
                chunks.append(SeqChunk(b, [0] * n, done))
            batch = build_batch(chunks, kv.block_table_host, DEV)
            T = batch.num_rows
            mixed = torch.randn(T, C, generator=gi, device=DEV).bfloat16()
            z = torch.randn(T, hv * dv, generator=gi, device=DEV).bfloat16()
            bb = torch.randn(T, hv, generator=gi, device=DEV).bfloat16()
            aa = torch.randn(T, hv, generator=gi, device=DEV).bfloat16()
            res.append(o.gdn(mixed, z, bb, aa, gd, m, batch, kv, 0).float())
        outs[name] = (torch.cat(res), kv.rec_state[0].clone(), kv.conv_state[0].float().clone())
    torch.cuda.synchronize()
    mx, rel = _report("gdn layer output", outs["cuda"][0], outs["ref"][0])
    assert rel < 0.03
    assert (outs["cuda"][1] - outs["ref"][1]).abs().max().item() < 0.05
    assert (outs["cuda"][2] - outs["ref"][2]).abs().max().item() < 0.02


@pytest.mark.parametrize("decay_scale", [1.0, 0.1])
def test_gdn_chunked_kernel_matches_the_recurrence(ops, decay_scale):
    """The chunked tensor-core form of the gated delta rule (128-token chunks, WY / UT transform, state carried in tensor
    memory), as one fused kernel and as chunk-parallel preparation + sequential scan, against the token-by-token kernel on the same inputs: 4096-token and ragged prompts, then a second step that
    starts from the state the first one left (a 300-token continuation next to a decode row), outputs and final states."""
    from blaze_b200.batch import SeqChunk, build_batch
    from blaze_b200.config import named_config
    cfg = named_config("qwen3-next-80b-a3b")
    cfg.linear_num_key_heads, cfg.linear_num_value_heads = 2, 4
    cfg.num_layers, cfg.layer_types = 1, ["linear_attention"]
    hk, hv, dk, dv = 2, 4, 128, 128
    g = torch.Generator(device=DEV).manual_seed(43)

    class G:
        pass
    gd = G()
    gd.k_heads, gd.v_heads = hk, hv
    C = 2 * hk * dk + hv * dv
    gd.conv_w = (torch.randn(C, 4, generator=g, device=DEV) * 0.3).bfloat16()
    gd.A_log = torch.log(torch.linspace(1, 4, hv, device=DEV) * decay_scale)        # strong and weak decay per token
    gd.dt_bias = torch.randn(hv, generator=g, device=DEV) * 0.1
    gd.norm_w = (1 + 0.1 * torch.randn(dv, generator=g, device=DEV)).bfloat16()

    class M:
        pass
    m = M()
    m.cfg, m.gdn_chunked = cfg, False
    steps = ([4096, 200, 5, 129], [300, 64, 1, 128])
    outs = {}
    keep = ops.GDN_CHUNK_MIN, ops.GDN_SPLIT
    try:
        for name, chunk_min, split in (("chunked", 64, False), ("split", 64, True), ("recurrent", 0, False)):
            ops.GDN_CHUNK_MIN, ops.GDN_SPLIT = chunk_min, split
            kv = KVCache(cfg, 4, 4, 320, "bf16", DEV, "logical")
            gi = torch.Generator(device=DEV).manual_seed(44)
            res = []
            for step, lens in enumerate(steps):
                chunks = [SeqChunk(b, [0] * n, sum(l[b] for l in steps[:step])) for b, n in enumerate(lens)]
                batch = build_batch(chunks, kv.block_table_host, DEV)
                T = batch.num_rows
                mixed = torch.randn(T, C, generator=gi, device=DEV).bfloat16()
                z = torch.randn(T, hv * dv, generator=gi, device=DEV).bfloat16()
                bb = torch.randn(T, hv, generator=gi, device=DEV).bfloat16()
                aa = torch.randn(T, hv, generator=gi, device=DEV).bfloat16()
                l0 = ops.launches
                res.append(ops.gdn(mixed, z, bb, aa, gd, m, batch, kv, 0).float())
                if name != "recurrent":
                    # conv, chunked rule (one kernel, or preparation + scan), token-by-token rule for the short rows, gated norm
                    assert ops.launches - l0 == (5 if split else 4)
            outs[name] = (torch.cat(res), kv.rec_state[0].clone())
    finally:
        ops.GDN_CHUNK_MIN, ops.GDN_SPLIT = keep
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    for name in ("chunked", "split"):
        assert torch.isfinite(outs[name][0]).all()
        _, rel = _report(f"gdn {name} vs recurrent, output (decay x{decay_scale})", outs[name][0], outs["recurrent"][0])
        assert rel < 0.02
        _, rel = _report(f"gdn {name} vs recurrent, final state", outs[name][1], outs["recurrent"][1])
        assert rel < 0.02


def test_host_kv_tier_roundtrip_on_device():
    """Spill a set of FP8 pages to pinned host memory and restore them into other pages: bytes come back identical."""
    from blaze_b200.config import ModelConfig, RopeConfig
    from blaze_b200.kv import KVCache
    from blaze_b200.kv_host import HostKVTier
    cfg = ModelConfig(hidden_size=512, num_heads=4, num_kv_heads=2, head_dim=128, num_layers=2, rope=RopeConfig(theta=1e6))
    cfg.layer_types = ["full_attention"] * 2
    kv = KVCache(cfg, 64, 4, 16, "fp8", "cuda", "umma")
    for i in kv.attn_layers:
        kv.kv[i].copy_(torch.randint(0, 255, kv.kv[i].shape, dtype=torch.uint8, device=DEV))
    tier = HostKVTier(kv, 32)
    src = [3, 9, 17, 4, 40]
    want = {i: kv.kv[i][src].clone() for i in kv.attn_layers}
    run = tier.spill(src)
    assert run is not None and tier.free_pages == 32 - 5
    for i in kv.attn_layers:
        kv.kv[i][src] = 0
    dst = [50, 51, 7, 8, 60]
    tier.restore(run, dst)
    torch.cuda.synchronize()
    for i in kv.attn_layers:
        assert torch.equal(kv.kv[i][dst], want[i])
    tier.drop(run)
    assert tier.free_pages == 32 and tier.free == [(0, 32)]


@pytest.mark.parametrize("fmt,M,N,K", [("bf16", 256, 5000, 512), ("bf16", 3, 1000, 256), ("nvfp4", 130, 2048, 1024)])
def test_head_argmax_in_the_gemm_epilogue(ops, fmt, M, N, K):
    g = torch.Generator(device=DEV).manual_seed(24)
    x = (torch.randn(M, K, generator=g, device=DEV)).bfloat16()
    w = torch.randn(N, K, generator=g, device=DEV) * 0.05
    w[7] = w[3]                                     # an exact tie between two columns: the lower one must win
    lin = Linear.from_dense(w, {"bf16": Format.DENSE, "nvfp4": Format.NVFP4}[fmt])
    logits = ops.linear(lin, x, out_dtype=torch.float32, wide=False)
    want_i, want_v = ops.argmax(logits, index_offset=11, want_values=True)
    got_i, got_v = ops.linear_argmax(lin, x, index_offset=11, want_values=True)
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    assert torch.equal(got_i, want_i) and torch.equal(got_v, want_v)
    assert torch.equal(ops.linear_argmax(lin, x), want_i - 11)


def test_autotuner_routes_linear_layers(ops, tmp_path, monkeypatch):
    """The tuner times the kernel variants of a layer shape, keeps the winner in its JSON cache, and ``CudaOps.linear`` follows
    the table; a second tuner instance reads the cache instead of timing again."""
    from blaze_b200 import tune
    g = torch.Generator(device=DEV).manual_seed(41)
    lin = Linear.from_dense(torch.randn(512, 8192, generator=g, device=DEV) * 0.02, Format.NVFP4)
    x = torch.randn(256, 8192, generator=g, device=DEV).bfloat16()
    t = tune.Tuning(str(tmp_path / "tune.json"))
    best = tune.tune_linear(ops, lin, 256, t, iters=3)
    assert best["kernel"] in ("tc", "sk") and best["ms"] > 0
    t.save()
    t2 = tune.Tuning(str(tmp_path / "tune.json"))
    assert t2.get("gemm1", 512, 8192, 256) == best
    want = ops.linear(lin, x, wide=False, sk=False)
    ops.tuning = t2
    try:
        l0 = ops.launches
        got = ops.linear(lin, x)
        assert ops.launches == l0 + 2                    # activation quantisation + one GEMM, whichever kernel was chosen
    finally:
        ops.tuning = None
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    _, rel = _report("tuned route vs one-CTA-per-tile kernel", got, want.float())
    assert rel < 2e-3


@pytest.mark.parametrize("D,rot,gated", [(128, 128, False), (256, 64, True), (64, 64, False)])
def test_attn_prep_mrope_positions(ops, D, rot, gated):
    """q/k-norm + rotary + page write with three position streams (M-RoPE): every frequency follows the stream its section
    names; also head_dim 256 with partial rotary and the output gate split (the Qwen3-Next attention shape)."""
    from blaze_b200.batch import SeqChunk, build_batch
    from blaze_b200.config import ModelConfig, RopeConfig, inv_freq
    Hq, Hkv, T = 4, 2, 37
    half = rot // 2
    sec = [half // 4, half // 4 + 2, half - (half // 4) * 2 - 2]
    cfg = ModelConfig(hidden_size=Hq * D, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, num_layers=1, attn_output_gate=gated,
                      rope=RopeConfig(theta=1e6, partial_rotary_factor=rot / D, mrope_section=sec))
    cfg.layer_types = ["full_attention"]
    g = torch.Generator(device=DEV).manual_seed(51)
    kv = KVCache(cfg, 8, 1, 4, "fp8", DEV, "umma")
    kv.set_pages(0, [3, 1, 5])
    p3 = torch.stack([torch.arange(T), torch.randint(0, 50, (T,)), torch.randint(0, 50, (T,))]).tolist()
    batch = build_batch([SeqChunk(0, [0] * T, 0, pos3=p3)], kv.block_table_host, DEV, attn_group=Hq // Hkv)
    assert batch.positions3 is not None and batch.positions3.shape == (3, T)
    model = _A()
    model.cfg = cfg
    model.inv_freq = torch.tensor(inv_freq(cfg), dtype=torch.float32, device=DEV)
    model.rope_scale, model.kv_rotate = 1.0, False
    attn = _A()
    attn.heads, attn.kv_heads = Hq, Hkv
    attn.q_norm = (1 + 0.1 * torch.randn(D, generator=g, device=DEV)).bfloat16()
    attn.k_norm = (1 + 0.1 * torch.randn(D, generator=g, device=DEV)).bfloat16()
    qkv = torch.randn(T, (Hq * (2 if gated else 1) + 2 * Hkv) * D, generator=g, device=DEV).bfloat16()
    q, gate = ops.attn_prep_store(qkv, attn, model, batch, kv, 0, None)
    cos, sin = ref.rope_cos_sin(batch.positions3, model.inv_freq, 1.0, sec)
    qr, kr, vr, gr = ref.attn_prep(qkv, Hq, Hkv, D, attn.q_norm, attn.k_norm, 1e-6, cos, sin, gated=gated)
    torch.cuda.synchronize()
    assert (q.float() - qr.float()).abs().max().item() < 0.07
    if gated:
        assert torch.equal(gate.view(T, Hq, D), gr.view(T, Hq, D).to(gate.dtype))
    # with one stream only the result must differ (the sections are really used)
    cos1, sin1 = ref.rope_cos_sin(batch.positions, model.inv_freq)
    q1, _, _, _ = ref.attn_prep(qkv, Hq, Hkv, D, attn.q_norm, attn.k_norm, 1e-6, cos1, sin1, gated=gated)
    assert (q.float() - q1.float()).abs().max().item() > 0.2
    kl, vl = kv.logical_kv(0)
    page, off = kv.block_table_host[0, (T - 1) // 16], (T - 1) % 16
    assert (kl[page, :, off].float() - kr[T - 1].float()).abs().max().item() <= 0.07 * kr[T - 1].float().abs().max().item() + 0.02
