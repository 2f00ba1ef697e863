// Exact FP8 GEMM for checkpoints with 128x128 fp32 weight block scales and 1x128 fp32 activation group scales:
//     C[m, n] = sum_kb  sa[kb, m] * sb[n / 128, kb] * ( A8[m, kb*128 : kb*128+128] . B8[n, kb*128 : kb*128+128] )  (+ bias[n])
// A8 / B8 are e4m3.  The hardware block-scaled MMA modes only take power-of-two (e8m0) scales per 32 elements, so a
// checkpoint's fp32 block scales cannot ride along with the operands.  Instead every 128-deep K block is multiplied on
// the tensor cores into its own TMEM accumulator (tcgen05.mma kind::f8f6f4, fp32 accumulate, overwrite mode), and the
// epilogue warps promote it: read the 128x128 partial from TMEM, multiply by the block's (row scale x tile scale)
// and add it to fp32 accumulators held in registers (64 per thread: one output row, 64 columns).  Two TMEM buffers
// take turns, so the tensor cores compute block kb+1 while block kb is being promoted (four buffers measured the same; so
// did polling instead of the suspended barrier wait, which was slower: the spinning warps take issue slots): per block the MMA needs about
// 256 cycles and the promotion (split over eight warps) about 100 of issue plus its TMEM load latency.
//
// 320 threads: warp 0 = TMA producer (one 128-byte-swizzled 128x128 e4m3 tile of A and of B per stage, 6 stages), warp 1
// = MMA issuer, warps 2-9 = promotion + store: two warps per TMEM lane quadrant, each owning 64 of the 128 columns, so that
// every scheduler has two promotion warps and the latency of one warp's TMEM loads hides behind the other's FMAs (with one
// warp per scheduler the tensor pipe sat at 32 % and the FMA pipe at 19 %).  Every wait is a bounded mbarrier wait that
// reports through the status word.  No TMA load is cluster-multicast.
//
// Reference counterpart: the FP8 block-scale linear of kernels/src/cuda/fp8_linear.cu (fp8_block_* kernels: dequantise to
// bf16 and run a bf16 GEMM, or 1x128-quantised activations with per-block fp32 rescale on mma.sync), routed from
// crates/blaze/src/linear.rs (Fp8Block variants).
#include "blaze/host.h"
#include "blaze/sm100.cuh"

namespace blz {

struct FbParams {
  int M, N, K;
  void* C;                   // bf16 or fp32 [M, N]
  long long ldc;             // elements
  int out_f32;
  const float* sa;           // [K / 128, ld_sa]: activation scale of (k block, row)
  long long ld_sa;
  const float* sb;           // [ceil(N / 128), K / 128]: weight scale of (n block, k block)
  const __nv_bfloat16* bias; // [N] or null
  int* status;
};

struct FbCfg {
  static constexpr int BM = 128, BN = 128, BK = 128;
  static constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK;
  static constexpr int STAGES = 6;
  static constexpr int NBUF = 2;                       // partial accumulators in flight (128 TMEM columns each)
  static constexpr int TMEM_COLS = NBUF * 128;
  static constexpr int SMEM = STAGES * (A_BYTES + B_BYTES) + 1024 /*align*/ + 256 /*barriers*/;
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
};

__global__ void __launch_bounds__(320, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, FbParams p) {
  using Cfg = FbCfg;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + STAGES * Cfg::A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + STAGES * Cfg::B_BYTES);
  uint64_t* full = bars;                      // [STAGES] operands of a k block have landed
  uint64_t* empty = bars + STAGES;            // [STAGES] the MMAs reading a stage have completed
  constexpr int NBUF = Cfg::NBUF;
  uint64_t* part_full = bars + 2 * STAGES;    // [NBUF] a k block's partial products are complete in TMEM buffer b
  uint64_t* part_empty = part_full + NBUF;    // [NBUF] the promotion warps have read buffer b (8 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(part_empty + NBUF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM;
  const int mt = blockIdx.x % tiles_m, nt = blockIdx.x / tiles_m;     // consecutive CTAs share a weight tile through L2
  const int nkb = p.K / Cfg::BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < NBUF; ++i) { mbar_init(&part_full[i], 1); mbar_init(&part_empty[i], 8); }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_trigger();        // this CTA holds its tensor memory: a dependent kernel that becomes resident cannot block it
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const int pre = min(STAGES, nkb);
      // weights do not depend on the kernel before this one: their first tiles go out before the dependency wait
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full[i], Cfg::A_BYTES + Cfg::B_BYTES);
        tma_load_2d(sB + i * Cfg::B_BYTES, &tmB, i * Cfg::BK, nt * BN, &full[i]);
      }
      pdl_wait();
      int s = 0; uint32_t ph = 0;
      for (int i = 0; i < nkb; ++i) {
        if (i >= pre) {
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status)) break;
          mbar_expect_tx(&full[s], Cfg::A_BYTES + Cfg::B_BYTES);
          tma_load_2d(sB + s * Cfg::B_BYTES, &tmB, i * Cfg::BK, nt * BN, &full[s]);
        }
        tma_load_2d(sA + s * Cfg::A_BYTES, &tmA, i * Cfg::BK, mt * BM, &full[s]);
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      int s = 0; uint32_t ph = 0;
      for (int i = 0; i < nkb; ++i) {
        const int b = i % NBUF;
        // buffer b was last filled for block i - NBUF: its promotion is completion number (i / NBUF - 1) of part_empty[b]
        if (i >= NBUF && !mbar_wait(&part_empty[b], (uint32_t)((i / NBUF - 1) & 1), abort_flag, p.status)) break;
        if (!mbar_wait(&full[s], ph, abort_flag, p.status)) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(sA + s * Cfg::A_BYTES), b_addr = smem_u32(sB + s * Cfg::B_BYTES);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          mma_f8(tmem + b * BN, desc_sw128(a_addr + j * 32), desc_sw128(b_addr + j * 32), make_idesc(0, 0, BM, BN), j > 0 ? 1u : 0u);
        mma_commit(&empty[s]);
        mma_commit(&part_full[b]);
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ promotion + store (256 threads)
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;       // which 64 columns of the tile this warp owns
    const int rl = q * 32 + lane;
    const int row = mt * BM + rl;
    const bool in_range = row < p.M;
    const float* sb = p.sb + (size_t)nt * nkb;
    constexpr int HC = BN / 2;
    float acc[HC];
#pragma unroll
    for (int i = 0; i < HC; ++i) acc[i] = 0.f;
    pdl_wait();                             // the activation scales come from the kernel before this one
    float sa_next = in_range ? p.sa[row] : 0.f;
    bool ok = true;
#pragma unroll 1
    for (int i = 0; i < nkb; ++i) {
      const int b = i % NBUF;
      const float s = sa_next * __ldg(sb + i);
      if (i + 1 < nkb) sa_next = in_range ? p.sa[(size_t)(i + 1) * p.ld_sa + row] : 0.f;
      // tcgen05.ld is warp-collective: the outcome of the wait is made warp-uniform before any lane loads
      ok = __all_sync(0xffffffffu, mbar_wait(&part_full[b], (uint32_t)((i / NBUF) & 1), abort_flag, p.status));
      if (!ok) break;
      tc_fence_after();
      const uint32_t t0 = tmem + b * BN + half * HC + ((uint32_t)(q * 32) << 16);
      uint32_t r0[32], r1[32];
      tmem_ld32(t0, r0);
      tmem_ld32(t0 + 32, r1);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        acc[j] = fmaf(__uint_as_float(r0[j]), s, acc[j]);
        acc[32 + j] = fmaf(__uint_as_float(r1[j]), s, acc[32 + j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&part_empty[b]);
    }
    if (ok && in_range) {
#pragma unroll
      for (int c = 0; c < HC / 8; ++c) {
        const int col0 = nt * BN + half * HC + c * 8;
        if (col0 >= p.N) break;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[j] = acc[c * 8 + j];
          if (p.bias && col0 + j < p.N) v[j] += bf2f(p.bias[col0 + j]);
        }
        const bool whole = col0 + 8 <= p.N;
        if (p.out_f32) {
          float* dst = reinterpret_cast<float*>(p.C) + (size_t)row * p.ldc + col0;
          if (whole && (p.ldc & 3) == 0) {
            *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (col0 + j < p.N) dst[j] = v[j];
          }
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)row * p.ldc + col0;
          if (whole && (p.ldc & 7) == 0) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                                                        pack_bf16x2(v[6], v[7]));
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (col0 + j < p.N) dst[j] = __float2bfloat16(v[j]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Activation quantiser: bf16 [T, K] -> e4m3 [T, K] with one fp32 scale per (row, 128-column group), scale = amax / 448,
// written k-block-major ([K / 128, ld_s]) so that the GEMM's promotion warps read them coalesced.  One warp per group.
__global__ void __launch_bounds__(256)
quant_fp8_block_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, float* __restrict__ scales,
                       long long ld_s, int T, int K) {
  pdl_wait();
  pdl_trigger();
  const int groups = K / 128;
  const long long g = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (g >= (long long)T * groups) return;
  const int row = (int)(g / groups), kb = (int)(g % groups);
  const int lane = threadIdx.x & 31;
  const uint2 raw = *reinterpret_cast<const uint2*>(x + (size_t)row * ldx + kb * 128 + lane * 4);
  const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  float v[4] = {__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1)};
  float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  m = warp_max(m);
  const float scale = fmaxf(m / 448.f, 1e-12f);
  uint32_t out = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(v[i] / scale, __NV_SATFINITE, __NV_E4M3);
    out |= (uint32_t)b << (8 * i);
  }
  *reinterpret_cast<uint32_t*>(q + (size_t)row * K + kb * 128 + lane * 4) = out;
  if (lane == 0) scales[(size_t)kb * ld_s + row] = scale;
}

}  // namespace blz

// A e4m3 [M, K] (lda bytes), B e4m3 [N, K] (ldb bytes), sa fp32 [K / 128, ld_sa], sb fp32 [ceil(N / 128), K / 128]; C bf16 or
// fp32 [M, N] with ldc in elements.  K must be a multiple of 128.
BLZ_API int blz_gemm_fp8_block(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc, int M, int N,
                               int K, const float* sa, long long ld_sa, const float* sb, const void* bias, int out_f32,
                               cudaStream_t stream) {
  using namespace blz;
  if (M <= 0 || N <= 0 || K <= 0 || K % 128 || !sa || !sb || ld_sa < M) return (int)cudaErrorInvalidValue;
  FbParams p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_f32 = out_f32;
  p.sa = sa; p.ld_sa = ld_sa; p.sb = sb; p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.status = status_word();
  CUtensorMap tmA, tmB;
  cudaError_t e = encode_tmap(&tmA, A, 1, (uint64_t)K, M, lda, 128, 128, 3);
  if (e != cudaSuccess) return (int)e;
  e = encode_tmap(&tmB, B, 1, (uint64_t)K, N, ldb, 128, 128, 3);
  if (e != cudaSuccess) return (int)e;
  auto kern = gemm_fp8_block_kernel;
  static PerDeviceOnce configured;
  e = configured.smem_limit(kern, FbCfg::SMEM);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(((M + 127) / 128) * ((N + 127) / 128));
  cfg.blockDim = dim3(320);
  cfg.dynamicSmemBytes = FbCfg::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return (int)cudaLaunchKernelEx(&cfg, kern, tmA, tmB, p);
}

// x bf16 [T, K] (ldx elements) -> q e4m3 [T, K] contiguous, scales fp32 [K / 128, ld_s].  K % 128 == 0, ldx % 4 == 0.
BLZ_API int blz_quant_fp8_block(const void* x, long long ldx, void* q, float* scales, long long ld_s, int T, int K,
                                cudaStream_t stream) {
  using namespace blz;
  if (T <= 0) return 0;
  if (K <= 0 || K % 128 || (ldx & 3) || ld_s < T) return (int)cudaErrorInvalidValue;
  const long long groups = (long long)T * (K / 128);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((groups + 7) / 8));
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return (int)cudaLaunchKernelEx(&cfg, quant_fp8_block_kernel, reinterpret_cast<const __nv_bfloat16*>(x), ldx,
                                 reinterpret_cast<uint8_t*>(q), scales, ld_s, T, K);
}
