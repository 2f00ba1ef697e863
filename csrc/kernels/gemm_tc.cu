// tcgen05 GEMM family:  C[M,N] = (A[M,K] · B[N,K]^T) * row_scale[m] * alpha[n] (+ bias[n])
//
//   kind 0  bf16 x bf16                      (kind::f16,  64 elements per 128-byte stage row)
//   kind 1  NVFP4 x NVFP4, e4m3 scale / 16   (kind::mxf4nvf4.block_scale.scale_vec::4X, 256 elements per row)
//   kind 2  MXFP8 x MXFP8, e8m0 scale / 32   (kind::mxf8f6f4.block_scale, 128 elements per row)
//   kind 3  e4m3 x e4m3, no block scales     (kind::f8f6f4; per-row / per-channel scales in the epilogue)
//
// One persistent CTA per SM, 192 threads: warp 0 = TMA producer, warp 1 = MMA issuer (one elected lane,
// owns the TMEM allocation), warps 2-5 = epilogue (one TMEM lane quadrant each).  Operands are staged in
// 128B-swizzled shared memory by TMA tensor loads (never multicast); scale factors arrive by 1-D bulk
// copies in the 128x4 tiled layout and are moved to tensor memory with tcgen05.cp; accumulators live in
// TMEM, double-buffered so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Covers what the reference spreads over kernels/src/cuda/nvfp4_gemm.cu (w4a4_kernel :114, sm_120a-only
// mma.sync), nvfp4_linear.cu (gemv / small-m mma kernels :49-:320), fp8_linear.cu (:40, :159, :270) and the
// cuBLAS call in gemm.cu:55.
#include "blaze/host.h"
#include "blaze/sm100.cuh"

namespace blz {

__device__ __forceinline__ long long gt_now() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define GT_STAMP(i) do { if (p.stamps) p.stamps[(size_t)blockIdx.x * 8 + (i)] = gt_now(); } while (0)

struct GemmParams {
  int M, N, K;               // K in elements
  void* C;                   // bf16 or fp32 [M, ldc]
  long long ldc;
  const float* row_scale;    // [M] or null
  const float* alpha;        // [N] or null
  const __nv_bfloat16* bias; // [N] or null
  const uint8_t* sfa;        // scale factors of A, 128x4-tiled (kinds 1, 2)
  const uint8_t* sfb;
  int sfa_col_tiles;         // number of 4-column tiles per 128-row tile in sfa / sfb
  // fused all-reduce (OUT mode 2): the epilogue adds this rank's partial tile into every rank's output through the
  // NVSwitch (multimem.red); the last CTA then meets the other ranks at a flag barrier, so kernel completion means
  // the summed output is complete in local memory.
  void* mc_out;              // multicast address of C (bf16 [M, ldc])
  unsigned* done_ctr;        // local counter of finished CTAs (returns to zero at the end of the kernel)
  uint32_t* peer_pad[8];     // one flag row per rank: pad[r][src_rank]
  uint32_t* epoch;           // local barrier epoch
  long long spin_limit;
  int rank, world;
  // fused reduce-scatter by push (push_rows_per > 0): rank o owns rows [o * push_rows_per, (o + 1) * push_rows_per) of the
  // summed output.  The epilogue stores each bf16 partial row straight into its owner's slot buffer
  // [source rank][push_rows_per][N] through peer memory; the last CTA of this rank then raises flag [source rank] on every
  // owner (release, system scope).  Nobody waits here: the owner's reduction kernel waits for its `world` flags.
  __nv_bfloat16* push_slot[8];
  uint32_t* push_flag[8];
  int push_rows_per;
  long long* stamps;         // optional diagnostics: [gridDim.x][8] global-timer stamps of the pushed epilogue (null = off)
  const int* tile_expert;    // grouped GEMM: expert of every 128-row M tile (-1 = skip); B / alpha / sfb rows are offset by expert * N
  // activations still in flight from the peers (fused all-reduce + norm that signals instead of waiting): the producer
  // sends the first weight tiles, then waits until counter[r] >= *wait_expect for every rank r, then loads A
  const uint32_t* wait_pad;  // own arrival counters, one uint32 per source rank (peers add to them)
  const uint32_t* wait_epoch;  // the count to wait for (device word, advanced by the signalling kernel)
  int wait_world;
  long long wait_limit;
  float* amax_val;           // arg-max epilogue (fp32 instantiation): per (N tile, row) best value ...
  int* amax_idx;             // ... and its column; C is not written.  Layout [N tiles][M].
  int act;                   // 1: B rows are [16 gate | 16 up] groups; the epilogue writes silu(gate) * up, bf16 [M, N/2]
  int b_kt;                  // > 0: B is tile-major, [N/128][b_kt][16 KB shared-memory image of a 128-row x 128-byte tile]
  const uint8_t* b_raw;      // base of B for the tile-major form (fetched with plain bulk copies, one per tile)
  int* status;
};

template <int KIND>
struct KindTraits;
template <> struct KindTraits<0> { static constexpr int KMMA = 16, ELEMS_PER_BYTE_X2 = 1, SF_ATOMS = 0; };
template <> struct KindTraits<1> { static constexpr int KMMA = 64, SF_ATOMS = 4; };
template <> struct KindTraits<2> { static constexpr int KMMA = 32, SF_ATOMS = 1; };
template <> struct KindTraits<3> { static constexpr int KMMA = 32, SF_ATOMS = 0; };

template <int KIND, int BN>
struct GemmCfg {
  static constexpr int BM = 128;
  static constexpr int KMMA = KindTraits<KIND>::KMMA;
  static constexpr int BK = KMMA * 4;                    // elements per stage; always 128 bytes per row
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int SF_ATOMS = KindTraits<KIND>::SF_ATOMS;   // 512-byte atoms per 128 rows per stage
  static constexpr int SFA_BYTES = SF_ATOMS * 512;
  static constexpr int SFB_BYTES = SF_ATOMS * 512 * (BN / 128);
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 5;
  static constexpr int ACC_BUFS = (BN == 256 && SF_ATOMS) ? 1 : 2;
  static constexpr int SF_COLS_PER_STAGE = SF_ATOMS * 4 * (1 + BN / 128);
  static constexpr int SF_COL0 = ACC_BUFS * BN;
  static constexpr int PUSH_ROW = 272;                                  // 256 bytes of a tile row + 16 (no bank conflicts)
  static constexpr int PUSH_STAGE = (BN == 128) ? 4 * 32 * PUSH_ROW : 0; // per-warp [32 rows] staging of the pushed epilogue
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + PUSH_STAGE;   // + 8*BN*4 static
  static_assert(SF_COL0 + STAGES * SF_COLS_PER_STAGE <= 512, "TMEM budget");
};

template <int KIND, int BN, bool OUT_F32>
__global__ void __launch_bounds__(192, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  pdl_trigger();
  using Cfg = GemmCfg<KIND, BN>;
  constexpr int BM = Cfg::BM, BK = Cfg::BK, STAGES = Cfg::STAGES, ACC = Cfg::ACC_BUFS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + STAGES * Cfg::A_BYTES;
  uint8_t* sSFA = sB + STAGES * Cfg::B_BYTES;
  uint8_t* sSFB = sSFA + STAGES * Cfg::SFA_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sSFB + STAGES * Cfg::SFB_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = acc_full + ACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + ACC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* push_stage = reinterpret_cast<uint8_t*>(bars) + 256;   // [4 warps][32 rows][PUSH_ROW bytes]
  __shared__ __align__(16) float s_alpha[4][BN];
  __shared__ __align__(16) float s_bias[4][BN];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_tiles = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < ACC; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (threadIdx.x == 0) GT_STAMP(0);

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    // what: 1 = the B tile (+ its scales) and the stage's byte count, 2 = the A tile (+ its scales), 3 = both
    auto issue = [&](int s, int mt, int nt, int ex, int kt, int what) {
      int atoms = 0;
      if constexpr (Cfg::SF_ATOMS > 0) atoms = min(Cfg::SF_ATOMS, p.sfa_col_tiles - kt * Cfg::SF_ATOMS);
      const int kc = (KIND == 0) ? kt * BK : kt * 128;   // coordinate in map elements (bf16 or bytes)
      if (what & 1) {
        uint32_t bytes = Cfg::A_BYTES + Cfg::B_BYTES;
        if constexpr (Cfg::SF_ATOMS > 0) bytes += atoms * 512 * (1 + BN / 128);
        mbar_expect_tx(&full[s], bytes);
        const int brow = ex * p.N + nt * BN;                  // first B row of this tile
        if (p.b_kt > 0) {
          // tile-major weights: every 128-row x 128-byte tile is stored as its swizzled shared-memory image, one
          // contiguous 16 KB run that a single bulk copy brings in
#pragma unroll
          for (int h = 0; h < BN / 128; ++h)
            bulk_load(sB + s * Cfg::B_BYTES + h * 16384,
                      p.b_raw + ((size_t)(nt * (BN / 128) + h) * p.b_kt + kt) * 16384, 16384, &full[s]);
        } else {
          tma_load_2d(sB + s * Cfg::B_BYTES, &tmB, kc, brow, &full[s]);
        }
        if constexpr (Cfg::SF_ATOMS > 0) {
#pragma unroll
          for (int h = 0; h < BN / 128; ++h) {
            const size_t b_off = ((size_t)(brow / 128 + h) * p.sfa_col_tiles + (size_t)kt * Cfg::SF_ATOMS) * 512;
            bulk_load(sSFB + s * Cfg::SFB_BYTES + h * Cfg::SFA_BYTES, p.sfb + b_off, atoms * 512, &full[s]);
          }
        }
      }
      if (what & 2) {
        tma_load_2d(sA + s * Cfg::A_BYTES, &tmA, kc, mt * BM, &full[s]);
        if constexpr (Cfg::SF_ATOMS > 0) {
          const size_t a_off = ((size_t)mt * p.sfa_col_tiles + (size_t)kt * Cfg::SF_ATOMS) * 512;
          bulk_load(sSFA + s * Cfg::SFA_BYTES, p.sfa + a_off, atoms * 512, &full[s]);
        }
      }
    };
    // The weights do not depend on the kernel before this one: the first tile's B stages go out first, then the producer
    // waits for that kernel (and, when armed, for the peers' arrival counters), then it loads the activations.
    int pre = 0;
    bool go = true;
    if (lane == 0 && (int)blockIdx.x < num_tiles && !p.tile_expert) {
      pre = min(STAGES, k_tiles);
      const int t = blockIdx.x;
      for (int kt = 0; kt < pre; ++kt) issue(kt, t % tiles_m, t / tiles_m, 0, kt, 1);
    }
    pre = __shfl_sync(0xffffffffu, pre, 0);
    pdl_wait();
    if (p.wait_pad != nullptr) {
      if (lane < p.wait_world) {
        const uint32_t want = *p.wait_epoch;
        const uint32_t* f = p.wait_pad + lane;
        const long long t0 = clock64();
        while (true) {
          uint32_t v;
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
          if ((int32_t)(v - want) >= 0) break;
          if (clock64() - t0 > p.wait_limit) { atomicCAS(p.status, kOk, kErrFlagTimeout); go = false; break; }
        }
      }
      __syncwarp();
      // the A tiles are fetched by the async proxy: order those reads after the flag observation
      if (lane == 0) asm volatile("fence.proxy.async;" ::: "memory");
      go = __all_sync(0xffffffffu, go);
      if (!go && lane == 0) *abort_flag = 1;
    }
    if (lane == 0 && go) {
      int s = 0; uint32_t ph = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        const int mt = t % tiles_m, nt = t / tiles_m;
        const int ex = p.tile_expert ? p.tile_expert[mt] : 0;
        if (ex < 0) continue;
        for (int kt = 0; kt < k_tiles; ++kt) {
          if (t == (int)blockIdx.x && kt < pre) {
            issue(s, mt, nt, ex, kt, 2);             // its weights are already on their way
          } else {
            if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status)) goto producer_done;
            issue(s, mt, nt, ex, kt, 3);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    producer_done:;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    pdl_wait();
    if (elect_one()) {
      int s = 0; uint32_t ph = 0;
      int it = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        if (p.tile_expert && p.tile_expert[t % tiles_m] < 0) continue;
        const int ab = it % ACC;
        const uint32_t aph = (it / ACC) & 1;
        ++it;
        if (!mbar_wait(&acc_empty[ab], aph ^ 1, abort_flag, p.status)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem + ab * BN;
        bool ok = true;
        for (int kt = 0; kt < k_tiles; ++kt) {
          if (!mbar_wait(&full[s], ph, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * Cfg::A_BYTES), b_addr = smem_u32(sB + s * Cfg::B_BYTES);
          const int nblk = min(4, (p.K - kt * BK + Cfg::KMMA - 1) / Cfg::KMMA);
          const uint32_t sf_t = tmem + Cfg::SF_COL0 + s * Cfg::SF_COLS_PER_STAGE;
          if constexpr (Cfg::SF_ATOMS > 0) {
            const int atoms = min(Cfg::SF_ATOMS, p.sfa_col_tiles - kt * Cfg::SF_ATOMS);
            for (int a = 0; a < atoms; ++a) {
              tmem_cp_sf(sf_t + a * 4, make_smem_desc(smem_u32(sSFA + s * Cfg::SFA_BYTES + a * 512), 0, 128, kSwzNone));
#pragma unroll
              for (int h = 0; h < BN / 128; ++h)
                tmem_cp_sf(sf_t + Cfg::SF_ATOMS * 4 + (a * (BN / 128) + h) * 4,
                           make_smem_desc(smem_u32(sSFB + s * Cfg::SFB_BYTES + h * Cfg::SFA_BYTES + a * 512), 0, 128, kSwzNone));
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (j < nblk) {
              const uint64_t da = desc_sw128(a_addr + j * 32), db = desc_sw128(b_addr + j * 32);
              const uint32_t acc = (kt > 0 || j > 0) ? 1u : 0u;
              if constexpr (KIND == 0) {
                mma_f16(d_tmem, da, db, make_idesc(1, 1, BM, BN), acc);
              } else if constexpr (KIND == 3) {
                mma_f8(d_tmem, da, db, make_idesc(0, 0, BM, BN), acc);
              } else if constexpr (KIND == 1) {
                mma_nvfp4(d_tmem, da, db, make_idesc_bs(1, 1, 0, BM, BN), sf_t + j * 4,
                          sf_t + Cfg::SF_ATOMS * 4 + j * 4 * (BN / 128), acc);
              } else {
                // one atom holds the scales of all four K blocks; the block is selected by the sf id
                mma_mxf8(d_tmem, da, db, make_idesc_bs(0, 0, 1, BM, BN, j, j), sf_t, sf_t + Cfg::SF_ATOMS * 4, acc);
              }
            }
          }
          mma_commit(&empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        mma_commit(&acc_full[ab]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    pdl_wait();
    const int q = warp & 3;                       // TMEM lane quadrant this warp may read
    int it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const int mt = t % tiles_m, nt = t / tiles_m;
      const int ex = p.tile_expert ? p.tile_expert[mt] : 0;
      if (ex < 0) continue;
      const int ab = it % ACC;
      const uint32_t aph = (it / ACC) & 1;
      ++it;
      // the row scale and the per-column multipliers / bias of this tile are fetched (and staged once per warp) while
      // the tile's MMAs are still running
      const int row = mt * BM + q * 32 + lane;
      const float rs = (p.row_scale && row < p.M) ? p.row_scale[row] : 1.0f;
      float* sal = s_alpha[warp - 2];
      float* sbi = s_bias[warp - 2];
      __syncwarp();
#pragma unroll
      for (int i = lane; i < BN; i += 32) {
        const int col = nt * BN + i;
        sal[i] = (p.alpha && col < p.N) ? __ldg(p.alpha + (size_t)ex * p.N + col) : 1.0f;
        sbi[i] = (p.bias && col < p.N) ? bf2f(p.bias[(size_t)ex * p.N + col]) : 0.0f;
      }
      __syncwarp();
      if (!mbar_wait(&acc_full[ab], aph, abort_flag, p.status)) break;
      tc_fence_after();
      if (threadIdx.x == 64) GT_STAMP(1);
      float best_v = -INFINITY;
      int best_i = 0x7fffffff;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem + ab * BN + c * 32 + ((uint32_t)(q * 32) << 16), r);
        tmem_ld_wait();
        const int col0 = nt * BN + c * 32;
        if (OUT_F32 && p.amax_val != nullptr) {
          // greedy head: keep the largest logit of this row within the tile (first maximum = lowest column)
          if (row < p.M && col0 < p.N) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float v = fmaf(__uint_as_float(r[i]) * rs, sal[c * 32 + i], sbi[c * 32 + i]);
              if (col0 + i < p.N && v > best_v) { best_v = v; best_i = col0 + i; }
            }
          }
          continue;
        }
        if (row < p.M && col0 < p.N) {
          // vector stores need the whole 32-column group inside N and rows that start on a 16-byte boundary
          const bool whole = col0 + 32 <= p.N && (p.ldc & (OUT_F32 ? 3 : 7)) == 0;
          if constexpr (OUT_F32) {
            float* dst = reinterpret_cast<float*>(p.C) + (size_t)row * p.ldc + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 al = *reinterpret_cast<const float4*>(sal + c * 32 + i);
              const float4 bi = *reinterpret_cast<const float4*>(sbi + c * 32 + i);
              float4 o;
              o.x = fmaf(__uint_as_float(r[i]) * rs, al.x, bi.x);
              o.y = fmaf(__uint_as_float(r[i + 1]) * rs, al.y, bi.y);
              o.z = fmaf(__uint_as_float(r[i + 2]) * rs, al.z, bi.z);
              o.w = fmaf(__uint_as_float(r[i + 3]) * rs, al.w, bi.w);
              if (whole) {
                *reinterpret_cast<float4*>(dst + i) = o;
              } else {
                if (col0 + i < p.N) dst[i] = o.x;
                if (col0 + i + 1 < p.N) dst[i + 1] = o.y;
                if (col0 + i + 2 < p.N) dst[i + 2] = o.z;
                if (col0 + i + 3 < p.N) dst[i + 3] = o.w;
              }
            }
          } else if (p.act) {
            // SwiGLU in the epilogue: columns [0,16) of the group are gate, [16,32) the matching up features
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)row * p.ldc + col0 / 2;
            uint32_t pk[8];
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              float a[2];
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                const float g = bf2f(__float2bfloat16(fmaf(__uint_as_float(r[i + j]) * rs, sal[c * 32 + i + j], sbi[c * 32 + i + j])));
                const float u = bf2f(__float2bfloat16(fmaf(__uint_as_float(r[16 + i + j]) * rs, sal[c * 32 + 16 + i + j], sbi[c * 32 + 16 + i + j])));
                a[j] = g / (1.f + __expf(-g)) * u;
              }
              pk[i / 2] = pack_bf16x2(a[0], a[1]);
            }
            if (whole) {
              *reinterpret_cast<uint4*>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              *reinterpret_cast<uint4*>(dst + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)row * p.ldc + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              const float4 a0 = *reinterpret_cast<const float4*>(sal + c * 32 + i);
              const float4 a1 = *reinterpret_cast<const float4*>(sal + c * 32 + i + 4);
              const float4 b0 = *reinterpret_cast<const float4*>(sbi + c * 32 + i);
              const float4 b1 = *reinterpret_cast<const float4*>(sbi + c * 32 + i + 4);
              const float o0 = fmaf(__uint_as_float(r[i]) * rs, a0.x, b0.x), o1 = fmaf(__uint_as_float(r[i + 1]) * rs, a0.y, b0.y);
              const float o2 = fmaf(__uint_as_float(r[i + 2]) * rs, a0.z, b0.z), o3 = fmaf(__uint_as_float(r[i + 3]) * rs, a0.w, b0.w);
              const float o4 = fmaf(__uint_as_float(r[i + 4]) * rs, a1.x, b1.x), o5 = fmaf(__uint_as_float(r[i + 5]) * rs, a1.y, b1.y);
              const float o6 = fmaf(__uint_as_float(r[i + 6]) * rs, a1.z, b1.z), o7 = fmaf(__uint_as_float(r[i + 7]) * rs, a1.w, b1.w);
              if (p.push_rows_per > 0) {
                // staged per warp as plain tile rows (272-byte pitch: the 16-byte stores of eight rows fall on distinct banks)
                if constexpr (BN == 128)
                  *reinterpret_cast<uint4*>(push_stage + ((warp - 2) * 32 + lane) * Cfg::PUSH_ROW + (c * 32 + i) * 2) =
                      make_uint4(pack_bf16x2(o0, o1), pack_bf16x2(o2, o3), pack_bf16x2(o4, o5), pack_bf16x2(o6, o7));
              } else if (p.mc_out != nullptr) {
                if (whole) {
                  const size_t off = ((size_t)row * p.ldc + col0 + i) * 2;
                  asm volatile("multimem.red.relaxed.sys.global.add.v4.bf16x2 [%0], {%1,%2,%3,%4};"
                               ::"l"(reinterpret_cast<uint8_t*>(p.mc_out) + off), "r"(pack_bf16x2(o0, o1)), "r"(pack_bf16x2(o2, o3)),
                                 "r"(pack_bf16x2(o4, o5)), "r"(pack_bf16x2(o6, o7))
                               : "memory");
                }
              } else if (whole) {
                *reinterpret_cast<uint4*>(dst + i) =
                    make_uint4(pack_bf16x2(o0, o1), pack_bf16x2(o2, o3), pack_bf16x2(o4, o5), pack_bf16x2(o6, o7));
              } else {
                if (col0 + i < p.N) dst[i] = __float2bfloat16(o0);
                if (col0 + i + 1 < p.N) dst[i + 1] = __float2bfloat16(o1);
                if (col0 + i + 2 < p.N) dst[i + 2] = __float2bfloat16(o2);
                if (col0 + i + 3 < p.N) dst[i + 3] = __float2bfloat16(o3);
                if (col0 + i + 4 < p.N) dst[i + 4] = __float2bfloat16(o4);
                if (col0 + i + 5 < p.N) dst[i + 5] = __float2bfloat16(o5);
                if (col0 + i + 6 < p.N) dst[i + 6] = __float2bfloat16(o6);
                if (col0 + i + 7 < p.N) dst[i + 7] = __float2bfloat16(o7);
              }
            }
          }
        }
        if constexpr (!OUT_F32 && BN == 128) {
          if (p.push_rows_per > 0 && c == BN / 32 - 1) {
            // the warp's 32 rows of the tile are staged: each lane sends its row (256 contiguous bytes) into the owner rank's
            // slot buffer with one bulk copy - asynchronous, so the SM does not sit on NVLink write round trips
            fence_async_smem();
            __syncwarp();
            if (threadIdx.x == 64) GT_STAMP(2);
            const int colt = nt * BN;
            if (row < p.M && colt < p.N) {
              const int owner = row / p.push_rows_per;
              __nv_bfloat16* prow = p.push_slot[owner] +
                                    ((size_t)p.rank * p.push_rows_per + (row - owner * p.push_rows_per)) * p.N + colt;
              const int bytes = min(BN, p.N - colt) * 2;
              bulk_store(prow, push_stage + ((warp - 2) * 32 + lane) * Cfg::PUSH_ROW, (uint32_t)bytes);
            }
            tma_store_commit();
            tma_store_wait_read();      // the staging rows may be overwritten by the next tile
            __syncwarp();
            if (threadIdx.x == 64) GT_STAMP(3);
          }
        }
      }
      if (OUT_F32 && p.amax_val != nullptr && row < p.M) {
        p.amax_val[(size_t)nt * p.M + row] = best_v;
        p.amax_idx[(size_t)nt * p.M + row] = best_i;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[ab]);
    }
  }
  if (p.push_rows_per > 0 && warp >= 2) tma_store_wait_all();   // this thread's pushed rows have been written
  if (threadIdx.x == 64) GT_STAMP(4);
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) GT_STAMP(5);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  if (p.push_rows_per > 0 && threadIdx.x == 0) {
    // every CTA's peer stores are ordered before its count; the last CTA of this rank raises its flag on every owner
    fence_acq_rel_sys();
    GT_STAMP(6);
    const unsigned prev = atomicAdd(p.done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      *p.done_ctr = 0;
      const uint32_t e = *p.epoch + 1;
      *p.epoch = e;
      fence_acq_rel_sys();
      for (int r = 0; r < p.world; ++r)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.push_flag[r] + p.rank), "r"(e) : "memory");
    }
  } else if (p.mc_out != nullptr && threadIdx.x == 0) {
    // every CTA's reductions are ordered before its count; the last CTA of this rank tells the peers and waits for them
    fence_acq_rel_sys();
    const unsigned prev = atomicAdd(p.done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      *p.done_ctr = 0;
      const uint32_t e = *p.epoch + 1;
      *p.epoch = e;
      fence_acq_rel_sys();
      for (int r = 0; r < p.world; ++r)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.peer_pad[r] + p.rank), "r"(e) : "memory");
      for (int r = 0; r < p.world; ++r) {
        const long long t0 = clock64();
        while (true) {
          uint32_t v;
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.peer_pad[p.rank] + r) : "memory");
          if ((int32_t)(v - e) >= 0) break;
          if (clock64() - t0 > p.spin_limit) { atomicCAS(p.status, kOk, kErrFlagTimeout); break; }
        }
      }
    }
  }
}

template <int KIND, int BN, bool OUT_F32>
static cudaError_t launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int max_ctas,
                          cudaStream_t stream) {
  using Cfg = GemmCfg<KIND, BN>;
  auto kern = gemm_tc_kernel<KIND, BN, OUT_F32>;
  static PerDeviceOnce configured;
  {
    cudaError_t e = configured.smem_limit(kern, Cfg::SMEM);
    if (e != cudaSuccess) return e;
  }
  const int tiles = ((p.M + 127) / 128) * ((p.N + BN - 1) / BN);
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  return launch_pdl(kern, dim3(grid), dim3(192), Cfg::SMEM, stream, tmA, tmB, p);
}

}  // namespace blz

namespace {
struct FuseArgs {
  void* mc_out = nullptr;
  unsigned* done_ctr = nullptr;
  uint32_t* peer_pad[8] = {nullptr};
  uint32_t* epoch = nullptr;
  long long spin_limit = 0;
  int rank = 0, world = 1;
};
thread_local FuseArgs g_fuse;
struct PushArgs {
  __nv_bfloat16* slot[8] = {nullptr};
  uint32_t* flag[8] = {nullptr};
  unsigned* done_ctr = nullptr;
  uint32_t* epoch = nullptr;
  int rank = 0, world = 1, rows_per = 0;
};
thread_local PushArgs g_push;
thread_local long long* g_stamps = nullptr;
struct WaitArgs {
  const uint32_t* pad = nullptr;
  const uint32_t* epoch = nullptr;
  int world = 0;
  long long limit = 0;
};
thread_local WaitArgs g_wait;
struct AmaxArgs {
  float* val = nullptr;
  int* idx = nullptr;
};
thread_local AmaxArgs g_amax;
}  // namespace

namespace blz {
// The one-shot arming (fused all-reduce, peer wait, arg-max epilogue) applies to exactly one GEMM call of this thread.
// Any GEMM entry point clears it on entry; an entry that cannot honour it reports whether something was armed.
bool gemm_oneshot_take_unsupported() {
  const bool armed = g_fuse.mc_out != nullptr || g_wait.pad != nullptr || g_amax.val != nullptr || g_push.rows_per > 0;
  g_fuse.mc_out = nullptr;
  g_push.rows_per = 0;
  g_wait.pad = nullptr;
  g_amax.val = nullptr; g_amax.idx = nullptr;
  return armed;
}
}  // namespace blz

// Arms the NEXT blz_gemm_tc call (fp32 output form, bn 128) on this thread as a greedy head: instead of writing the
// logits it records, per 128-column tile and row, the largest value and its column in val / idx ([ceil(N/128)][M]);
// blz_argmax_parts then reduces over the tiles.
BLZ_API int blz_gemm_argmax_parts(void* val, void* idx) {
  if (!val || !idx) return (int)cudaErrorInvalidValue;
  g_amax.val = reinterpret_cast<float*>(val);
  g_amax.idx = reinterpret_cast<int*>(idx);
  return 0;
}

// Arms the NEXT blz_gemm_tc call on this thread to wait, inside its producer warp and after it has sent its first weight
// tiles, for the A operand: arrival counter r of `counters` (uint32 per source rank, in this GPU's memory) must reach the
// value in the device word `expect` for every rank r < world.  A signalling collective kernel advances `expect` by its
// block count when it starts and every one of its blocks adds one to the peers' counters on its way out.
BLZ_API int blz_gemm_wait_flags(const void* counters, const void* expect, int world, int timeout_ms) {
  if (!counters || !expect || world < 1 || world > 8) return (int)cudaErrorInvalidValue;
  g_wait.pad = reinterpret_cast<const uint32_t*>(counters);
  g_wait.epoch = reinterpret_cast<const uint32_t*>(expect);
  g_wait.world = world;
  g_wait.limit = (long long)(timeout_ms > 0 ? timeout_ms : 10000) * 1900000LL;
  return 0;
}

// Arms the NEXT blz_gemm_tc call on this thread as a fused GEMM + all-reduce: its epilogue reduces the bf16 partial
// tiles into `mc_out` (the multicast view of a zeroed output buffer that every rank maps) and the kernel ends with a
// cross-rank barrier.  pads[r] points at rank r's flag row (world uint32), epoch / done_ctr are local device words.
BLZ_API int blz_gemm_fuse_allreduce(void* mc_out, void* done_ctr, void* const* pads, void* epoch, int rank, int world,
                                    int timeout_ms) {
  if (!mc_out || world < 1 || world > 8) return (int)cudaErrorInvalidValue;
  g_fuse.mc_out = mc_out;
  g_fuse.done_ctr = reinterpret_cast<unsigned*>(done_ctr);
  g_fuse.epoch = reinterpret_cast<uint32_t*>(epoch);
  g_fuse.rank = rank; g_fuse.world = world;
  g_fuse.spin_limit = (long long)(timeout_ms > 0 ? timeout_ms : 10000) * 1900000LL;
  for (int r = 0; r < world; ++r) g_fuse.peer_pad[r] = reinterpret_cast<uint32_t*>(pads[r]);
  return 0;
}

// Diagnostics: the NEXT blz_gemm_tc call records global-timer stamps per CTA in stamps[blockIdx.x][8]: 0 set-up done,
// 1 first accumulator complete, 2 tile staged, 3 rows handed to the copy engine, 4 pushed rows written, 5 CTA joined,
// 6 system fence done (pushed epilogue only for 2-6).
BLZ_API int blz_gemm_debug_stamps(void* stamps) { g_stamps = reinterpret_cast<long long*>(stamps); return 0; }

// Arms the NEXT blz_gemm_tc call on this thread as a fused GEMM + reduce-scatter by push: the bf16 output rows are not
// written to C but stored into the slot buffer of the rank that owns them (slots[o] = rank o's buffer
// [world][rows_per][N], bf16; row r belongs to rank r / rows_per), and when this rank's last CTA is done it writes the
// advanced epoch to flags[o][rank] on every owner.  done_ctr / epoch: zero-initialised local device words; the epoch word is
// what the owner's reduction kernel compares its flags with (blz_comm_slots_norm).  Needs N % 32 == 0.
BLZ_API int blz_gemm_push_rs(void* const* slots, void* const* flags, void* done_ctr, void* epoch, int rank, int world, int rows_per) {
  if (!slots || !flags || !done_ctr || !epoch || world < 1 || world > 8 || rows_per < 1) return (int)cudaErrorInvalidValue;
  for (int r = 0; r < world; ++r) {
    g_push.slot[r] = reinterpret_cast<__nv_bfloat16*>(slots[r]);
    g_push.flag[r] = reinterpret_cast<uint32_t*>(flags[r]);
  }
  g_push.done_ctr = reinterpret_cast<unsigned*>(done_ctr);
  g_push.epoch = reinterpret_cast<uint32_t*>(epoch);
  g_push.rank = rank; g_push.world = world; g_push.rows_per = rows_per;
  return 0;
}

// kind: 0 bf16, 1 nvfp4, 2 mxfp8, 3 fp8.  A [M, K] and B [N, K] row-major (packed bytes for 4/8-bit kinds);
// lda / ldb in BYTES.  out_f32: C is fp32, else bf16; ldc in elements.  bn: 128 or 256 (0 = choose).
// act = 1: B's rows come in groups of [16 gate | 16 up] features and C is bf16 [M, N/2] = silu(gate) * up (ldc % 8 == 0).
// b_kt > 0: B is the tile-major repack [ceil(N/128)][b_kt][128][128 bytes] (zero padded), b_kt = ceil(row bytes / 128).
BLZ_API int blz_gemm_tc(int kind, const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc,
                        int M, int N, int K, const float* row_scale, const float* alpha, const void* bias,
                        const void* sfa, const void* sfb, int out_f32, int bn, int max_ctas, const int* tile_expert,
                        int num_experts, int b_kt, int act, cudaStream_t stream) {
  using namespace blz;
  // snapshot and clear the one-shot arming first: an early return below must not leave it armed for an unrelated GEMM
  const FuseArgs fuse = g_fuse;
  const WaitArgs wait = g_wait;
  const AmaxArgs amax = g_amax;
  const PushArgs push = g_push;
  g_push.rows_per = 0;
  g_fuse.mc_out = nullptr;
  g_wait.pad = nullptr;
  g_amax.val = nullptr; g_amax.idx = nullptr;
  if (M <= 0 || N <= 0 || K <= 0 || kind < 0 || kind > 3) return (int)cudaErrorInvalidValue;
  const int kmma = kind == 0 ? 16 : kind == 1 ? 64 : 32;
  if (K % kmma) return (int)cudaErrorInvalidValue;
  if ((kind == 1 || kind == 2) && (!sfa || !sfb)) return (int)cudaErrorInvalidValue;
  if (bn == 0) {
    // block-scaled kinds keep two accumulator buffers only at BN = 128; the dense kinds have room for BN = 256
    const long tiles128 = (long)((M + 127) / 128) * ((N + 127) / 128);
    bn = ((kind == 0 || kind == 3) && tiles128 >= 2L * sm_count() && N % 256 == 0) ? 256 : 128;
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.row_scale = row_scale; p.alpha = alpha;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.sfa = reinterpret_cast<const uint8_t*>(sfa); p.sfb = reinterpret_cast<const uint8_t*>(sfb);
  p.sfa_col_tiles = kind == 1 ? (K + 63) / 64 : kind == 2 ? (K + 127) / 128 : 0;
  p.status = status_word();
  p.tile_expert = tile_expert;
  p.b_kt = b_kt;
  p.b_raw = reinterpret_cast<const uint8_t*>(B);
  p.act = act;
  if (act && (out_f32 || N % 32 || (ldc & 7) || tile_expert)) return (int)cudaErrorInvalidValue;
  if (b_kt > 0 && tile_expert) return (int)cudaErrorInvalidValue;
  p.mc_out = nullptr; p.done_ctr = nullptr; p.epoch = nullptr; p.spin_limit = 0; p.rank = 0; p.world = 1;
  p.push_rows_per = 0;
  p.stamps = g_stamps;
  g_stamps = nullptr;
  if (push.rows_per > 0) {
    if (out_f32 || (N % 8) || act || tile_expert || fuse.mc_out || amax.val ||
        (long long)push.rows_per * push.world < M)
      return (int)cudaErrorInvalidValue;
    p.push_rows_per = push.rows_per;
    for (int r = 0; r < push.world; ++r) { p.push_slot[r] = push.slot[r]; p.push_flag[r] = push.flag[r]; }
  }
  p.wait_pad = wait.pad; p.wait_epoch = wait.epoch; p.wait_world = wait.world;
  p.wait_limit = wait.limit;
  p.amax_val = amax.val; p.amax_idx = amax.idx;
  if (p.amax_val && (!out_f32 || tile_expert)) return (int)cudaErrorInvalidValue;
  if (p.amax_val || push.rows_per > 0) bn = 128;
  if (fuse.mc_out) {
    if (out_f32 || (N % 32)) return (int)cudaErrorInvalidValue;
    p.mc_out = fuse.mc_out; p.done_ctr = fuse.done_ctr; p.epoch = fuse.epoch; p.spin_limit = fuse.spin_limit;
    p.rank = fuse.rank; p.world = fuse.world;
    for (int r = 0; r < fuse.world; ++r) p.peer_pad[r] = fuse.peer_pad[r];
  }
  if (push.rows_per > 0) {
    p.done_ctr = push.done_ctr; p.epoch = push.epoch; p.rank = push.rank; p.world = push.world;
  }
  const uint64_t b_rows = (uint64_t)N * (tile_expert ? (num_experts > 0 ? num_experts : 1) : 1);
  if (tile_expert && N % bn) return (int)cudaErrorInvalidValue;
  CUtensorMap tmA, tmB;
  cudaError_t e;
  if (kind == 0) {
    e = encode_tmap(&tmA, A, 2, K, M, lda, 64, 128, 3);
    if (e != cudaSuccess) return (int)e;
    if (b_kt > 0) e = encode_tmap(&tmB, B, 2, 64, (uint64_t)((N + 127) / 128) * b_kt * 128, 128, 64, 128, 3);
    else e = encode_tmap(&tmB, B, 2, K, b_rows, ldb, 64, bn, 3);
  } else {
    const uint64_t kbytes = kind == 1 ? K / 2 : K;
    e = encode_tmap(&tmA, A, 1, kbytes, M, lda, 128, 128, 3);
    if (e != cudaSuccess) return (int)e;
    if (b_kt > 0) e = encode_tmap(&tmB, B, 1, 128, (uint64_t)((N + 127) / 128) * b_kt * 128, 128, 128, 128, 3);
    else e = encode_tmap(&tmB, B, 1, kbytes, b_rows, ldb, 128, bn, 3);
  }
  if (e != cudaSuccess) return (int)e;
#define BLZ_GEMM_CASE(KD, BNV)                                                                        \
  if (kind == KD && bn == BNV)                                                                        \
    return (int)(out_f32 ? launch<KD, BNV, true>(tmA, tmB, p, max_ctas, stream)                       \
                         : launch<KD, BNV, false>(tmA, tmB, p, max_ctas, stream));
  BLZ_GEMM_CASE(0, 128) BLZ_GEMM_CASE(0, 256) BLZ_GEMM_CASE(1, 128) BLZ_GEMM_CASE(1, 256)
  BLZ_GEMM_CASE(2, 128) BLZ_GEMM_CASE(2, 256) BLZ_GEMM_CASE(3, 128) BLZ_GEMM_CASE(3, 256)
#undef BLZ_GEMM_CASE
  return (int)cudaErrorInvalidValue;
}
