// Wide-N GEMM on tcgen05: one 128-row operand tile against up to 256 rows of the other operand per MMA, so that each
// instruction reads 1.5 shared-memory bytes per accumulator column instead of 2 — the 4-bit kinds are otherwise bound by
// shared-memory reads, not by the tensor pipe — and each scale-factor copy is amortised over twice the math.
//
// Two orientations of  C[tokens, features] = X[tokens, K] · W[features, K]^T :
//   plain   (prefill)  lanes = 128 tokens,   columns = 256 features;
//   swapped (decode)   lanes = 128 features, columns = all tokens of the step (64 / 128 / 256), so every weight byte is
//                      fetched by exactly one CTA; the K range can be split over several CTAs, whose fp32 partial tiles
//                      meet in a workspace and are summed in a fixed order by the CTA that finishes last (deterministic).
//
// The accumulator (up to 256 TMEM columns) is single-buffered: eight epilogue warps pull the whole tile into registers
// (128 columns per thread), hand the TMEM back at once, and do the scaling / conversion / stores while the next tile's
// MMAs run.
//
// Counterpart in the reference: the small-m NVFP4 paths of kernels/src/cuda/nvfp4_linear.cu (weight-streaming GEMV /
// skinny GEMM, :524) and the tiled kernels/src/cuda/nvfp4_gemm.cu — there built on mma.sync; the split and the
// orientation swap are this implementation's own.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "blaze/host.h"
#include "blaze/sm100.cuh"

namespace blz {

bool gemm_oneshot_take_unsupported();   // gemm_tc.cu

struct WideParams {
  int lanes_total;            // rows of the lane operand (tokens when plain, features when swapped)
  int cols_total;             // rows of the column operand
  int K;                      // elements
  void* C;                    // [tokens, ldc] bf16 or fp32
  long long ldc;
  int out_f32;
  const float* lane_scale;    // per lane-operand row, or null
  const float* col_scale;     // per column-operand row, or null
  const __nv_bfloat16* bias;  // per feature, or null
  const uint8_t* sf_lane;     // 128x4-tiled scale factors of the lane operand (block-scaled kinds)
  const uint8_t* sf_col;
  int sf_col_tiles;           // 4-column scale tiles per 128-row tile
  int ksplit;                 // CTAs sharing one output tile along K
  float* ws;                  // [tiles * ksplit][128][BN] fp32 partial tiles (ksplit > 1)
  unsigned* ctr;              // [tiles] arrival counters, zero between launches
  int act;                    // 1 (plain orientation): columns are [16 gate | 16 up] groups; C = silu(gate) * up, bf16 [tokens, N/2]
  int w_kt;                   // > 0: the weight operand is tile-major, [rows/128][w_kt][16 KB swizzled tile image]
  const uint8_t* w_raw;       // its base (fetched with plain bulk copies)
  int* status;
};

template <int KIND>
struct WKind;
template <> struct WKind<0> { static constexpr int KMMA = 16, SF_ATOMS = 0; };
template <> struct WKind<1> { static constexpr int KMMA = 64, SF_ATOMS = 4; };
template <> struct WKind<2> { static constexpr int KMMA = 32, SF_ATOMS = 1; };
template <> struct WKind<3> { static constexpr int KMMA = 32, SF_ATOMS = 0; };

template <int KIND, int BN>
struct WideCfg {
  static constexpr int KMMA = WKind<KIND>::KMMA;
  static constexpr int BK = KMMA * 4;                       // 128 bytes of K per row and stage
  static constexpr int SF_ATOMS = WKind<KIND>::SF_ATOMS;
  static constexpr int NB = (BN + 127) / 128;               // 128-row scale tiles of the column operand
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int SFA_BYTES = SF_ATOMS * 512;
  static constexpr int SFB_BYTES = SF_ATOMS * 512 * NB;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int RAW_STAGES = (216 * 1024) / STAGE_BYTES;
  static constexpr int SF_COLS = SF_ATOMS * 4 * (1 + NB);
  static constexpr int STAGES_BY_TMEM = SF_COLS ? (512 - BN) / SF_COLS : 8;
  static constexpr int STAGES = RAW_STAGES < 8 ? (RAW_STAGES < STAGES_BY_TMEM ? RAW_STAGES : STAGES_BY_TMEM)
                                               : (8 < STAGES_BY_TMEM ? 8 : STAGES_BY_TMEM);
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
  static constexpr int CPT = BN / 2;                        // accumulator columns per epilogue thread
  static constexpr int THREADS = 320;                       // producer, MMA issuer, 8 epilogue warps
  static_assert(BN + STAGES * SF_COLS <= 512, "TMEM budget");
  static_assert(STAGES >= 2, "pipeline depth");
};

template <int KIND, int BN, bool SWAP>
__global__ void __launch_bounds__(320, 1) gemm_wide_kernel(const __grid_constant__ CUtensorMap tmA,
                                                            const __grid_constant__ CUtensorMap tmB, const WideParams p) {
  pdl_trigger();
  using Cfg = WideCfg<KIND, BN>;
  constexpr int STAGES = Cfg::STAGES, BK = Cfg::BK, CPT = Cfg::CPT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = base;
  uint8_t* sB = sA + STAGES * Cfg::A_BYTES;
  uint8_t* sSFA = sB + STAGES * Cfg::B_BYTES;
  uint8_t* sSFB = sSFA + STAGES * Cfg::SFA_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sSFB + STAGES * Cfg::SFB_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = acc_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_last = const_cast<int*>(abort_flag) + 1;
  __shared__ float s_cs[BN];          // per-column multiplier of the current tile
  __shared__ float s_cb[BN];          // per-column bias (plain orientation)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_l = (p.lanes_total + 127) / 128;
  const int tiles_c = (p.cols_total + BN - 1) / BN;
  const int k_tiles = (p.K + BK - 1) / BK;
  const int kb_per = (k_tiles + p.ksplit - 1) / p.ksplit;
  const int units = tiles_l * tiles_c * p.ksplit;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 8);
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
  constexpr uint32_t SF_COL0 = BN;
  pdl_wait();

  // unit u -> (lane tile, column tile, k slice); lane tiles of one column tile are neighbours so that CTAs running
  // together share the column operand in L2
  auto decode = [&](int u, int& lt, int& ct, int& ks) {
    ks = u % p.ksplit;
    const int t = u / p.ksplit;
    lt = t % tiles_l;
    ct = t / tiles_l;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (elect_one()) {
      int s = 0; uint32_t ph = 0;
      for (int u = blockIdx.x; u < units; u += gridDim.x) {
        int lt, ct, ks;
        decode(u, lt, ct, ks);
        const int kt0 = ks * kb_per, kt1 = min(k_tiles, kt0 + kb_per);
        for (int kt = kt0; kt < kt1; ++kt) {
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status)) goto producer_done;
          uint32_t bytes = Cfg::A_BYTES + Cfg::B_BYTES;
          int atoms = 0;
          if constexpr (Cfg::SF_ATOMS > 0) {
            atoms = min(Cfg::SF_ATOMS, p.sf_col_tiles - kt * Cfg::SF_ATOMS);
            bytes += atoms * 512 * (1 + Cfg::NB);
          }
          mbar_expect_tx(&full[s], bytes);
          const int kc = (KIND == 0) ? kt * BK : kt * 128;
          if (p.w_kt > 0 && SWAP) {
            bulk_load(sA + s * Cfg::A_BYTES, p.w_raw + ((size_t)lt * p.w_kt + kt) * 16384, 16384, &full[s]);
          } else {
            tma_load_2d(sA + s * Cfg::A_BYTES, &tmA, kc, lt * 128, &full[s]);
          }
          if (p.w_kt > 0 && !SWAP) {
#pragma unroll
            for (int h = 0; h < Cfg::NB; ++h)
              bulk_load(sB + s * Cfg::B_BYTES + h * 16384, p.w_raw + ((size_t)(ct * Cfg::NB + h) * p.w_kt + kt) * 16384, 16384,
                        &full[s]);
          } else {
            tma_load_2d(sB + s * Cfg::B_BYTES, &tmB, kc, ct * BN, &full[s]);
          }
          if constexpr (Cfg::SF_ATOMS > 0) {
            const size_t a_off = ((size_t)lt * p.sf_col_tiles + (size_t)kt * Cfg::SF_ATOMS) * 512;
            bulk_load(sSFA + s * Cfg::SFA_BYTES, p.sf_lane + a_off, atoms * 512, &full[s]);
#pragma unroll
            for (int h = 0; h < Cfg::NB; ++h) {
              const size_t b_off = ((size_t)((ct * BN) / 128 + h) * p.sf_col_tiles + (size_t)kt * Cfg::SF_ATOMS) * 512;
              bulk_load(sSFB + s * Cfg::SFB_BYTES + h * Cfg::SFA_BYTES, p.sf_col + b_off, atoms * 512, &full[s]);
            }
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    producer_done:;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      int s = 0; uint32_t ph = 0;
      uint32_t it = 0;
      for (int u = blockIdx.x; u < units; u += gridDim.x) {
        int lt, ct, ks;
        decode(u, lt, ct, ks);
        const int kt0 = ks * kb_per, kt1 = min(k_tiles, kt0 + kb_per);
        if (!mbar_wait(acc_empty, (it & 1) ^ 1, abort_flag, p.status)) break;
        ++it;
        tc_fence_after();
        bool ok = true;
        for (int kt = kt0; kt < kt1; ++kt) {
          if (!mbar_wait(&full[s], ph, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * Cfg::A_BYTES), b_addr = smem_u32(sB + s * Cfg::B_BYTES);
          const int nblk = min(4, (p.K - kt * BK + Cfg::KMMA - 1) / Cfg::KMMA);
          const uint32_t sf_t = tmem + SF_COL0 + s * Cfg::SF_COLS;
          if constexpr (Cfg::SF_ATOMS > 0) {
            const int atoms = min(Cfg::SF_ATOMS, p.sf_col_tiles - kt * Cfg::SF_ATOMS);
            for (int a = 0; a < atoms; ++a) {
              tmem_cp_sf(sf_t + a * 4, make_smem_desc(smem_u32(sSFA + s * Cfg::SFA_BYTES + a * 512), 0, 128, kSwzNone));
#pragma unroll
              for (int h = 0; h < Cfg::NB; ++h)
                tmem_cp_sf(sf_t + Cfg::SF_ATOMS * 4 + (a * Cfg::NB + h) * 4,
                           make_smem_desc(smem_u32(sSFB + s * Cfg::SFB_BYTES + h * Cfg::SFA_BYTES + a * 512), 0, 128, kSwzNone));
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (j < nblk) {
              const uint64_t da = desc_sw128(a_addr + j * 32), db = desc_sw128(b_addr + j * 32);
              const uint32_t acc = (kt > kt0 || j > 0) ? 1u : 0u;
              if constexpr (KIND == 0) {
                mma_f16(tmem, da, db, make_idesc(1, 1, 128, BN), acc);
              } else if constexpr (KIND == 3) {
                mma_f8(tmem, da, db, make_idesc(0, 0, 128, BN), acc);
              } else if constexpr (KIND == 1) {
                mma_nvfp4(tmem, da, db, make_idesc_bs(1, 1, 0, 128, BN), sf_t + j * 4,
                          sf_t + Cfg::SF_ATOMS * 4 + j * 4 * Cfg::NB, acc);
              } else {
                mma_mxf8(tmem, da, db, make_idesc_bs(0, 0, 1, 128, BN, j, j), sf_t, sf_t + Cfg::SF_ATOMS * 4, acc);
              }
            }
          }
          mma_commit(&empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        mma_commit(acc_full);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int e = warp - 2;
    const int q = warp & 3;                      // TMEM lane quadrant this warp may read
    const int half = e >> 2;                     // which half of the columns
    const int etid = threadIdx.x - 64;           // 0..255
    uint32_t it = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      int lt, ct, ks;
      decode(u, lt, ct, ks);
      // per-column multipliers (and bias when the columns are features) of this tile
      bar_sync(1, 256);                          // the previous tile's readers are done with s_cs / s_cb
      for (int i = etid; i < BN; i += 256) {
        const int col = ct * BN + i;
        s_cs[i] = (p.col_scale && col < p.cols_total) ? __ldg(p.col_scale + col) : 1.0f;
        s_cb[i] = (!SWAP && p.bias && col < p.cols_total) ? bf2f(p.bias[col]) : 0.0f;
      }
      const int lrow = lt * 128 + q * 32 + lane;                 // row of the lane operand held by this thread
      const float ls = (p.lane_scale && lrow < p.lanes_total) ? __ldg(p.lane_scale + lrow) : 1.0f;
      const float lb = (SWAP && p.bias && lrow < p.lanes_total) ? bf2f(p.bias[lrow]) : 0.0f;
      const bool got_acc = mbar_wait(acc_full, it & 1, abort_flag, p.status);
      ++it;
      tc_fence_after();
      uint32_t r[CPT];
#pragma unroll
      for (int c = 0; c < CPT / 32; ++c)
        tmem_ld32(tmem + half * CPT + c * 32 + ((uint32_t)(q * 32) << 16), *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);     // the accumulator is in registers: the next tile may start
      // s_cs / s_cb are complete; and the warps agree on whether the wait ran out, so that none is left at a barrier
      if (!bar_red_and(1, 256, got_acc)) break;

      if (p.ksplit > 1) {
        // park the partial tile, then the CTA that arrives last for this output tile sums all slices in slice order
        const int tile = u / p.ksplit;
        float* mine = p.ws + ((size_t)u * 128 + q * 32 + lane) * BN + half * CPT;
#pragma unroll
        for (int i = 0; i < CPT; i += 4)
          *reinterpret_cast<uint4*>(mine + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
        __threadfence();
        bar_sync(2, 256);
        if (etid == 0) {
          const unsigned prev = atomicAdd(p.ctr + tile, 1u);
          const int last = prev == (unsigned)(p.ksplit - 1);
          if (last) p.ctr[tile] = 0;
          *s_last = last;
        }
        bar_sync(2, 256);
        if (!*s_last) continue;
        __threadfence();
#pragma unroll
        for (int i = 0; i < CPT; ++i) r[i] = 0;
        for (int s2 = 0; s2 < p.ksplit; ++s2) {
          const float* src = p.ws + ((size_t)(tile * p.ksplit + s2) * 128 + q * 32 + lane) * BN + half * CPT;
#pragma unroll
          for (int i = 0; i < CPT; i += 4) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + i));
            r[i] = __float_as_uint(__uint_as_float(r[i]) + v.x);
            r[i + 1] = __float_as_uint(__uint_as_float(r[i + 1]) + v.y);
            r[i + 2] = __float_as_uint(__uint_as_float(r[i + 2]) + v.z);
            r[i + 3] = __float_as_uint(__uint_as_float(r[i + 3]) + v.w);
          }
        }
      }

      const int c0 = ct * BN + half * CPT;       // first column (row of the column operand) of this thread
      if constexpr (SWAP) {
        // lanes are features, columns are tokens: C[token][feature]
        const int feat = lrow;
        const bool feat_ok = feat < p.lanes_total;
        if (p.out_f32) {
          float* C = reinterpret_cast<float*>(p.C);
#pragma unroll
          for (int i = 0; i < CPT; ++i) {
            const int tok = c0 + i;
            if (feat_ok && tok < p.cols_total)
              C[(size_t)tok * p.ldc + feat] = fmaf(__uint_as_float(r[i]) * ls, s_cs[half * CPT + i], lb);
          }
        } else {
          // neighbouring lanes trade every other token so that each writes two adjacent features at once
          __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.C);
          const bool odd = lane & 1;
          const bool pair_ok = (p.lanes_total & 1) == 0 && (p.ldc & 1) == 0;
#pragma unroll
          for (int i = 0; i < CPT; i += 2) {
            const float v0 = fmaf(__uint_as_float(r[i]) * ls, s_cs[half * CPT + i], lb);
            const float v1 = fmaf(__uint_as_float(r[i + 1]) * ls, s_cs[half * CPT + i + 1], lb);
            const float give = odd ? v0 : v1;
            const float got = __shfl_xor_sync(0xffffffffu, give, 1);
            const int tok = c0 + i + (odd ? 1 : 0);
            if (tok < p.cols_total) {
              if (pair_ok) {
                if (feat_ok) {
                  const uint32_t pk = odd ? pack_bf16x2(got, v1) : pack_bf16x2(v0, got);
                  *reinterpret_cast<uint32_t*>(C + (size_t)tok * p.ldc + (feat & ~1)) = pk;
                }
              } else {
                // odd widths: plain element stores
                const int f_lo = feat & ~1;
                if (f_lo < p.lanes_total) C[(size_t)tok * p.ldc + f_lo] = __float2bfloat16(odd ? got : v0);
                if (f_lo + 1 < p.lanes_total) C[(size_t)tok * p.ldc + f_lo + 1] = __float2bfloat16(odd ? v1 : got);
              }
            }
          }
        }
      } else {
        // lanes are tokens, columns are features
        const int tok = lrow;
        if (tok < p.lanes_total) {
          if (p.out_f32) {
            float* dst = reinterpret_cast<float*>(p.C) + (size_t)tok * p.ldc + c0;
#pragma unroll
            for (int i = 0; i < CPT; i += 4) {
              if (c0 + i + 4 <= p.cols_total && (p.ldc & 3) == 0) {
                float4 o;
                o.x = fmaf(__uint_as_float(r[i]) * ls, s_cs[half * CPT + i], s_cb[half * CPT + i]);
                o.y = fmaf(__uint_as_float(r[i + 1]) * ls, s_cs[half * CPT + i + 1], s_cb[half * CPT + i + 1]);
                o.z = fmaf(__uint_as_float(r[i + 2]) * ls, s_cs[half * CPT + i + 2], s_cb[half * CPT + i + 2]);
                o.w = fmaf(__uint_as_float(r[i + 3]) * ls, s_cs[half * CPT + i + 3], s_cb[half * CPT + i + 3]);
                *reinterpret_cast<float4*>(dst + i) = o;
              } else {
                for (int j = 0; j < 4; ++j)
                  if (c0 + i + j < p.cols_total)
                    dst[i + j] = fmaf(__uint_as_float(r[i + j]) * ls, s_cs[half * CPT + i + j], s_cb[half * CPT + i + j]);
              }
            }
          } else if (p.act) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)tok * p.ldc + c0 / 2;
#pragma unroll
            for (int gq = 0; gq < CPT; gq += 32) {
              uint32_t pk[8];
#pragma unroll
              for (int i = 0; i < 16; i += 2) {
                float a[2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                  const int cg = half * CPT + gq + i + j, cu = cg + 16;
                  const float g = bf2f(__float2bfloat16(fmaf(__uint_as_float(r[gq + i + j]) * ls, s_cs[cg], s_cb[cg])));
                  const float u = bf2f(__float2bfloat16(fmaf(__uint_as_float(r[gq + 16 + i + j]) * ls, s_cs[cu], s_cb[cu])));
                  a[j] = g / (1.f + __expf(-g)) * u;
                }
                pk[i / 2] = pack_bf16x2(a[0], a[1]);
              }
              if (c0 + gq + 32 <= p.cols_total) {
                *reinterpret_cast<uint4*>(dst + gq / 2) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                *reinterpret_cast<uint4*>(dst + gq / 2 + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
              }
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)tok * p.ldc + c0;
#pragma unroll
            for (int i = 0; i < CPT; i += 8) {
              float o[8];
#pragma unroll
              for (int j = 0; j < 8; ++j)
                o[j] = fmaf(__uint_as_float(r[i + j]) * ls, s_cs[half * CPT + i + j], s_cb[half * CPT + i + j]);
              if (c0 + i + 8 <= p.cols_total && (p.ldc & 7) == 0) {
                *reinterpret_cast<uint4*>(dst + i) =
                    make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (c0 + i + j < p.cols_total) dst[i + j] = __float2bfloat16(o[j]);
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

template <int KIND, int BN, bool SWAP>
static cudaError_t launch_wide(const CUtensorMap& tmA, const CUtensorMap& tmB, const WideParams& p, int units, int max_ctas,
                               cudaStream_t stream) {
  using Cfg = WideCfg<KIND, BN>;
  auto kern = gemm_wide_kernel<KIND, BN, SWAP>;
  static PerDeviceOnce configured;
  {
    cudaError_t e = configured.smem_limit(kern, Cfg::SMEM);
    if (e != cudaSuccess) return e;
  }
  int grid = units < sm_count() ? units : sm_count();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  return launch_pdl(kern, dim3(grid), dim3(Cfg::THREADS), Cfg::SMEM, stream, tmA, tmB, p);
}

}  // namespace blz

// How many CTAs should share one output tile along K: fewest rounds of (k blocks + fixed cost) over the SMs.
BLZ_API int blz_gemm_wide_ksplit(int tiles, int k_tiles, int sms) {
  static const int cand[] = {1, 2, 3, 4, 6, 8};
  int best = 1;
  long best_cost = 1L << 60;
  for (int c : cand) {
    if (c > k_tiles) break;
    const long rounds = ((long)tiles * c + sms - 1) / sms;
    const long cost = rounds * ((k_tiles + c - 1) / c + 3) + (c > 1 ? 2 : 0);
    if (cost < best_cost) { best_cost = cost; best = c; }
  }
  return best;
}

// C[M, N] = X[M, K] · W[N, K]^T with the same operand conventions as blz_gemm_tc (ldx / ldw in BYTES, ldc in elements).
// swap = 1: features on the TMEM lanes, the M <= 256 tokens on the columns (decode); swap = 0: tokens on the lanes, 256
// features per tile (needs N % 256 == 0).  ksplit > 1 (swap only) needs `ws` (fp32, tiles * ksplit * 128 * bn floats) and
// `ctr` (one zeroed uint32 per tile; the kernel leaves them zero).  w_kt > 0: W is the tile-major repack described at
// blz_gemm_tc.  Returns cudaErrorInvalidValue for shapes it does not cover.
BLZ_API int blz_gemm_wide(int kind, const void* X, long long ldx, const void* W, long long ldw, void* C, long long ldc, int M,
                          int N, int K, const float* row_scale, const float* alpha, const void* bias, const void* sfx,
                          const void* sfw, int out_f32, int swap, int ksplit, void* ws, long long ws_bytes, void* ctr,
                          int max_ctas, int w_kt, int act, cudaStream_t stream) {
  using namespace blz;
  // this kernel has no fused all-reduce / peer-wait / arg-max epilogue: a call armed for one is refused (and disarmed)
  if (gemm_oneshot_take_unsupported()) return (int)cudaErrorNotSupported;
  if (M <= 0 || N <= 0 || K <= 0 || kind < 0 || kind > 3) return (int)cudaErrorInvalidValue;
  const int kmma = kind == 0 ? 16 : kind == 1 ? 64 : 32;
  if (K % kmma) return (int)cudaErrorInvalidValue;
  if ((kind == 1 || kind == 2) && (!sfx || !sfw)) return (int)cudaErrorInvalidValue;
  int bn;
  if (swap) {
    if (M > 256) return (int)cudaErrorInvalidValue;
    bn = M <= 64 ? 64 : (M <= 128 ? 128 : 256);
  } else {
    if (N % 256) return (int)cudaErrorInvalidValue;
    bn = 256;
    ksplit = 1;
  }
  if (ksplit < 1) ksplit = 1;
  WideParams p;
  p.K = K; p.C = C; p.ldc = ldc; p.out_f32 = out_f32;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.sf_col_tiles = kind == 1 ? (K + 63) / 64 : kind == 2 ? (K + 127) / 128 : 0;
  p.status = status_word();
  p.w_kt = w_kt;
  p.w_raw = reinterpret_cast<const uint8_t*>(W);
  p.act = act;
  if (act && (swap || out_f32 || (ldc & 7))) return (int)cudaErrorInvalidValue;
  const void *A, *B;
  long long lda, ldb;
  if (swap) {
    p.lanes_total = N; p.cols_total = M;
    p.lane_scale = alpha; p.col_scale = row_scale;
    p.sf_lane = reinterpret_cast<const uint8_t*>(sfw); p.sf_col = reinterpret_cast<const uint8_t*>(sfx);
    A = W; lda = ldw; B = X; ldb = ldx;
  } else {
    p.lanes_total = M; p.cols_total = N;
    p.lane_scale = row_scale; p.col_scale = alpha;
    p.sf_lane = reinterpret_cast<const uint8_t*>(sfx); p.sf_col = reinterpret_cast<const uint8_t*>(sfw);
    A = X; lda = ldx; B = W; ldb = ldw;
  }
  const int tiles = ((p.lanes_total + 127) / 128) * ((p.cols_total + bn - 1) / bn);
  const int bk = kmma * 4;
  const int k_tiles = (K + bk - 1) / bk;
  if (ksplit > k_tiles) ksplit = k_tiles;
  // every slice must own at least one k block
  while (ksplit > 1 && (long)((k_tiles + ksplit - 1) / ksplit) * (ksplit - 1) >= k_tiles) --ksplit;
  p.ksplit = ksplit;
  p.ws = reinterpret_cast<float*>(ws);
  p.ctr = reinterpret_cast<unsigned*>(ctr);
  if (ksplit > 1) {
    const long long need = (long long)tiles * ksplit * 128 * bn * 4;
    if (!ws || !ctr || ws_bytes < need) return (int)cudaErrorInvalidValue;
  }
  CUtensorMap tmA, tmB;
  cudaError_t e;
  {
    const int es = kind == 0 ? 2 : 1;                                   // bytes per tensor-map element
    const uint64_t inner = kind == 0 ? (uint64_t)K : (kind == 1 ? (uint64_t)K / 2 : (uint64_t)K);
    const uint32_t box0 = 128 / es;
    const uint64_t wrows = (uint64_t)((N + 127) / 128) * (w_kt > 0 ? w_kt : 0) * 128;
    if (w_kt > 0 && swap) e = encode_tmap(&tmA, A, es, box0, wrows, 128, box0, 128, 3);
    else e = encode_tmap(&tmA, A, es, inner, p.lanes_total, lda, box0, 128, 3);
    if (e != cudaSuccess) return (int)e;
    if (w_kt > 0 && !swap) e = encode_tmap(&tmB, B, es, box0, wrows, 128, box0, 128, 3);
    else e = encode_tmap(&tmB, B, es, inner, p.cols_total, ldb, box0, bn, 3);
  }
  if (e != cudaSuccess) return (int)e;
  const int units = tiles * ksplit;
#define BLZ_WIDE_CASE(KD, BNV, SW) \
  if (kind == KD && bn == BNV && (swap != 0) == SW) return (int)launch_wide<KD, BNV, SW>(tmA, tmB, p, units, max_ctas, stream);
  BLZ_WIDE_CASE(0, 64, true) BLZ_WIDE_CASE(0, 128, true) BLZ_WIDE_CASE(0, 256, true) BLZ_WIDE_CASE(0, 256, false)
  BLZ_WIDE_CASE(1, 64, true) BLZ_WIDE_CASE(1, 128, true) BLZ_WIDE_CASE(1, 256, true) BLZ_WIDE_CASE(1, 256, false)
  BLZ_WIDE_CASE(2, 64, true) BLZ_WIDE_CASE(2, 128, true) BLZ_WIDE_CASE(2, 256, true) BLZ_WIDE_CASE(2, 256, false)
  BLZ_WIDE_CASE(3, 64, true) BLZ_WIDE_CASE(3, 128, true) BLZ_WIDE_CASE(3, 256, true) BLZ_WIDE_CASE(3, 256, false)
#undef BLZ_WIDE_CASE
  return (int)cudaErrorInvalidValue;
}
