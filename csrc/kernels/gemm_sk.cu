// Small-M (decode) tcgen05 GEMM with the K range split over a thread-block cluster:
//     C[M,N] = (A[M,K] · B[N,K]^T) * row_scale[m] * alpha[n] (+ bias[n]),  bf16 output
// for the same four operand kinds as gemm_tc.cu (0 bf16, 1 NVFP4, 2 MXFP8, 3 FP8).
//
// Why another kernel: at decode sizes (M <= 256 rows) a GEMM has only a few dozen 128x128 output tiles, so a kernel with
// one CTA per tile leaves a third of the 148 SMs idle and each busy SM pulls its tile's whole K range through its own
// L2 port (measured ~90 GB/s per SM): the time follows bytes per SM, not bytes per GPU.  Here every output tile is
// computed by a cluster of `ks` CTAs, each streaming 1/ks of the K range into its own TMEM accumulator; the partial
// accumulators then meet in distributed shared memory: every CTA owns a slice of the tile's columns, receives all peers'
// partials of that slice in its own shared memory (posted remote stores), sums them in CTA-rank order (so the result is
// bit-reproducible), applies the scales and writes bf16.  No global workspace, no atomics.
//
// Two CTAs fit on an SM (3-stage ring of 36 KB, 256 TMEM columns each), so the prologue / epilogue of one overlaps the
// main loop of the other.  192 threads: warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-5 = epilogue / reducers.
// Every wait after start-up is a bounded mbarrier wait; the hardware cluster barrier is used once, right after barrier
// initialisation, where no role can have failed yet.  No TMA load is cluster-multicast.
//
// Reference counterparts: the split-K small-m kernels of kernels/src/cuda/nvfp4_linear.cu (nvfp4_mma_kernel :185, split
// over warps with a shared-memory reduce; tuner-chosen split :523), fp8_linear.cu :40/:159/:270, and the GEMM router
// crates/blaze/src/linear.rs:535-760.
#include "blaze/host.h"
#include "blaze/sm100.cuh"

namespace blz {

struct SkParams {
  int M, N, K;
  __nv_bfloat16* C;
  long long ldc;
  const float* row_scale;    // [M] or null
  const float* alpha;        // [N] or null
  const __nv_bfloat16* bias; // [N] or null
  const uint8_t* sfa;        // scale factors, 128x4-tiled (kinds 1, 2)
  const uint8_t* sfb;
  int sf_col_tiles;          // 4-column scale tiles per 128-row tile along K
  int ks;                    // cluster size = number of K slices
  int act;                   // 1: B rows are [16 gate | 16 up] groups, C = silu(gate) * up, bf16 [M, N/2] (ks must be 1)
  int* status;
  unsigned* dbg;             // optional [gridDim.x] progress bits per CTA (diagnostics; null = off)
  unsigned long long* prof;  // optional [gridDim.x][16] time stamps per CTA (diagnostics; null = off)
};

#define SK_MARK(bit) do { if (p.dbg) atomicOr(p.dbg + blockIdx.x, (unsigned)(bit)); } while (0)
// time stamps (global nanosecond timer) per CTA, slot i of prof[blockIdx.x][16]
__device__ __forceinline__ unsigned long long sk_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define SK_STAMP(i) do { if (p.prof) p.prof[(size_t)blockIdx.x * 16 + (i)] = sk_now(); } while (0)

template <int KIND> struct SkKind;
template <> struct SkKind<0> { static constexpr int KMMA = 16, SF_ATOMS = 0; };
template <> struct SkKind<1> { static constexpr int KMMA = 64, SF_ATOMS = 4; };
template <> struct SkKind<2> { static constexpr int KMMA = 32, SF_ATOMS = 1; };
template <> struct SkKind<3> { static constexpr int KMMA = 32, SF_ATOMS = 0; };

template <int KIND>
struct SkCfg {
  static constexpr int BM = 128, BN = 128;
  static constexpr int KMMA = SkKind<KIND>::KMMA;
  static constexpr int BK = KMMA * 4;                  // 128 bytes per operand row per stage
  static constexpr int A_BYTES = BM * 128, B_BYTES = BN * 128;
  static constexpr int SF_ATOMS = SkKind<KIND>::SF_ATOMS;
  static constexpr int SF_BYTES = SF_ATOMS * 512;      // per operand per stage
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + 2 * SF_BYTES;
  static constexpr int STAGES = 3;
  static constexpr int SF_COLS_PER_STAGE = SF_ATOMS * 4 * 2;
  static constexpr int SF_COL0 = BN;                   // one accumulator, then the scale columns
  static constexpr int TMEM_COLS = 256;
  static constexpr int PART_BYTES = 96 * 1024;         // most the cluster reduction receives (3 x 2 groups x 32 columns)
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + 2 * BN * 4 /*alpha, bias*/;
  static_assert(SF_COL0 + STAGES * SF_COLS_PER_STAGE <= TMEM_COLS, "TMEM budget");
  static_assert(PART_BYTES <= STAGES * (A_BYTES + B_BYTES), "the partial must fit the operand ring");
  static_assert(2 * (SMEM + 1024) <= 228 * 1024, "two CTAs per SM");
};

__device__ __forceinline__ float silu_mul_bf16(float g, float u) {
  g = bf2f(__float2bfloat16(g));
  u = bf2f(__float2bfloat16(u));
  return g / (1.f + __expf(-g)) * u;
}

template <int KIND>
__global__ void __launch_bounds__(192, 2)
gemm_sk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, SkParams p) {
  using Cfg = SkCfg<KIND>;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + STAGES * Cfg::A_BYTES;
  uint8_t* sSFA = sB + STAGES * Cfg::B_BYTES;
  uint8_t* sSFB = sSFA + STAGES * Cfg::SF_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sSFB + STAGES * Cfg::SF_BYTES);
  uint64_t* full = bars;                    // [STAGES]
  uint64_t* empty = bars + STAGES;          // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;   // [1]
  uint64_t* part_ready = acc_full + 1;      // [1] every CTA of the cluster has parked its partial (ks remote arrivals)
  uint64_t* ring_free = part_ready + 1;     // [1] every CTA of the cluster has finished its main loop (its ring may be written)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ring_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_alpha = reinterpret_cast<float*>(bars) + 64;   // [BN] per-column multipliers of this tile (after 256 bytes of barriers)
  float* s_bias = s_alpha + BN;                            // [BN]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) SK_STAMP(0);
  const int ks = p.ks;
  const int tiles_m = (p.M + BM - 1) / BM;
  const int tile = blockIdx.x / ks;
  const int kr = ks > 1 ? (int)cluster_ctarank() : 0;
  const int mt = tile % tiles_m, nt = tile / tiles_m;
  const int k_tiles = (p.K + BK - 1) / BK;
  const int kb0 = (int)((long long)kr * k_tiles / ks), kb1 = (int)((long long)(kr + 1) * k_tiles / ks);
  const int nkb = kb1 - kb0;                // >= 1: the launcher keeps ks <= k_tiles

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    mbar_init(acc_full, 1);
    mbar_init(part_ready, ks);
    mbar_init(ring_free, ks);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (threadIdx.x == 0) SK_MARK(1);
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) { SK_MARK(2); SK_STAMP(1); }
  // A dependent kernel may become resident from here on: this CTA already holds its tensor memory, so a successor that
  // takes what is left can never keep this kernel from making progress.
  pdl_trigger();
  if (ks > 1) cluster_arrive();             // the peers' barriers are initialised before anyone arrives on them remotely
  const uint32_t tmem = *tmem_slot;
  if (threadIdx.x == 0) SK_MARK(4);

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      auto issue = [&](int s, int kt, int what) {
        int atoms = 0;
        if constexpr (Cfg::SF_ATOMS > 0) atoms = min(Cfg::SF_ATOMS, p.sf_col_tiles - kt * Cfg::SF_ATOMS);
        const int kc = (KIND == 0) ? kt * BK : kt * 128;
        if (what & 1) {
          mbar_expect_tx(&full[s], Cfg::A_BYTES + Cfg::B_BYTES + (uint32_t)atoms * 1024u);
          tma_load_2d(sB + s * Cfg::B_BYTES, &tmB, kc, nt * BN, &full[s]);
          if constexpr (Cfg::SF_ATOMS > 0)
            bulk_load(sSFB + s * Cfg::SF_BYTES, p.sfb + ((size_t)nt * p.sf_col_tiles + (size_t)kt * Cfg::SF_ATOMS) * 512,
                      atoms * 512, &full[s]);
        }
        if (what & 2) {
          tma_load_2d(sA + s * Cfg::A_BYTES, &tmA, kc, mt * BM, &full[s]);
          if constexpr (Cfg::SF_ATOMS > 0)
            bulk_load(sSFA + s * Cfg::SF_BYTES, p.sfa + ((size_t)mt * p.sf_col_tiles + (size_t)kt * Cfg::SF_ATOMS) * 512,
                      atoms * 512, &full[s]);
        }
      };
      // the weights do not depend on the kernel before this one: their first tiles go out before the dependency wait
      const int pre = min(STAGES, nkb);
      for (int i = 0; i < pre; ++i) issue(i, kb0 + i, 1);
      pdl_wait();
      int s = 0; uint32_t ph = 0;
      for (int i = 0; i < nkb; ++i) {
        if (i < pre) {
          issue(s, kb0 + i, 2);
        } else {
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status)) break;
          issue(s, kb0 + i, 3);
        }
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
      SK_MARK(8);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      int s = 0; uint32_t ph = 0;
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        const int kt = kb0 + i;
        if (!mbar_wait(&full[s], ph, abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        if (i == 0) SK_STAMP(2);
        const uint32_t a_addr = smem_u32(sA + s * Cfg::A_BYTES), b_addr = smem_u32(sB + s * Cfg::B_BYTES);
        const int nblk = min(4, (p.K - kt * BK + Cfg::KMMA - 1) / Cfg::KMMA);
        const uint32_t sf_t = tmem + Cfg::SF_COL0 + s * Cfg::SF_COLS_PER_STAGE;
        if constexpr (Cfg::SF_ATOMS > 0) {
          const int atoms = min(Cfg::SF_ATOMS, p.sf_col_tiles - kt * Cfg::SF_ATOMS);
          for (int a = 0; a < atoms; ++a) {
            tmem_cp_sf(sf_t + a * 4, make_smem_desc(smem_u32(sSFA + s * Cfg::SF_BYTES + a * 512), 0, 128, kSwzNone));
            tmem_cp_sf(sf_t + Cfg::SF_ATOMS * 4 + a * 4,
                       make_smem_desc(smem_u32(sSFB + s * Cfg::SF_BYTES + a * 512), 0, 128, kSwzNone));
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (j < nblk) {
            const uint64_t da = desc_sw128(a_addr + j * 32), db = desc_sw128(b_addr + j * 32);
            const uint32_t acc = (i > 0 || j > 0) ? 1u : 0u;
            if constexpr (KIND == 0) {
              mma_f16(tmem, da, db, make_idesc(1, 1, BM, BN), acc);
            } else if constexpr (KIND == 3) {
              mma_f8(tmem, da, db, make_idesc(0, 0, BM, BN), acc);
            } else if constexpr (KIND == 1) {
              mma_nvfp4(tmem, da, db, make_idesc_bs(1, 1, 0, BM, BN), sf_t + j * 4, sf_t + Cfg::SF_ATOMS * 4 + j * 4, acc);
            } else {
              mma_mxf8(tmem, da, db, make_idesc_bs(0, 0, 1, BM, BN, j, j), sf_t, sf_t + Cfg::SF_ATOMS * 4, acc);
            }
          }
        }
        mma_commit(&empty[s]);
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
      if (ok) mma_commit(acc_full);
      SK_MARK(16);
      SK_STAMP(3);
    }
  }
  __syncwarp();
  if (ks > 1) cluster_wait();               // all threads, unconditionally (pairs with cluster_arrive above)
  if (threadIdx.x == 64) SK_MARK(32);

  if (warp >= 2) {
    // ------------------------------------------------------------------ epilogue / reducers (128 threads)
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int rl = q * 32 + lane;           // row of the tile owned by this thread
    const int row = mt * BM + rl;
    const bool in_range = row < p.M;
    // per-column multipliers and bias of this tile, staged once while the main loop runs
    {
      const int col = nt * BN + rl;
      s_alpha[rl] = (p.alpha && col < p.N) ? __ldg(p.alpha + col) : 1.0f;
      s_bias[rl] = (p.bias && col < p.N) ? bf2f(p.bias[col]) : 0.0f;
    }
    const float rs = (p.row_scale && in_range) ? p.row_scale[row] : 1.0f;
    bar_sync(1, 128);
    pdl_wait();                             // C may still be read by the kernel before this one
    // tcgen05.ld is warp-collective: every lane of the warp must take the same path through the loads below, so the
    // outcome of the wait is made warp-uniform and only the global stores are predicated on the row being in range
    const bool got = __all_sync(0xffffffffu, mbar_wait(acc_full, 0, abort_flag, p.status));
    tc_fence_after();
    if (threadIdx.x == 64) { SK_MARK(got ? 64 : 0x10000); SK_STAMP(4); }
    // finished values of one group of columns [col0, col0 + n) of this thread's row -> scales, bias, activation, store
    auto finish = [&](float* v, int col0_tile, int n) {
      const int col0 = nt * BN + col0_tile;
      if (!in_range || col0 >= p.N) return;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < n) v[i] = fmaf(v[i] * rs, s_alpha[col0_tile + i], s_bias[col0_tile + i]);
      const bool vec = (p.ldc & 7) == 0 && col0 + n <= p.N;
      if (p.act) {               // n == 32: [16 gate | 16 up] -> 16 outputs
        __nv_bfloat16* dst = p.C + (size_t)row * p.ldc + col0 / 2;
        uint32_t pk[8];
#pragma unroll
        for (int i = 0; i < 16; i += 2) pk[i / 2] = pack_bf16x2(silu_mul_bf16(v[i], v[16 + i]), silu_mul_bf16(v[i + 1], v[17 + i]));
        if (vec) {
          *reinterpret_cast<uint4*>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          *reinterpret_cast<uint4*>(dst + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
        return;
      }
      __nv_bfloat16* dst = p.C + (size_t)row * p.ldc + col0;
      if (vec) {
#pragma unroll
        for (int i = 0; i < 32; i += 8)
          if (i < n)
            *reinterpret_cast<uint4*>(dst + i) = make_uint4(pack_bf16x2(v[i], v[i + 1]), pack_bf16x2(v[i + 2], v[i + 3]),
                                                            pack_bf16x2(v[i + 4], v[i + 5]), pack_bf16x2(v[i + 6], v[i + 7]));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < n && col0 + i < p.N) dst[i] = __float2bfloat16(v[i]);
      }
    };
    if (ks == 1) {
      if (got) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem + c * 32 + ((uint32_t)(q * 32) << 16), r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          finish(v, c * 32, 32);
        }
      }
      if (threadIdx.x == 64) SK_STAMP(7);
    } else {
      // ---- reduction over the cluster by pushing: the tile's columns are cut into groups (8 columns; 32 with the SwiGLU
      //      epilogue, which needs a gate group and its up group together); CTA r of the cluster owns the groups
      //      [r * ng / ks, (r + 1) * ng / ks) and receives every CTA's partial of them in its own shared memory (the operand
      //      ring, free once every CTA of the cluster has finished its main loop), slot [source CTA][group][column quad][row].
      //      Remote stores are posted, so nobody waits on a round trip per value; the owner then sums its slots in
      //      source-rank order from local shared memory.
      const int gw = p.act ? 32 : 8, ng = BN / gw, qpg = gw / 4;          // group width, groups per tile, quads per group
      const int GL = (ng + ks - 1) / ks;                                   // most groups any CTA owns
      const uint32_t ring_addr = smem_u32(ring_free), ready_addr = smem_u32(part_ready), recv_addr = smem_u32(smem);
      if (threadIdx.x == 64) {
        for (int r = 0; r < ks; ++r) mbar_arrive_remote(mapa_shared(ring_addr, r));
      }
      // an aborted CTA still arrives and still waits, so that its peers are not left waiting for it
      const bool free_all = __all_sync(0xffffffffu, mbar_wait_cluster(ring_free, 0, abort_flag, p.status));
      if (threadIdx.x == 64) { SK_MARK(128); SK_STAMP(5); }
      if (got && free_all) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem + c * 32 + ((uint32_t)(q * 32) << 16), r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int cq = c * 8 + j;                        // column quad of the tile
            const int g = cq / qpg, jq = cq % qpg;
            const int owner = (g * ks + ks - 1) / ng;        // the r with r * ng / ks <= g < (r + 1) * ng / ks
            const int gl = g - owner * ng / ks;
            const uint32_t dst = mapa_shared(recv_addr + (uint32_t)(((kr * GL + gl) * qpg + jq) * BM + rl) * 16u, owner);
            st_dsmem_f4(dst, __uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                        __uint_as_float(r[4 * j + 3]));
          }
        }
      }
      fence_acq_rel_cluster();
      bar_sync(1, 128);
      if (threadIdx.x == 64) {
        for (int r = 0; r < ks; ++r) mbar_arrive_remote(mapa_shared(ready_addr, r));
      }
      const bool all = mbar_wait_cluster(part_ready, 0, abort_flag, p.status);
      if (threadIdx.x == 64) { SK_MARK(all ? 256 : 0x20000); SK_STAMP(6); }
      if (all && got && free_all && !*abort_flag) {
        const int g0 = kr * ng / ks, g1 = (kr + 1) * ng / ks;
        const float4* recv = reinterpret_cast<const float4*>(smem);
        for (int g = g0; g < g1; ++g) {
          float v[32];
#pragma unroll
          for (int jq = 0; jq < 8; ++jq) {
            if (jq < qpg) {
              float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
              for (int r = 0; r < ks; ++r) {          // source-rank order: the sum does not depend on timing
                const float4 a = recv[((r * GL + (g - g0)) * qpg + jq) * BM + rl];
                acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
              }
              v[4 * jq] = acc.x; v[4 * jq + 1] = acc.y; v[4 * jq + 2] = acc.z; v[4 * jq + 3] = acc.w;
            }
          }
          finish(v, g * gw, gw);
        }
      }
      if (threadIdx.x == 64) { SK_MARK(512); SK_STAMP(7); }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
    if (lane == 0) SK_MARK(2048);
  }
  if (threadIdx.x == 0) SK_STAMP(9);
}

template <int KIND>
static void fill_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int grid, int ks, cudaStream_t stream) {
  cfg = cudaLaunchConfig_t{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = SkCfg<KIND>::SMEM;
  cfg.stream = stream;
  int n = 0;
  if (ks > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = ks;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
}

template <int KIND>
static cudaError_t launch_sk(const CUtensorMap& tmA, const CUtensorMap& tmB, const SkParams& p, cudaStream_t stream) {
  auto kern = gemm_sk_kernel<KIND>;
  static PerDeviceOnce configured;
  {
    cudaError_t e = configured.smem_limit(kern, SkCfg<KIND>::SMEM);
    if (e != cudaSuccess) return e;
  }
  const int tiles = ((p.M + 127) / 128) * ((p.N + 127) / 128);
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  fill_config<KIND>(cfg, attr, tiles * p.ks, p.ks, stream);
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, p);
}

// How many CTAs of this kernel run at the same time on the current device when launched in clusters of `ks` (clusters are
// placed whole inside one GPC, so this can be less than 2 x SMs).  Cached per device and cluster size.
template <int KIND>
static int coresident_ctas(int ks) {
  static int cache[64][9] = {{0}};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || ks < 1 || ks > 8) return 2 * sm_count();
  if (cache[dev][ks]) return cache[dev][ks];
  auto kern = gemm_sk_kernel<KIND>;
  static PerDeviceOnce configured;
  int n = 0;
  if (configured.smem_limit(kern, SkCfg<KIND>::SMEM) == cudaSuccess) {
    if (ks == 1) {
      int per_sm = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 192, SkCfg<KIND>::SMEM) == cudaSuccess) n = per_sm * sm_count();
    } else {
      cudaLaunchConfig_t cfg;
      cudaLaunchAttribute attr[2];
      fill_config<KIND>(cfg, attr, ks * sm_count(), ks, nullptr);
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) == cudaSuccess) n = clusters * ks;
    }
  }
  if (n <= 0) n = sm_count();
  cache[dev][ks] = n;
  return n;
}

static int coresident(int kind, int ks) {
  switch (kind) {
    case 0: return coresident_ctas<0>(ks);
    case 1: return coresident_ctas<1>(ks);
    case 2: return coresident_ctas<2>(ks);
    default: return coresident_ctas<3>(ks);
  }
}

// K slices for a GEMM of `tiles` output tiles and `k_tiles` k-blocks: the most slices (at most `max_ks`, never more than
// k-blocks) whose CTAs all run at the same time; a grid that needs a second wave is not worth splitting.
static int choose_ks(int kind, int tiles, int k_tiles, int max_ks) {
  int best = 1;
  for (int ks = 2; ks <= max_ks && ks <= k_tiles; ++ks)
    if ((long)tiles * ks <= coresident(kind, ks)) best = ks;
  return best;
}

}  // namespace blz

namespace { thread_local unsigned* g_sk_dbg = nullptr; thread_local unsigned long long* g_sk_prof = nullptr; }
// Diagnostics: the NEXT blz_gemm_sk call records per CTA, in prof[blockIdx.x][16], global-timer stamps (ns): 0 entry, 1 set-up
// done, 2 first operands landed, 3 last MMA issued, 4 accumulator complete, 5 partial parked, 6 all partials ready, 7 slice
// reduced and stored, 8 peers done reading, 9 exit.
BLZ_API int blz_gemm_sk_profile(void* prof) { g_sk_prof = reinterpret_cast<unsigned long long*>(prof); return 0; }
// Diagnostics: the NEXT blz_gemm_sk call on this thread records, per CTA, which stages it reached as bits of dbg[blockIdx.x]
// (1 barriers set up, 2 tensor memory held, 4 cluster arrive, 8 loads issued, 16 MMAs issued, 32 cluster barrier passed,
// 64 accumulator complete, 128 partial parked, 256 all partials ready, 512 slice reduced, 1024 peers done reading,
// 2048 tensor memory released; 0x10000 / 0x20000 / 0x40000: the matching wait gave up).  dbg needs tiles * ks words.
BLZ_API int blz_gemm_sk_debug(void* dbg) { g_sk_dbg = reinterpret_cast<unsigned*>(dbg); return 0; }

// The K-slice count blz_gemm_sk would pick for this shape on the current device (what an autotuner varies around).
BLZ_API int blz_gemm_sk_default_ks(int kind, int M, int N, int K) {
  using namespace blz;
  if (M <= 0 || N <= 0 || K <= 0 || kind < 0 || kind > 3) return 0;
  const int bk = (kind == 0 ? 16 : kind == 1 ? 64 : 32) * 4;
  return choose_ks(kind, ((M + 127) / 128) * ((N + 127) / 128), (K + bk - 1) / bk, 8);
}

// CTAs of the kernel that run at the same time when launched in clusters of ks (what a grid should stay under).
BLZ_API int blz_gemm_sk_coresident(int kind, int ks) {
  if (kind < 0 || kind > 3 || ks < 1 || ks > 8) return 0;
  return blz::coresident(kind, ks);
}

// kind: 0 bf16, 1 nvfp4, 2 mxfp8, 3 fp8.  A [M, K] and B [N, K] row-major (packed bytes for 4/8-bit kinds); lda / ldb in
// BYTES; C bf16 with ldc in elements.  ks: K slices = cluster size, 1..8 (0 = choose).  act = 1: SwiGLU epilogue as in
// blz_gemm_tc (needs ks <= 4, N % 32 == 0 and ldc % 8 == 0).
BLZ_API int blz_gemm_sk(int kind, const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc, int M,
                        int N, int K, const float* row_scale, const float* alpha, const void* bias, const void* sfa,
                        const void* sfb, int ks, int act, cudaStream_t stream) {
  using namespace blz;
  if (M <= 0 || N <= 0 || K <= 0 || kind < 0 || kind > 3 || ks < 0 || ks > 8) return (int)cudaErrorInvalidValue;
  const int kmma = kind == 0 ? 16 : kind == 1 ? 64 : 32;
  if (K % kmma) return (int)cudaErrorInvalidValue;
  if ((kind == 1 || kind == 2) && (!sfa || !sfb)) return (int)cudaErrorInvalidValue;
  if (act && (N % 32 || (ldc & 7) || ks > 4)) return (int)cudaErrorInvalidValue;
  const int k_tiles = (K + kmma * 4 - 1) / (kmma * 4);
  const int tiles = ((M + 127) / 128) * ((N + 127) / 128);
  if (ks == 0) ks = choose_ks(kind, tiles, k_tiles, act ? 4 : 8);
  if (ks > k_tiles) ks = k_tiles;
  SkParams p;
  p.M = M; p.N = N; p.K = K; p.C = reinterpret_cast<__nv_bfloat16*>(C); p.ldc = ldc;
  p.row_scale = row_scale; p.alpha = alpha; p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.sfa = reinterpret_cast<const uint8_t*>(sfa); p.sfb = reinterpret_cast<const uint8_t*>(sfb);
  p.sf_col_tiles = kind == 1 ? (K + 63) / 64 : kind == 2 ? (K + 127) / 128 : 0;
  p.ks = ks; p.act = act;
  p.status = status_word();
  p.dbg = g_sk_dbg;
  g_sk_dbg = nullptr;
  p.prof = g_sk_prof;
  g_sk_prof = nullptr;
  CUtensorMap tmA, tmB;
  cudaError_t e;
  if (kind == 0) {
    e = encode_tmap(&tmA, A, 2, K, M, lda, 64, 128, 3);
    if (e != cudaSuccess) return (int)e;
    e = encode_tmap(&tmB, B, 2, K, N, ldb, 64, 128, 3);
  } else {
    const uint64_t kbytes = kind == 1 ? K / 2 : K;
    e = encode_tmap(&tmA, A, 1, kbytes, M, lda, 128, 128, 3);
    if (e != cudaSuccess) return (int)e;
    e = encode_tmap(&tmB, B, 1, kbytes, N, ldb, 128, 128, 3);
  }
  if (e != cudaSuccess) return (int)e;
  switch (kind) {
    case 0: return (int)launch_sk<0>(tmA, tmB, p, stream);
    case 1: return (int)launch_sk<1>(tmA, tmB, p, stream);
    case 2: return (int)launch_sk<2>(tmA, tmB, p, stream);
    default: return (int)launch_sk<3>(tmA, tmB, p, stream);
  }
}
