// Grouped expert GEMM for decode-sized routing (a few rows per expert), features on the tensor-core lanes:
//     C[row, f] = (X[row, :] · W_e[f, :]) * row_scale[row] * alpha[e * N + f]      for the rows routed to expert e
// The routed rows sit in a padded row space where every expert starts on a 128-row boundary (moe_plan / moe_scatter), so a
// "row tile" (128 rows) belongs to one expert and holds `tile_rows[mt]` live rows, usually 8-32.  One CTA computes one
// (row tile, 128-feature tile): the weight tile is the MMA's 128-lane operand, the live rows, rounded up to 32, are its
// column operand (N = 32 .. 128), so a tile with 16 live rows costs 16 KB of weights + 4 KB of activations per K block
// instead of 16 KB + 16 KB of mostly padding, and a quarter of the tensor-core time.  Expert weights are read exactly once
// per step whatever the routing.
//
// Epilogue variants: plain bf16 rows, or (act = 1) SwiGLU on a weight whose rows are interleaved [16 gate | 16 up]: the
// gate and up value of one feature sit 16 lanes apart in the same warp, one shuffle joins them and the [rows, 2I]
// intermediate never reaches memory.
//
// The same kernel serves dense layers at small batch (at most 128 rows, e.g. single-user decoding or a verify step):
// tile_expert = null means one "expert" whose rows are the whole activation matrix.  Few rows mean few feature tiles and a
// long K range per tile, so the K range can be split over a thread-block cluster of `ks` CTAs: each streams 1/ks of the
// weights of its feature tile, and the fp32 partials (128 features x 32..128 rows, a few KB) meet in distributed shared
// memory: every CTA owns a slice of the row columns, receives all peers' partials of that slice with posted remote stores,
// sums them in CTA-rank order (bit-reproducible) and writes the result.
//
// A CTA of the expert GEMM computes `ft_per` feature tiles of its row tile one after the other: the operand ring keeps
// streaming across them, and while the epilogue drains one accumulator (64 TMEM columns when the tile has at most 64 live
// rows) the MMAs of the next tile fill the other, so set-up and drain are paid once per CTA instead of once per 8 K blocks.
//
// 192 threads: warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-5 = epilogue.  Two CTAs per SM (3-stage ring).  Every
// wait is a bounded mbarrier wait; the hardware cluster barrier is used once, right after barrier initialisation, where no
// role can have failed yet.  No TMA load is cluster-multicast.
//
// Reference counterparts: kernels/src/cuda/moe_narrow.cu (per-expert small-m kernels, :171-484) and moe_wide.cu (:125-313).
#include "blaze/host.h"
#include "blaze/sm100.cuh"

namespace blz {

struct MoeGemmParams {
  int N, K;                  // features per expert, reduction length (elements)
  __nv_bfloat16* C;          // [padded rows, ldc]
  long long ldc;
  const float* row_scale;    // [padded rows] or null
  const float* alpha;        // [experts * N] or null
  const uint8_t* sfw;        // weight scale factors, 128x4-tiled over [experts * N] rows
  const uint8_t* sfx;        // activation scale factors, 128x4-tiled over the padded rows
  int sf_col_tiles;
  const int* tile_expert;    // [row tiles] expert of the tile, -1 = unused; null = dense layer (one row tile of `rows` rows)
  const int* tile_rows;      // [row tiles] live rows of the tile
  int rows;                  // dense layer: rows of the activation matrix (<= 128)
  const __nv_bfloat16* bias; // [N] or null (dense layers)
  int ks;                    // cluster size = K slices (1 = no cluster)
  int ft_per;                // feature tiles one CTA computes one after the other (1 when ks > 1)
  int act;                   // 1: SwiGLU epilogue, C is [rows, N / 2]
  int* status;
};

template <int KIND> struct MgKind;
template <> struct MgKind<0> { static constexpr int KMMA = 16, SF_ATOMS = 0; };
template <> struct MgKind<1> { static constexpr int KMMA = 64, SF_ATOMS = 4; };
template <> struct MgKind<2> { static constexpr int KMMA = 32, SF_ATOMS = 1; };

template <int KIND>
struct MgCfg {
  static constexpr int KMMA = MgKind<KIND>::KMMA;
  static constexpr int BK = KMMA * 4;                  // 128 bytes per operand row per stage
  static constexpr int W_BYTES = 128 * 128, X_BYTES = 128 * 128;
  static constexpr int SF_ATOMS = MgKind<KIND>::SF_ATOMS;
  static constexpr int SF_BYTES = SF_ATOMS * 512;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES + 2 * SF_BYTES;
  static constexpr int STAGES = 3;
  static constexpr int SF_COLS_PER_STAGE = SF_ATOMS * 4 * 2;
  static constexpr int SF_COL0 = 128;
  static constexpr int TMEM_COLS = 256;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256 + 128 * 4;
  static constexpr int PART_BYTES = 8 * 2 * 128 * 16 * 2;       // most the cluster reduction receives: 8 sources x 2 groups of 8 columns
  static_assert(SF_COL0 + STAGES * SF_COLS_PER_STAGE <= TMEM_COLS, "TMEM budget");
  static_assert(2 * (SMEM + 1024) <= 228 * 1024, "two CTAs per SM");
  static_assert(PART_BYTES <= STAGES * (W_BYTES + X_BYTES), "the partials must fit the operand ring");
};

__device__ __forceinline__ float mg_silu_mul(float g, float u) {
  g = bf2f(__float2bfloat16(g));
  u = bf2f(__float2bfloat16(u));
  return g / (1.f + __expf(-g)) * u;
}

template <int KIND>
__global__ void __launch_bounds__(192, 2)
moe_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, MoeGemmParams p) {
  using Cfg = MgCfg<KIND>;
  constexpr int BK = Cfg::BK, STAGES = Cfg::STAGES;
  const int tiles_n = p.N / 128;
  const int ks = p.ks;
  const int unit = blockIdx.x / ks;                      // (row tile, feature tile); the cluster's CTAs share it
  const int kr = ks > 1 ? (int)cluster_ctarank() : 0;
  const int groups_n = (tiles_n + p.ft_per - 1) / p.ft_per;
  const int ft0 = (unit % groups_n) * p.ft_per, mt = unit / groups_n;
  const int nf = min(p.ft_per, tiles_n - ft0);           // feature tiles of this CTA
  const int ex = p.tile_expert ? p.tile_expert[mt] : 0;
  const int rows = ex < 0 ? 0 : min(p.tile_expert ? p.tile_rows[mt] : p.rows, 128);
  if (rows <= 0) return;                    // whole cluster, before anything is allocated
  const int ncols = (rows + 31) & ~31;      // MMA N: 32, 64, 96 or 128
  const int nb = ncols <= 64 ? 2 : 1;       // accumulators in flight (64 TMEM columns apart)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sW = smem;
  uint8_t* sX = sW + STAGES * Cfg::W_BYTES;
  uint8_t* sSFW = sX + STAGES * Cfg::X_BYTES;
  uint8_t* sSFX = sSFW + STAGES * Cfg::SF_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sSFX + STAGES * Cfg::SF_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;   // [2] a feature tile's accumulator is complete
  uint64_t* acc_empty = acc_full + 2;       // [2] the epilogue has read it (4 arrivals)
  uint64_t* part_ready = acc_empty + 2;     // every CTA of the cluster has parked its partials (ks remote arrivals)
  uint64_t* ring_free = part_ready + 1;     // every CTA of the cluster has finished its main loop (its ring may be written)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ring_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_rs = reinterpret_cast<float*>(bars) + 64;       // [128] row scales of this tile (after 256 bytes of barriers)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_tiles = (p.K + BK - 1) / BK;
  const int kb0 = (int)((long long)kr * k_tiles / ks), kb1 = (int)((long long)(kr + 1) * k_tiles / ks);
  const int nkb = kb1 - kb0;                // >= 1: the launcher keeps ks <= k_tiles
  const size_t wbase = (size_t)ex * p.N;    // first weight row of this expert

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    mbar_init(part_ready, ks);
    mbar_init(ring_free, ks);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmW);
    prefetch_tmap(&tmX);
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_trigger();
  if (ks > 1) cluster_arrive();             // the peers' barriers are initialised before anyone arrives on them remotely
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      auto issue = [&](int s, int kt, int what, size_t wrow0) {
        int atoms = 0;
        if constexpr (Cfg::SF_ATOMS > 0) atoms = min(Cfg::SF_ATOMS, p.sf_col_tiles - kt * Cfg::SF_ATOMS);
        const int kc = (KIND == 0) ? kt * BK : kt * 128;
        if (what & 1) {       // weights: do not depend on the kernel before this one
          mbar_expect_tx(&full[s], Cfg::W_BYTES + (uint32_t)ncols * 128u + (uint32_t)atoms * 1024u);
          tma_load_2d(sW + s * Cfg::W_BYTES, &tmW, kc, (int)wrow0, &full[s]);
          if constexpr (Cfg::SF_ATOMS > 0)
            bulk_load(sSFW + s * Cfg::SF_BYTES, p.sfw + ((wrow0 >> 7) * p.sf_col_tiles + (size_t)kt * Cfg::SF_ATOMS) * 512,
                      atoms * 512, &full[s]);
        }
        if (what & 2) {       // routed rows, 32 at a time
          for (int c = 0; c < ncols; c += 32)
            tma_load_2d(sX + s * Cfg::X_BYTES + c * 128, &tmX, kc, mt * 128 + c, &full[s]);
          if constexpr (Cfg::SF_ATOMS > 0)
            bulk_load(sSFX + s * Cfg::SF_BYTES, p.sfx + ((size_t)mt * p.sf_col_tiles + (size_t)kt * Cfg::SF_ATOMS) * 512,
                      atoms * 512, &full[s]);
        }
      };
      const int pre = min(STAGES, nkb);
      for (int i = 0; i < pre; ++i) issue(i, kb0 + i, 1, wbase + (size_t)ft0 * 128);
      pdl_wait();
      int s = 0; uint32_t ph = 0;
      bool ok = true;
      for (int fi = 0; fi < nf && ok; ++fi) {
        const size_t wrow0 = wbase + (size_t)(ft0 + fi) * 128;
        for (int i = 0; i < nkb; ++i) {
          if (fi == 0 && i < pre) {
            issue(s, kb0 + i, 2, wrow0);
          } else {
            if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status)) { ok = false; break; }
            issue(s, kb0 + i, 3, wrow0);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      int s = 0; uint32_t ph = 0;
      bool ok = true;
      for (int fi = 0; fi < nf && ok; ++fi) {
        const int ab = fi % nb;
        // accumulator ab was last filled for tile fi - nb: its read-out is completion number (fi / nb - 1) of acc_empty[ab]
        if (fi >= nb && !mbar_wait(&acc_empty[ab], (uint32_t)((fi / nb - 1) & 1), abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem + ab * 64;
        for (int i = 0; i < nkb; ++i) {
          if (!mbar_wait(&full[s], ph, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t w_addr = smem_u32(sW + s * Cfg::W_BYTES), x_addr = smem_u32(sX + s * Cfg::X_BYTES);
          const int kt = kb0 + i;
          const int nblk = min(4, (p.K - kt * BK + Cfg::KMMA - 1) / Cfg::KMMA);
          const uint32_t sf_t = tmem + Cfg::SF_COL0 + s * Cfg::SF_COLS_PER_STAGE;      // weights' scales, then the rows' scales
          if constexpr (Cfg::SF_ATOMS > 0) {
            const int atoms = min(Cfg::SF_ATOMS, p.sf_col_tiles - kt * Cfg::SF_ATOMS);
            for (int a = 0; a < atoms; ++a) {
              tmem_cp_sf(sf_t + a * 4, make_smem_desc(smem_u32(sSFW + s * Cfg::SF_BYTES + a * 512), 0, 128, kSwzNone));
              tmem_cp_sf(sf_t + Cfg::SF_ATOMS * 4 + a * 4,
                         make_smem_desc(smem_u32(sSFX + s * Cfg::SF_BYTES + a * 512), 0, 128, kSwzNone));
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (j < nblk) {
              const uint64_t dw = desc_sw128(w_addr + j * 32), dx = desc_sw128(x_addr + j * 32);
              const uint32_t acc = (i > 0 || j > 0) ? 1u : 0u;
              if constexpr (KIND == 0) {
                mma_f16(d_tmem, dw, dx, make_idesc(1, 1, 128, ncols), acc);
              } else if constexpr (KIND == 1) {
                mma_nvfp4(d_tmem, dw, dx, make_idesc_bs(1, 1, 0, 128, ncols), sf_t + j * 4, sf_t + Cfg::SF_ATOMS * 4 + j * 4, acc);
              } else {
                mma_mxf8(d_tmem, dw, dx, make_idesc_bs(0, 0, 1, 128, ncols, j, j), sf_t, sf_t + Cfg::SF_ATOMS * 4, acc);
              }
            }
          }
          mma_commit(&empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) mma_commit(&acc_full[ab]);
      }
    }
  }
  __syncwarp();
  if (ks > 1) cluster_wait();               // all threads, unconditionally (pairs with cluster_arrive above)
  if (warp >= 2) {
    // ------------------------------------------------------------------ epilogue: lane = feature, column = routed row
    const int q = warp & 3;
    const int fl = q * 32 + lane;                       // feature of this thread inside the tile
    int ft = ft0;                                       // feature tile being finished
    float al = p.alpha ? __ldg(p.alpha + wbase + (size_t)ft * 128 + fl) : 1.0f;
    float bs = p.bias ? bf2f(p.bias[ft * 128 + fl]) : 0.0f;
    pdl_wait();
    s_rs[fl] = (p.row_scale && fl < rows) ? p.row_scale[(size_t)mt * 128 + fl] : 1.0f;
    bar_sync(1, 128);
    // tcgen05.ld is warp-collective: the outcome of the wait is made warp-uniform, only the stores are predicated
    bool got = __all_sync(0xffffffffu, mbar_wait(&acc_full[0], 0, abort_flag, p.status));
    tc_fence_after();
    // finished sums of this thread's feature for the row columns [c0, c0 + n): scales, bias, activation, store.
    // Called by all lanes of a warp with the same c0 and n.
    auto finish = [&](const float* v, int c0, int n) {
      if (p.act) {
        // lanes 0-15 hold the gate, lanes 16-31 the up value of 16 features: one exchange joins them
        const int fo = (ft * 128 + q * 32) / 2 + (lane & 15);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (j < n) {
            const float x = fmaf(v[j] * al, s_rs[c0 + j], bs);
            const float o = __shfl_xor_sync(0xffffffffu, x, 16);
            if (lane < 16 && c0 + j < rows) p.C[((size_t)mt * 128 + c0 + j) * p.ldc + fo] = __float2bfloat16(mg_silu_mul(x, o));
          }
        }
      } else {
        const int f = ft * 128 + fl;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < n && c0 + j < rows) p.C[((size_t)mt * 128 + c0 + j) * p.ldc + f] = __float2bfloat16(fmaf(v[j] * al, s_rs[c0 + j], bs));
      }
    };
    if (ks == 1) {
      for (int fi = 0; fi < nf && got; ++fi) {
        const int ab = fi % nb;
        if (fi > 0) {
          ft = ft0 + fi;
          al = p.alpha ? __ldg(p.alpha + wbase + (size_t)ft * 128 + fl) : 1.0f;
          bs = p.bias ? bf2f(p.bias[ft * 128 + fl]) : 0.0f;
          got = __all_sync(0xffffffffu, mbar_wait(&acc_full[ab], (uint32_t)((fi / nb) & 1), abort_flag, p.status));
          tc_fence_after();
          if (!got) break;
        }
        for (int c = 0; c < ncols; c += 32) {
          uint32_t r[32];
          tmem_ld32(tmem + ab * 64 + c + ((uint32_t)(q * 32) << 16), r);
          tmem_ld_wait();
          if (c + 32 >= ncols) {       // the accumulator is in registers: hand it back before the stores
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[ab]);
          }
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          finish(v, c, 32);
        }
      }
    } else {
      // ---- reduction over the cluster by pushing: the row columns are cut into groups of 8; CTA r of the cluster owns the
      //      groups [r * ng / ks, (r + 1) * ng / ks) and receives every CTA's partials of them in its own shared memory (the
      //      operand ring, free once every CTA of the cluster has finished its main loop), slot [source CTA][group][column
      //      quad][feature].  Remote stores are posted; the owner then sums its slots in source-rank order.
      constexpr int gw = 8, qpg = 2;
      const int ng = ncols / gw;
      const int GL = (ng + ks - 1) / ks;
      const uint32_t ring_addr = smem_u32(ring_free), ready_addr = smem_u32(part_ready), recv_addr = smem_u32(smem);
      if (threadIdx.x == 64) {
        for (int r = 0; r < ks; ++r) mbar_arrive_remote(mapa_shared(ring_addr, r));
      }
      // an aborted CTA still arrives and still waits, so that its peers are not left waiting for it
      const bool free_all = __all_sync(0xffffffffu, mbar_wait_cluster(ring_free, 0, abort_flag, p.status));
      if (got && free_all) {
        for (int c = 0; c < ncols / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem + c * 32 + ((uint32_t)(q * 32) << 16), r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int cq = c * 8 + j;                        // column quad of the tile
            const int g = cq / qpg, jq = cq % qpg;
            const int owner = (g * ks + ks - 1) / ng;        // the r with r * ng / ks <= g < (r + 1) * ng / ks
            const int gl = g - owner * ng / ks;
            const uint32_t dst = mapa_shared(recv_addr + (uint32_t)(((kr * GL + gl) * qpg + jq) * 128 + fl) * 16u, owner);
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
      const bool all = __all_sync(0xffffffffu, mbar_wait_cluster(part_ready, 0, abort_flag, p.status));
      if (all && got && free_all && !*abort_flag) {
        const int g0 = kr * ng / ks, g1 = (kr + 1) * ng / ks;
        const float4* recv = reinterpret_cast<const float4*>(smem);
        for (int g = g0; g < g1; ++g) {
          float v[8];
#pragma unroll
          for (int jq = 0; jq < qpg; ++jq) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < ks; ++r) {          // source-rank order: the sum does not depend on timing
              const float4 a = recv[((r * GL + (g - g0)) * qpg + jq) * 128 + fl];
              acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
            }
            v[4 * jq] = acc.x; v[4 * jq + 1] = acc.y; v[4 * jq + 2] = acc.z; v[4 * jq + 3] = acc.w;
          }
          finish(v, g * gw, gw);
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

template <int KIND>
static cudaError_t launch_moe_gemm(const CUtensorMap& tmW, const CUtensorMap& tmX, const MoeGemmParams& p, int row_tiles,
                                   cudaStream_t stream) {
  const int ks = p.ks;
  auto kern = moe_gemm_kernel<KIND>;
  static PerDeviceOnce configured;
  cudaError_t e = configured.smem_limit(kern, MgCfg<KIND>::SMEM);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  const int groups_n = (p.N / 128 + p.ft_per - 1) / p.ft_per;
  cfg.gridDim = dim3((unsigned)(row_tiles * groups_n * ks));
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = MgCfg<KIND>::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
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
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p);
}

}  // namespace blz

// kind: 0 bf16, 1 nvfp4, 2 mxfp8.  X: routed rows [row_tiles * 128, K] in the padded row space (packed bytes for 4/8-bit
// kinds, ldx in bytes); W: stacked expert weights [experts * N, K] (ldw in bytes); C bf16 [row_tiles * 128, ldc].
// N % 128 == 0.  act = 1: SwiGLU on [16 gate | 16 up] interleaved weight rows, C is [rows, N / 2].
BLZ_API int blz_moe_gemm(int kind, const void* X, long long ldx, const void* W, long long ldw, void* C, long long ldc,
                         int row_tiles, int N, int K, int experts, const float* row_scale, const float* alpha, const void* sfx,
                         const void* sfw, const int* tile_expert, const int* tile_rows, int act, cudaStream_t stream) {
  using namespace blz;
  if (row_tiles <= 0) return 0;
  if (N <= 0 || K <= 0 || kind < 0 || kind > 2 || N % 128 || experts <= 0 || !tile_expert || !tile_rows)
    return (int)cudaErrorInvalidValue;
  const int kmma = kind == 0 ? 16 : kind == 1 ? 64 : 32;
  if (K % kmma) return (int)cudaErrorInvalidValue;
  if ((kind == 1 || kind == 2) && (!sfx || !sfw)) return (int)cudaErrorInvalidValue;
  MoeGemmParams p;
  p.N = N; p.K = K; p.C = reinterpret_cast<__nv_bfloat16*>(C); p.ldc = ldc;
  p.row_scale = row_scale; p.alpha = alpha;
  p.sfw = reinterpret_cast<const uint8_t*>(sfw); p.sfx = reinterpret_cast<const uint8_t*>(sfx);
  p.sf_col_tiles = kind == 1 ? (K + 63) / 64 : kind == 2 ? (K + 127) / 128 : 0;
  p.tile_expert = tile_expert; p.tile_rows = tile_rows; p.act = act;
  p.rows = 0; p.bias = nullptr; p.ks = 1;
  {
    // feature tiles per CTA: long enough streams to amortise a CTA's set-up, still at least four CTAs per row tile
    static int forced = -1;
    if (forced < 0) { const char* e = getenv("BLAZE_MOE_FT_PER"); forced = e ? atoi(e) : 0; }
    const int tiles_n = N / 128;
    p.ft_per = forced > 0 ? forced : (tiles_n >= 12 ? (tiles_n % 4 == 0 ? 4 : 3) : (tiles_n >= 6 ? 2 : 1));
    if (p.ft_per > tiles_n) p.ft_per = tiles_n;
  }
  p.status = status_word();
  CUtensorMap tmW, tmX;
  cudaError_t e;
  const uint64_t w_rows = (uint64_t)experts * N, x_rows = (uint64_t)row_tiles * 128;
  if (kind == 0) {
    e = encode_tmap(&tmW, W, 2, K, w_rows, ldw, 64, 128, 3);
    if (e != cudaSuccess) return (int)e;
    e = encode_tmap(&tmX, X, 2, K, x_rows, ldx, 64, 32, 3);
  } else {
    const uint64_t kbytes = kind == 1 ? K / 2 : K;
    e = encode_tmap(&tmW, W, 1, kbytes, w_rows, ldw, 128, 128, 3);
    if (e != cudaSuccess) return (int)e;
    e = encode_tmap(&tmX, X, 1, kbytes, x_rows, ldx, 128, 32, 3);
  }
  if (e != cudaSuccess) return (int)e;
  switch (kind) {
    case 0: return (int)launch_moe_gemm<0>(tmW, tmX, p, row_tiles, stream);
    case 1: return (int)launch_moe_gemm<1>(tmW, tmX, p, row_tiles, stream);
    default: return (int)launch_moe_gemm<2>(tmW, tmX, p, row_tiles, stream);
  }
}

// Dense layer at small batch: C[M, N] = (X[M, K] · W[N, K]^T) * row_scale[m] * alpha[n] (+ bias[n]) for M <= 128 rows, features on
// the MMA lanes, the K range split over a cluster of ks CTAs (0 = choose: enough CTAs to cover the SMs twice, at most 8 and at
// most one K block each).  Rows past M are never read (the tensor map ends at row M, the copy engine fills zeros); the scale
// factors of X must be a whole 128-row tile.  act as in blz_moe_gemm.
BLZ_API int blz_gemm_narrow(int kind, const void* X, long long ldx, const void* W, long long ldw, void* C, long long ldc, int M,
                            int N, int K, const float* row_scale, const float* alpha, const void* bias, const void* sfx,
                            const void* sfw, int ks, int act, cudaStream_t stream) {
  using namespace blz;
  if (M <= 0) return 0;
  if (M > 128 || N <= 0 || K <= 0 || kind < 0 || kind > 2 || N % 128 || ks < 0 || ks > 8) return (int)cudaErrorInvalidValue;
  const int kmma = kind == 0 ? 16 : kind == 1 ? 64 : 32;
  if (K % kmma) return (int)cudaErrorInvalidValue;
  if ((kind == 1 || kind == 2) && (!sfx || !sfw)) return (int)cudaErrorInvalidValue;
  if (act && (N % 32 || (ldc & 7))) return (int)cudaErrorInvalidValue;
  const int k_tiles = (K + kmma * 4 - 1) / (kmma * 4);
  const int tiles = N / 128;
  if (ks == 0) {
    ks = 1;
    while (ks < 8 && tiles * ks * 2 <= 2 * sm_count() && ks * 2 <= k_tiles) ks *= 2;
  }
  if (ks > k_tiles) ks = k_tiles;
  MoeGemmParams p;
  p.N = N; p.K = K; p.C = reinterpret_cast<__nv_bfloat16*>(C); p.ldc = ldc;
  p.row_scale = row_scale; p.alpha = alpha;
  p.sfw = reinterpret_cast<const uint8_t*>(sfw); p.sfx = reinterpret_cast<const uint8_t*>(sfx);
  p.sf_col_tiles = kind == 1 ? (K + 63) / 64 : kind == 2 ? (K + 127) / 128 : 0;
  p.tile_expert = nullptr; p.tile_rows = nullptr; p.rows = M; p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.ks = ks; p.act = act; p.ft_per = 1;
  p.status = status_word();
  CUtensorMap tmW, tmX;
  cudaError_t e;
  const uint64_t x_rows = (uint64_t)M;
  if (kind == 0) {
    e = encode_tmap(&tmW, W, 2, K, N, ldw, 64, 128, 3);
    if (e != cudaSuccess) return (int)e;
    e = encode_tmap(&tmX, X, 2, K, x_rows, ldx, 64, 32, 3);
  } else {
    const uint64_t kbytes = kind == 1 ? K / 2 : K;
    e = encode_tmap(&tmW, W, 1, kbytes, N, ldw, 128, 128, 3);
    if (e != cudaSuccess) return (int)e;
    e = encode_tmap(&tmX, X, 1, kbytes, x_rows, ldx, 128, 32, 3);
  }
  if (e != cudaSuccess) return (int)e;
  switch (kind) {
    case 0: return (int)launch_moe_gemm<0>(tmW, tmX, p, 1, stream);
    case 1: return (int)launch_moe_gemm<1>(tmW, tmX, p, 1, stream);
    default: return (int)launch_moe_gemm<2>(tmW, tmX, p, 1, stream);
  }
}
