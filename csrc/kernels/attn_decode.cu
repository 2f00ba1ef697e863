// Paged GQA decode / speculative-verify attention over FP8 KV on tcgen05, tokens on the TMEM lanes.
//
// With one (or a few) query tokens per sequence only `q_len * group` rows are live; putting them on the MMA's
// M dimension would leave 124 of 128 softmax rows idle and makes the exponential unit the bottleneck.  Here the
// problem is transposed:
//     S^T = K Q^T   : A = K tile [128 tokens x D] (smem, straight from the page pool), B = Q [NMAX rows x D]
//     O^T_t = V^T P^T : A = V^T tile [D x 128 tokens] (smem, from the pool), B = P [NMAX rows x 128 tokens]
// so every softmax thread owns one key position and touches only NMAX (16 or 32) columns of tensor memory, and
// every accumulate thread owns one output dimension with NMAX running sums in registers.  Row maxima are
// exchanged across the four softmax warps once per tile; row sums are reduced once per work item.
//
// Work item = (sequence, kv head, block of NMAX rows, kv split); persistent CTAs; 320 threads (page loader warp,
// MMA warp, two sets of four softmax warps that take alternate tiles and are merged per work item like kv splits);
// 2 CTAs per SM when at most 8 rows are live.  Every wait is a bounded mbarrier wait.
//
// Reference counterparts: kernels/src/cuda/mha_nvfp4.cu mha_decode_kernel :259 and mha_combine_kernel :572,
// kernels/src/cuda/mha_verify.cu verify_kernel :50.
#include "blaze/attn.cuh"
#include "blaze/host.h"

namespace blz {

// NMAX = MMA N (rows per work item, 16 or 32); RMAX = rows kept in registers by the softmax threads (>= live rows).
template <int NMAX, int RMAX>
struct DecCfg {
  static constexpr int D = 128;
  static constexpr int PAGE_BYTES = 16 * D;
  static constexpr int TILE_BYTES = 8 * PAGE_BYTES;
  static constexpr int THREADS = 320;                // loader warp, MMA warp, two sets of four softmax warps
  static constexpr int CTAS_PER_SM = RMAX <= 8 ? 2 : 1;
  static constexpr int STAGES = CTAS_PER_SM == 2 ? 3 : 5;   // depth of the K ring and of the V ring (released separately)
  static constexpr int Q_BYTES = NMAX * D;
  static constexpr int P_BYTES = NMAX * 128;
  static constexpr int NB = 3;                       // S^T / P / O^T buffers (softmax runs up to two tiles ahead of the fold)
  static constexpr int TMEM_COLS = NMAX <= 16 ? 128 : 256;
  static constexpr int SMEM = 2 * Q_BYTES + STAGES * 2 * TILE_BYTES + NB * P_BYTES + 128 + 640;
};

__device__ __forceinline__ bool timed_wait(long long& acc, bool on, uint64_t* bar, uint32_t par, volatile int* abort_flag,
                                           int* status) {
  if (!on) return mbar_wait(bar, par, abort_flag, status);
  const long long t = clock64();
  const bool r = mbar_wait(bar, par, abort_flag, status);
  acc += clock64() - t;
  return r;
}

template <int N>
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, uint32_t (&r)[N]) {
  if constexpr (N == 16) tmem_ld16(taddr, r); else tmem_ld32(taddr, r);
}

template <int NMAX, int RMAX>
__global__ void __launch_bounds__(320, (DecCfg<NMAX, RMAX>::CTAS_PER_SM)) attn_decode_kernel(AttnParams p) {
  pdl_trigger();
  using Cfg = DecCfg<NMAX, RMAX>;
  constexpr int ST = Cfg::STAGES, D = Cfg::D, NB = Cfg::NB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint8_t* sK = smem;
  uint8_t* sV = sK + ST * Cfg::TILE_BYTES;
  uint8_t* sQ = sV + ST * Cfg::TILE_BYTES;
  uint8_t* sP = sQ + 2 * Cfg::Q_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + NB * Cfg::P_BYTES);
  uint64_t* k_full = bars;                 // [ST]
  uint64_t* v_full = k_full + ST;          // [ST]
  uint64_t* k_empty = v_full + ST;         // [ST] released when S^T = K Q^T of the tile has completed
  uint64_t* v_empty = k_empty + ST;        // [ST] released when O^T = V^T P^T of the tile has completed
  uint64_t* s_full = v_empty + ST;         // [NB]
  uint64_t* s_empty = s_full + NB;         // [NB]
  uint64_t* p_full = s_empty + NB;         // [NB]
  uint64_t* o_full = p_full + NB;          // [NB]
  uint64_t* o_empty = o_full + NB;         // [NB]
  uint64_t* wm_bar = o_empty + NB;         // [NB] row-max exchange among the softmax warps
  uint64_t* q_full = wm_bar + NB;          // [2]
  uint64_t* q_empty = q_full + 2;          // [2]
  uint64_t* fin_bar = q_empty + 2;         // [1] both sets have published their partial results
  uint64_t* acc_free = fin_bar + 1;        // [1] set 0 has consumed set 1's partial results
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ float s_c[2][NMAX];
  __shared__ int s_pos[2][NMAX];
  __shared__ uint32_t s_mask[2][NMAX];   // tree verify: which of the sequence's new tokens a row may see (bit per token)
  __shared__ float s_wmax[Cfg::NB][4][NMAX];
  __shared__ float s_l[2][4][RMAX];                  // [set][warp][row] partial row sums
  __shared__ float s_m[RMAX];                        // set 1's row maxima
  __shared__ float s_acc[RMAX][128];                 // set 1's output sums

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < ST; ++i) { mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_empty[i], 1); }
    for (int i = 0; i < NB; ++i) {
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4); mbar_init(&p_full[i], 4);
      mbar_init(&o_full[i], 1); mbar_init(&o_empty[i], 4); mbar_init(&wm_bar[i], 4);
    }
    for (int i = 0; i < 2; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
    mbar_init(fin_bar, 8); mbar_init(acc_free, 4);
    *abort_flag = 0;
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < 2 * Cfg::Q_BYTES / 16; i += blockDim.x) reinterpret_cast<uint4*>(sQ)[i] = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();          // the queries and this step's K/V rows come from the kernel before this one

  const int group = p.Hq / p.Hkv;
  const int total = p.num_items * p.Hkv * p.row_blocks * p.splits;
  int g = 0, item_it = 0;
  long long pc[13];
#pragma unroll
  for (int i = 0; i < 13; ++i) pc[i] = 0;
  const long long t_start = clock64();
#define TW(cat, bar, par) timed_wait(pc[cat], p.prof != nullptr, bar, par, abort_flag, p.status)

  for (int w = blockIdx.x; w < total; w += gridDim.x) {
    const int split = w % p.splits;
    const int rb = (w / p.splits) % p.row_blocks;
    const int kh = (w / (p.splits * p.row_blocks)) % p.Hkv;
    const int b = w / (p.splits * p.row_blocks * p.Hkv);
    const int r0 = p.q_start[b], qlen = p.q_start[b + 1] - r0;
    const int rows_total = qlen * group;
    if (rows_total < p.min_rows || rows_total > p.max_rows) continue;
    const int row0 = rb * NMAX;
    const int nrows = min(NMAX, rows_total - row0);
    if (nrows <= 0) continue;
    const int ctx = p.ctx_len[b];
    const int kv_end = ctx - qlen + (row0 + nrows - 1) / group + 1;       // keys visible to the block's last row
    const int tiles_all = (kv_end + 127) >> 7;
    const int per = (tiles_all + p.splits - 1) / p.splits;
    const int t0 = split * per;
    const int n = max(min(tiles_all, t0 + per) - t0, 0);
    const int slot = p.slots[b];

    if (warp == 0) {
      // -------------------------------------------------------------- page loader
      const int* bt = p.block_table + (size_t)slot * p.bt_stride;
      const int npages = (kv_end + 15) >> 4;
      if (n > 0) {
        // ---- this item's Q rows → e4m3 in the K-major core-matrix layout, plus the per-row constants
        // Items of at most 8 live rows (plain decode at group 4 or 8, two verify rows) are prepared by the K half of the
        // warp alone, 4 or 2 lanes per row: the two halves then never meet, and this half moves on to the next item's Q
        // rows and K tiles while the V half is still waiting for ring slots of this one.  (The rows beyond RMAX of both Q
        // buffers are zeroed once, before the loop.)
        constexpr bool HALF = RMAX <= 8;
        constexpr int LPR = RMAX <= 4 ? 4 : RMAX <= 8 ? 2 : (32 / NMAX == 0 ? 1 : 32 / NMAX);   // lanes per row
        constexpr int DPL = D / LPR;                               // dims per lane
        constexpr uint32_t QMASK = HALF ? 0x0000FFFFu : 0xFFFFFFFFu;
        if (!HALF || lane < 16) {
        const int qb = item_it & 1;
        const int rr = lane / LPR, part = lane % LPR;
        const int R = row0 + rr;
        const bool live = rr < nrows;
        const int tq = R / group, hq = kh * group + R % group;
        uint4 raw[DPL / 8];
        float amax = 0.f;
        if (live) {
          const __nv_bfloat16* qrow = p.q + ((size_t)(r0 + tq) * p.Hq + hq) * D + part * DPL;
#pragma unroll
          for (int j = 0; j < DPL / 8; ++j) raw[j] = *reinterpret_cast<const uint4*>(qrow + j * 8);
#pragma unroll
          for (int j = 0; j < DPL / 8; ++j) {
            const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw[j]);
#pragma unroll
            for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(bf2f(e[k])));
          }
        }
        if (LPR >= 2) amax = fmaxf(amax, __shfl_xor_sync(QMASK, amax, 1));
        if (LPR == 4) amax = fmaxf(amax, __shfl_xor_sync(QMASK, amax, 2));
        const float qscale = fmaxf(amax, 1e-12f) / 448.f;
        const float qinv = 1.f / qscale;
        if (!TW(10, &q_empty[qb], ((item_it >> 1) & 1) ^ 1)) break;
        uint8_t* qdst = sQ + qb * Cfg::Q_BYTES + (rr >> 3) * (8 * D) + (rr & 7) * 16 + (part * DPL / 16) * 128;
#pragma unroll
        for (int j = 0; j < DPL / 16; ++j) {
          uint4 o = make_uint4(0, 0, 0, 0);
          if (live) {
            const __nv_bfloat16* e0 = reinterpret_cast<const __nv_bfloat16*>(&raw[2 * j]);
            const __nv_bfloat16* e1 = reinterpret_cast<const __nv_bfloat16*>(&raw[2 * j + 1]);
            o.x = pack_e4m3x4(bf2f(e0[0]) * qinv, bf2f(e0[1]) * qinv, bf2f(e0[2]) * qinv, bf2f(e0[3]) * qinv);
            o.y = pack_e4m3x4(bf2f(e0[4]) * qinv, bf2f(e0[5]) * qinv, bf2f(e0[6]) * qinv, bf2f(e0[7]) * qinv);
            o.z = pack_e4m3x4(bf2f(e1[0]) * qinv, bf2f(e1[1]) * qinv, bf2f(e1[2]) * qinv, bf2f(e1[3]) * qinv);
            o.w = pack_e4m3x4(bf2f(e1[4]) * qinv, bf2f(e1[5]) * qinv, bf2f(e1[6]) * qinv, bf2f(e1[7]) * qinv);
          }
          *reinterpret_cast<uint4*>(qdst + j * 128) = o;
        }
        if (part == 0) {
          s_c[qb][rr] = p.scale_log2 * qscale;
          s_pos[qb][rr] = live ? ctx - qlen + tq : -1;
          if constexpr (RMAX > 4) s_mask[qb][rr] = (live && p.tree_mask) ? (uint32_t)p.tree_mask[r0 + tq] : 0xFFFFFFFFu;
        }
        fence_async_smem();
        __syncwarp(QMASK);
        if (lane == 0) mbar_arrive(&q_full[qb]);
        }
      }
      // The lower half of the warp streams K tiles, the upper half V^T tiles: the two rings are released at different
      // times (K after S^T = K Q^T, V two tiles later after O^T = V^T P^T), so each half waits only for its own ring
      // (and, for plain decode items, runs through the work items at its own pace).
      // (the page number of the next tile is fetched before the wait for its ring slot, off the critical path)
      if (lane < 16) {
        int page = 0;
        if (lane < 8 && n > 0) { const int pidx = t0 * 8 + lane; page = pidx < npages ? bt[pidx] : 0; }
        for (int i = 0; i < n; ++i) {
          const int gi = g + i, s = gi % ST;
          int next = 0;
          if (lane < 8 && i + 1 < n) { const int pidx = (t0 + i + 1) * 8 + lane; next = pidx < npages ? bt[pidx] : 0; }
          if (!TW(0, &k_empty[s], ((gi / ST) & 1) ^ 1)) break;
          if (lane == 0) mbar_expect_tx(&k_full[s], Cfg::TILE_BYTES);
          __syncwarp(0x0000FFFFu);
          if (lane < 8) {
            const uint8_t* src = p.pool + (size_t)page * p.page_stride + (size_t)kh * p.head_stride;   // page 0 = zero scratch page
            bulk_load(sK + s * Cfg::TILE_BYTES + lane * Cfg::PAGE_BYTES, src, Cfg::PAGE_BYTES, &k_full[s]);
          }
          __syncwarp(0x0000FFFFu);
          page = next;
        }
      } else {
        int page = 0;
        if (lane < 24 && n > 0) { const int pidx = t0 * 8 + lane - 16; page = pidx < npages ? bt[pidx] : 0; }
        for (int i = 0; i < n; ++i) {
          const int gi = g + i, s = gi % ST;
          int next = 0;
          if (lane < 24 && i + 1 < n) { const int pidx = (t0 + i + 1) * 8 + lane - 16; next = pidx < npages ? bt[pidx] : 0; }
          if (!mbar_wait(&v_empty[s], ((gi / ST) & 1) ^ 1, abort_flag, p.status)) break;
          if (lane == 16) mbar_expect_tx(&v_full[s], Cfg::TILE_BYTES);
          __syncwarp(0xFFFF0000u);
          if (lane < 24) {
            const int pg = lane - 16;
            const uint8_t* src = p.pool + (size_t)page * p.page_stride + (size_t)kh * p.head_stride + Cfg::PAGE_BYTES;
            bulk_load(sV + s * Cfg::TILE_BYTES + pg * Cfg::PAGE_BYTES, src, Cfg::PAGE_BYTES, &v_full[s]);
          }
          __syncwarp(0xFFFF0000u);
          page = next;
        }
      }
      if constexpr (RMAX > 8) __syncwarp();
    } else if (warp == 1) {
      // -------------------------------------------------------------- MMA issuer
      if (lane == 0 && n > 0) {
        bool ok = TW(6, &q_full[item_it & 1], (item_it >> 1) & 1);
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + (item_it & 1) * Cfg::Q_BYTES);
        auto issue_pv = [&](int gj) -> bool {
          const int s = gj % ST, pb = gj % NB;
          if (!TW(3, &v_full[s], (gj / ST) & 1)) return false;
          if (!TW(4, &p_full[pb], (gj / NB) & 1)) return false;
          if (!TW(5, &o_empty[pb], ((gj / NB) & 1) ^ 1)) return false;
          tc_fence_after();
          const uint32_t pa = smem_u32(sP + pb * Cfg::P_BYTES), va = smem_u32(sV + s * Cfg::TILE_BYTES);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mma_f8(tmem + NB * NMAX + pb * NMAX,
                   make_smem_desc(va + ks * 2 * Cfg::PAGE_BYTES, Cfg::PAGE_BYTES, 128, kSwzNone),
                   make_smem_desc(pa + ks * 256, 128, 1024, kSwzNone), make_idesc(0, 0, 128, NMAX), ks > 0);
          mma_commit(&o_full[pb]);
          mma_commit(&v_empty[s]);
          return true;
        };
        for (int i = 0; i < n && ok; ++i) {
          const int gi = g + i, s = gi % ST, sb = gi % NB;
          if (!TW(1, &k_full[s], (gi / ST) & 1)) { ok = false; break; }
          if (!TW(2, &s_empty[sb], ((gi / NB) & 1) ^ 1)) { ok = false; break; }
          tc_fence_after();
          const uint32_t ka = smem_u32(sK + s * Cfg::TILE_BYTES);
#pragma unroll
          for (int ks = 0; ks < D / 32; ++ks)
            mma_f8(tmem + sb * NMAX, make_smem_desc(ka + ks * 256, 128, 8 * D, kSwzNone),
                   make_smem_desc(q_addr + ks * 256, 128, 8 * D, kSwzNone), make_idesc(0, 0, 128, NMAX), ks > 0);
          mma_commit(&s_full[sb]);
          mma_commit(&k_empty[s]);
          if (i > 1) ok = issue_pv(gi - 2);
        }
        if (ok && n > 1) ok = issue_pv(g + n - 2);
        if (ok) ok = issue_pv(g + n - 1);
        if (ok) mma_commit(&q_empty[item_it & 1]);
      }
    } else {
      // -------------------------------------------------------------- softmax (thread = key position) and
      //                                                                accumulate (thread = output dimension)
      const int qd = warp & 3;
      const int set = (warp - 2) >> 2;                     // two softmax warp sets take alternate tiles
      const int t = qd * 32 + lane;
      const uint32_t lane_bits = (uint32_t)(qd * 32) << 16;
      float m_run[RMAX], l_part[RMAX], acc[RMAX];
#pragma unroll
      for (int i = 0; i < RMAX; ++i) { m_run[i] = -INFINITY; l_part[i] = 0.f; acc[i] = 0.f; }
      bool ok = true;
      const int qb = item_it & 1;
      if (n > 0 && !TW(6, &q_full[qb], (item_it >> 1) & 1)) break;     // per-row constants are published with Q
      // add tile gj's O^T (relative to this set's row maxima at tile gj) to the running sums
      auto fold = [&](int gj) -> bool {
        const int ob = gj % NB;
        if (!TW(9, &o_full[ob], (gj / NB) & 1)) return false;
        tc_fence_after();
        // only the first RMAX columns hold live rows: a plain decode step reads 4 of the 16
        constexpr int LDN = RMAX <= 4 ? 4 : NMAX;
        uint32_t o[LDN];
        if constexpr (RMAX <= 4) tmem_ld4(tmem + NB * NMAX + ob * NMAX + lane_bits, o);
        else tmem_ldn<NMAX>(tmem + NB * NMAX + ob * NMAX + lane_bits, o);
        tmem_ld_wait();
#pragma unroll
        for (int r = 0; r < RMAX; ++r) {
          if (r >= nrows) break;
          acc[r] += __uint_as_float(o[r]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_empty[ob]);
        return true;
      };
      int last = -1;
      for (int i = set; i < n && ok; i += 2) {
        const int gi = g + i, sb = gi % NB;
        if (!TW(7, &s_full[sb], (gi / NB) & 1)) { ok = false; break; }
        tc_fence_after();
        constexpr int LDN = RMAX <= 4 ? 4 : NMAX;
        uint32_t v[LDN];
        if constexpr (RMAX <= 4) tmem_ld4(tmem + sb * NMAX + lane_bits, v);
        else tmem_ldn<NMAX>(tmem + sb * NMAX + lane_bits, v);
        tmem_ld_wait();
        const int key = (t0 + i) * 128 + t;
        float x[RMAX];
#pragma unroll
        for (int r = 0; r < RMAX; ++r) {
          if (r >= nrows) break;
          bool vis = key <= s_pos[qb][r];
          if constexpr (RMAX > 4) {
            // tree verify: among the sequence's own new tokens (keys from ctx - qlen on) a row sees its ancestors only
            // (a word covers the first 32 new tokens; plain causal rows - no tree mask - may be longer and are not masked)
            const int j = key - (ctx - qlen);
            if (vis && p.tree_mask != nullptr && j >= 0 && j < 32) vis = (s_mask[qb][r] >> j) & 1u;
          }
          x[r] = vis ? __uint_as_float(v[r]) * s_c[qb][r] : -INFINITY;
          const float wm = warp_max_redux(x[r]);
          if (lane == 0) s_wmax[sb][qd][r] = wm;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&wm_bar[sb]);
        // fold this set's previous tile while the other warps of the set catch up
        if (last >= 0 && !fold(last)) { ok = false; break; }
        if (!TW(8, &wm_bar[sb], (gi / NB) & 1)) { ok = false; break; }
        uint8_t* pdst = sP + sb * Cfg::P_BYTES + (t >> 4) * 128 + (t & 15);
#pragma unroll
        for (int r = 0; r < RMAX; ++r) {
          if (r >= nrows) break;
          const float mt = fmaxf(fmaxf(s_wmax[sb][0][r], s_wmax[sb][1][r]), fmaxf(s_wmax[sb][2][r], s_wmax[sb][3][r]));
          const float m_new = fmaxf(m_run[r], mt);
          // A row may see no key of this tile (an earlier chain row when the new tokens straddle a tile boundary); if that
          // is the first tile this warp set handles for the row, both maxima are -inf and their difference is not a number.
          const bool none = m_new == -INFINITY;
          const float alpha = none ? 1.f : ex2(m_run[r] - m_new);     // ex2(-inf) = 0 on the first tile with visible keys
          const float pr = none ? 0.f : ex2(x[r] - m_new + 8.f);      // masked keys: ex2(-inf) = 0; P scaled by 2^8
          l_part[r] = l_part[r] * alpha + pr;
          acc[r] *= alpha;
          m_run[r] = m_new;
          pdst[(r >> 3) * 1024 + (r & 7) * 16] = (uint8_t)__nv_cvt_float_to_fp8(pr, __NV_SATFINITE, __NV_E4M3);
        }
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) { mbar_arrive(&s_empty[sb]); mbar_arrive(&p_full[sb]); }
        last = gi;
      }
      if (ok && last >= 0) ok = fold(last);
      if (!ok) break;
      // ---- merge the two sets and the four warps of each: row sums, maxima, output sums
      if (n > 0) {
        // the exchange buffers are single: set 1 writes them only after set 0 has read the previous item's
        if (set == 1 && !TW(11, acc_free, (item_it & 1) ^ 1)) break;
#pragma unroll
        for (int r = 0; r < RMAX; ++r) {
          if (r >= nrows) break;
          const float ws = warp_sum(l_part[r]);
          if (lane == 0) s_l[set][qd][r] = ws;
          if (set == 1) s_acc[r][t] = acc[r];
          if (set == 1 && t == 0) s_m[r] = m_run[r];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(fin_bar);
        if (!TW(11, fin_bar, item_it & 1)) break;
        if (set == 0) {
#pragma unroll
          for (int r = 0; r < RMAX; ++r) {
            if (r >= nrows) break;
            const float mb = s_m[r];
            const float m = fmaxf(m_run[r], mb);
            // (a set that saw no visible key of the row has maximum -inf and contributes nothing)
            const float fa = m_run[r] == -INFINITY ? 0.f : ex2(m_run[r] - m), fb = mb == -INFINITY ? 0.f : ex2(mb - m);
            const float l = (s_l[0][0][r] + s_l[0][1][r] + s_l[0][2][r] + s_l[0][3][r]) * fa +
                            (s_l[1][0][r] + s_l[1][1][r] + s_l[1][2][r] + s_l[1][3][r]) * fb;
            const float o = acc[r] * fa + s_acc[r][t] * fb;
            const int R = row0 + r;
            const int tq = R / group, hq = kh * group + R % group;
            if (p.splits == 1) {
              p.out[((size_t)(r0 + tq) * p.Hq + hq) * D + t] = __float2bfloat16(l > 0.f ? o * p.v_scale / l : 0.f);
            } else {
              p.part_o[((size_t)w * NMAX + r) * D + t] = o;
              if (t == 0) {
                p.part_ml[((size_t)w * NMAX + r) * 2] = m;
                p.part_ml[((size_t)w * NMAX + r) * 2 + 1] = l;
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_free);
        }
      } else if (set == 0 && p.splits > 1) {
        for (int r = 0; r < nrows; ++r) {
          p.part_o[((size_t)w * NMAX + r) * D + t] = 0.f;
          if (t == 0) {
            p.part_ml[((size_t)w * NMAX + r) * 2] = -INFINITY;
            p.part_ml[((size_t)w * NMAX + r) * 2 + 1] = 0.f;
          }
        }
      }
    }
    g += n;
    if (n > 0) ++item_it;
    if (*abort_flag) break;
  }
#undef TW
  if (p.prof && blockIdx.x < 8 && lane == 0 && warp < 3) {
    pc[12] = clock64() - t_start;
    for (int i = 0; i < 13; ++i) p.prof[((size_t)blockIdx.x * 3 + warp) * 16 + i] = pc[i];
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

// Merge kv-split partials of the decode kernel.  One CTA per (sequence, kv head, row block); thread = dimension.
template <int NMAX>
__global__ void attn_decode_combine_kernel(AttnParams p) {
  pdl_trigger();
  pdl_wait();
  constexpr int D = 128;
  const int rb = blockIdx.x % p.row_blocks;
  const int kh = (blockIdx.x / p.row_blocks) % p.Hkv;
  const int b = blockIdx.x / (p.row_blocks * p.Hkv);
  const int group = p.Hq / p.Hkv;
  const int r0 = p.q_start[b], qlen = p.q_start[b + 1] - r0;
  const int rows_total = qlen * group;
  if (rows_total < p.min_rows || rows_total > p.max_rows) return;
  const int row0 = rb * NMAX;
  const int nrows = min(NMAX, rows_total - row0);
  const int t = threadIdx.x;
  for (int r = 0; r < nrows; ++r) {
    float m = -INFINITY;
    for (int s = 0; s < p.splits; ++s) {
      const size_t w = (size_t)blockIdx.x * p.splits + s;
      if (p.part_ml[(w * NMAX + r) * 2 + 1] > 0.f) m = fmaxf(m, p.part_ml[(w * NMAX + r) * 2]);
    }
    float l = 0.f, o = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const size_t w = (size_t)blockIdx.x * p.splits + s;
      const float ls = p.part_ml[(w * NMAX + r) * 2 + 1];
      if (!(ls > 0.f)) continue;
      const float f = exp2f(p.part_ml[(w * NMAX + r) * 2] - m);
      l += ls * f;
      o += p.part_o[(w * NMAX + r) * D + t] * f;
    }
    const int R = row0 + r;
    const int tq = R / group, hq = kh * group + R % group;
    p.out[((size_t)(r0 + tq) * p.Hq + hq) * D + t] = __float2bfloat16(l > 0.f ? o * p.v_scale / l : 0.f);
  }
}

template <int NMAX, int RMAX>
static cudaError_t launch_decode(const AttnParams& p, int max_ctas, cudaStream_t stream) {
  using Cfg = DecCfg<NMAX, RMAX>;
  static PerDeviceOnce configured;
  {
    cudaError_t e = configured.smem_limit(attn_decode_kernel<NMAX, RMAX>, Cfg::SMEM);
    if (e != cudaSuccess) return e;
  }
  const int total = p.num_items * p.Hkv * p.row_blocks * p.splits;
  const int cap = Cfg::CTAS_PER_SM * sm_count();
  int grid = total < cap ? total : cap;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  cudaError_t e = launch_pdl(attn_decode_kernel<NMAX, RMAX>, dim3(grid), dim3(Cfg::THREADS), Cfg::SMEM, stream, p);
  if (e != cudaSuccess || p.splits == 1) return e;
  return launch_pdl(attn_decode_combine_kernel<NMAX>, dim3(p.num_items * p.Hkv * p.row_blocks), dim3(128), 0, stream, p);
}

}  // namespace blz

// Decode / verify attention for every sequence with min_rows <= q_len * (Hq / Hkv) <= max_rows.
// nmax: 16 or 32 rows per work item; row_blocks = ceil(max rows of any processed sequence / nmax).
// Scratch for splits > 1: part_o = B*Hkv*row_blocks*splits*nmax*128 floats, part_ml = ...*nmax*2 floats.
// tree_mask (optional, [T] int32, indexed like q's rows): bit j of row i's word = row i may attend to the j-th new token
// of its sequence (itself and its ancestors in a draft tree; at most 32 new tokens per sequence).  Null = causal rows.
// Plain decode work items (at most 4 live rows per KV head) ignore it: a single new token sees only itself.
BLZ_API int blz_attn_decode_tree(const void* q, void* out, const void* pool, const int* block_table, const int* slots,
                            const int* q_start, const int* ctx_len, int num_seqs, int Hq, int Hkv, int D, int bt_stride, long long page_stride, long long head_stride,
                            float scale, float k_scale, float v_scale, int nmax, int row_blocks, int min_rows,
                            int max_rows, int splits, float* part_o, float* part_ml, int max_ctas, long long* prof,
                            const int* tree_mask, cudaStream_t stream) {
  using namespace blz;
  if (num_seqs <= 0) return 0;
  if (D != 128 || Hq % Hkv || (nmax != 16 && nmax != 32) || row_blocks < 1 || splits < 1 ||
      (splits > 1 && (!part_o || !part_ml)))
    return (int)cudaErrorInvalidValue;
  // every processed sequence has at most max_rows rows per kv head: the row blocks must cover them, or rows would be skipped
  if (max_rows < (1 << 29) && (long long)row_blocks * nmax < max_rows) return (int)cudaErrorInvalidValue;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.pool = (const uint8_t*)pool;
  p.page_stride = page_stride > 0 ? page_stride : (long long)Hkv * 2 * 16 * D;
  p.head_stride = head_stride > 0 ? head_stride : (long long)2 * 16 * D;
  p.block_table = block_table; p.slots = slots; p.q_start = q_start; p.ctx_len = ctx_len;
  p.item_seq = nullptr; p.item_q0 = nullptr; p.part_o = part_o; p.part_ml = part_ml;
  p.num_items = num_seqs; p.Hq = Hq; p.Hkv = Hkv; p.bt_stride = bt_stride; p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f * k_scale; p.v_scale = v_scale;
  p.tokens_per_block = 0; p.min_rows = min_rows; p.max_rows = max_rows; p.row_blocks = row_blocks;
  p.status = status_word();
  p.prof = prof;
  p.tree_mask = tree_mask;
  if (nmax == 32) return (int)launch_decode<32, 32>(p, max_ctas, stream);
  const int live = max_rows < 16 ? max_rows : 16;     // most live rows of any work item
  if (live <= 4 && !tree_mask) return (int)launch_decode<16, 4>(p, max_ctas, stream);
  if (live <= 8) return (int)launch_decode<16, 8>(p, max_ctas, stream);
  return (int)launch_decode<16, 16>(p, max_ctas, stream);
}

BLZ_API int blz_attn_decode(const void* q, void* out, const void* pool, const int* block_table, const int* slots,
                            const int* q_start, const int* ctx_len, int num_seqs, int Hq, int Hkv, int D, int bt_stride, long long page_stride, long long head_stride,
                            float scale, float k_scale, float v_scale, int nmax, int row_blocks, int min_rows,
                            int max_rows, int splits, float* part_o, float* part_ml, int max_ctas, long long* prof,
                            cudaStream_t stream) {
  return blz_attn_decode_tree(q, out, pool, block_table, slots, q_start, ctx_len, num_seqs, Hq, Hkv, D, bt_stride, page_stride,
                              head_stride, scale, k_scale, v_scale, nmax, row_blocks, min_rows, max_rows, splits, part_o, part_ml,
                              max_ctas, prof, nullptr, stream);
}

// ------------------------------------------------------------------------------------------------------------------
// Allocation-free variant (see blaze/attn_noalloc.h): the split-KV partials live in a library-owned device array.
#include <cstdio>
#include <mutex>

#include "blaze/attn_noalloc.h"

namespace {
// partial outputs [work][16][128] floats followed by (max, sum) pairs [work][16][2] floats
static __device__ __align__(256) unsigned char g_noalloc_scratch[BLZ_ATTN_NOALLOC_SCRATCH_BYTES];
static __device__ int g_noalloc_status;

struct NoAllocDev {
  bool ready = false;
  float* scratch = nullptr;     // device address of g_noalloc_scratch on that device
  int* status = nullptr;
};
NoAllocDev g_noalloc_dev[64];
std::mutex g_noalloc_mu;          // guards the first-call set-up of a device
thread_local char g_noalloc_err[256] = "";
}  // namespace

// Reads and clears the status word that blz_attn_decode_noalloc's kernels report into on the current device (0 = fine,
// 1 = a bounded wait inside the kernel ran out and the call's output is not valid).  Synchronises the device; returns -1
// when no call has been made on this device yet or the copy fails.  Allocates nothing.
extern "C" __attribute__((visibility("default"))) int blz_attn_decode_noalloc_status(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_dev[dev].ready) return -1;
  }
  int h = 0;
  if (cudaMemcpyFromSymbol(&h, g_noalloc_status, sizeof(int)) != cudaSuccess) return -1;
  if (h != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_noalloc_status, &zero, sizeof(int)) != cudaSuccess) return -1;
  }
  return h;
}

extern "C" __attribute__((visibility("default"))) const char* blz_attn_decode_noalloc_error(void) { return g_noalloc_err; }

extern "C" __attribute__((visibility("default"))) long long blz_attn_decode_noalloc_bytes(int num_seqs, int Hkv, int row_blocks,
                                                                                          int splits) {
  const long long work = (long long)num_seqs * Hkv * row_blocks * splits;
  return work * 16 * (128 + 2) * (long long)sizeof(float);
}

extern "C" __attribute__((visibility("default"))) int blz_attn_decode_noalloc(
    const void* q, void* out, const void* pool, const int* block_table, const int* slots, const int* q_start, const int* ctx_len,
    int num_seqs, int Hq, int Hkv, int D, int bt_stride, long long page_stride, long long head_stride, float scale, float k_scale, float v_scale, int row_blocks, int min_rows,
    int max_rows, int splits, int max_ctas, cudaStream_t stream) {
  using namespace blz;
  g_noalloc_err[0] = 0;
  if (num_seqs <= 0) return 0;
  if (D != 128 || Hkv <= 0 || Hq % Hkv || row_blocks < 1 || splits < 1) {
    snprintf(g_noalloc_err, sizeof(g_noalloc_err), "unsupported shape: head_dim %d, heads %d/%d, row_blocks %d, splits %d", D, Hq,
             Hkv, row_blocks, splits);
    return (int)cudaErrorInvalidValue;
  }
  if (max_rows < (1 << 29) && (long long)row_blocks * 16 < max_rows) {
    snprintf(g_noalloc_err, sizeof(g_noalloc_err), "row_blocks %d x 16 rows do not cover max_rows %d: rows would be skipped",
             row_blocks, max_rows);
    return (int)cudaErrorInvalidValue;
  }
  const long long need = blz_attn_decode_noalloc_bytes(num_seqs, Hkv, row_blocks, splits);
  if (splits > 1 && need > (long long)BLZ_ATTN_NOALLOC_SCRATCH_BYTES) {
    snprintf(g_noalloc_err, sizeof(g_noalloc_err),
             "split-KV scratch of %lld bytes (%d seqs x %d kv heads x %d row blocks x %d splits) exceeds the built-in %u bytes; "
             "use fewer splits or blz_attn_decode with caller-owned scratch",
             need, num_seqs, Hkv, row_blocks, splits, (unsigned)BLZ_ATTN_NOALLOC_SCRATCH_BYTES);
    return (int)cudaErrorInvalidValue;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    snprintf(g_noalloc_err, sizeof(g_noalloc_err), "cudaGetDevice failed (%d)", (int)e);
    return (int)(e != cudaSuccess ? e : cudaErrorInvalidDevice);
  }
  NoAllocDev& d = g_noalloc_dev[dev];
  std::unique_lock<std::mutex> setup_lock(g_noalloc_mu);
  if (!d.ready) {
    // first call on this device, with this device current: resolve the device addresses of the library-owned arrays.
    // In host code the array names are host-side stand-ins, never device pointers.
    void* p_scratch = nullptr;
    void* p_status = nullptr;
    e = cudaGetSymbolAddress(&p_scratch, g_noalloc_scratch);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&p_status, g_noalloc_status);
    if (e != cudaSuccess) {
      snprintf(g_noalloc_err, sizeof(g_noalloc_err), "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return (int)e;
    }
    d.scratch = reinterpret_cast<float*>(p_scratch);
    d.status = reinterpret_cast<int*>(p_status);
    d.ready = true;
  }
  setup_lock.unlock();
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.pool = (const uint8_t*)pool;
  p.page_stride = page_stride > 0 ? page_stride : (long long)Hkv * 2 * 16 * D;
  p.head_stride = head_stride > 0 ? head_stride : (long long)2 * 16 * D;
  p.block_table = block_table; p.slots = slots; p.q_start = q_start; p.ctx_len = ctx_len;
  p.item_seq = nullptr; p.item_q0 = nullptr;
  const long long work = (long long)num_seqs * Hkv * row_blocks * splits;
  p.part_o = d.scratch;
  p.part_ml = d.scratch + work * 16 * 128;
  p.num_items = num_seqs; p.Hq = Hq; p.Hkv = Hkv; p.bt_stride = bt_stride; p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f * k_scale; p.v_scale = v_scale;
  p.tokens_per_block = 0; p.min_rows = min_rows; p.max_rows = max_rows; p.row_blocks = row_blocks;
  p.status = d.status;
  p.prof = nullptr;
  const int live = max_rows < 16 ? max_rows : 16;
  if (live <= 4) e = launch_decode<16, 4>(p, max_ctas, stream);
  else if (live <= 8) e = launch_decode<16, 8>(p, max_ctas, stream);
  else e = launch_decode<16, 16>(p, max_ctas, stream);
  if (e != cudaSuccess) snprintf(g_noalloc_err, sizeof(g_noalloc_err), "launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}
