// Paged GQA attention over FP8 (e4m3) KV on tcgen05: prefill chunks, decode and speculative-verify rows
// in one kernel.
//
// A work item is (sequence, kv head, block of <=128 query rows, kv split).  Query rows pack the GQA group
// into the MMA M dimension: row r = (token q0 + r / group, head kv_head * group + r % group), so every K/V
// byte fetched from HBM is used by the whole group.  Q is quantised to e4m3 per row in the kernel.
//   S = Q K^T   : A = Q [128 x D] (smem), B = K tile [128 tokens x D] (smem, straight from the page pool)
//   O_t = P V   : A = P [128 x 128 tokens] e4m3 (smem, written by the softmax warps), B = V^T tile [D x 128]
// Both accumulators live in TMEM (S and O_t double-buffered).  Pages are stored in the pool already in
// the canonical no-swizzle K-major core-matrix layout, so one 1-D bulk copy per page and operand feeds the
// tensor core with no register pass.  The online-softmax state (max, sum, output row) stays in registers:
// one thread per query row.
//
// Roles, head_dim 128 (192 threads): warp 0 loads pages (block-table walk + bulk copies), warp 1 issues MMAs, warps 2-5
// run softmax / accumulation on TMEM lane quadrant (warp & 3).
// head_dim 256 (384 threads = three warpgroups): an output row has 256 fp32 accumulators, too many for one thread, so
// warps 0-3 run softmax and accumulate output columns 0-127, warps 4-7 accumulate columns 128-255 (they get each tile's
// rescale factor and the final row sum through shared memory), warp 8 loads, warp 9 issues MMAs.  The register file is
// re-divided between the warpgroups with setmaxnreg (240 / 200 / 64 per thread).  The 256-column output accumulator is
// single-buffered in TMEM (S stays double-buffered): 2 x 128 + 256 = 512 columns.
//
// Reference counterparts: kernels/src/cuda/mha_nvfp4.cu mha_decode_kernel :259 + mha_combine_kernel :572
// (mma.sync, register dequant), mha_verify.cu :50, mha_prefill.cu prefill_kernel :118 (FA2 style, D=256 only).
#include "blaze/host.h"
#include "blaze/sm100.cuh"
#include "blaze/attn.cuh"
#include <type_traits>

namespace blz {

template <int D>
struct AttnCfg {
  static constexpr int TILE = 128;                 // tokens per KV tile
  static constexpr int PAGE_BYTES = 16 * D;        // one operand (K or V^T) of one page and head
  static constexpr int TILE_BYTES = 8 * PAGE_BYTES;
  static constexpr int STAGES = D == 128 ? 4 : 2;
  static constexpr int Q_BYTES = 128 * D;
  static constexpr int P_BYTES = 128 * 128;
  static constexpr bool WIDE = D > 128;            // two accumulator warpgroups, one output buffer in TMEM
  static constexpr int THREADS = WIDE ? 384 : 192;
  static constexpr int OBUF = WIDE ? 1 : 2;
  static constexpr int XCH_BYTES = WIDE ? (4 * 128 + 2 * 128 * 2) * 4 : 0;   // rescale factors [4][128], (max, sum) [2][128][2]
  static constexpr int SMEM = Q_BYTES + STAGES * 2 * TILE_BYTES + 2 * P_BYTES + XCH_BYTES + 1024 + 512;
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
};

template <int N> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

template <int D>
__global__ void __launch_bounds__(AttnCfg<D>::THREADS, 1) attn_tc_kernel(AttnParams p) {
  using Cfg = AttnCfg<D>;
  constexpr int ST = Cfg::STAGES;
  constexpr bool WIDE = Cfg::WIDE;
  constexpr int OBUF = Cfg::OBUF;
  constexpr int ACC = WIDE ? 128 : D;              // output columns accumulated by one thread
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::Q_BYTES;
  uint8_t* sV = sK + ST * Cfg::TILE_BYTES;
  uint8_t* sP = sV + ST * Cfg::TILE_BYTES;
  float* s_alpha = reinterpret_cast<float*>(sP + 2 * Cfg::P_BYTES);     // WIDE: [4][128] rescale factor of (tile & 3, row)
  float* s_fin = s_alpha + 4 * 128;                                     // WIDE: [2][128][2] (max, sum) of (item & 1, row)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * Cfg::P_BYTES + Cfg::XCH_BYTES);
  uint64_t* k_full = bars;                 // [ST]
  uint64_t* v_full = k_full + ST;          // [ST]
  uint64_t* kv_empty = v_full + ST;        // [ST]
  uint64_t* s_full = kv_empty + ST;        // [2]
  uint64_t* s_empty = s_full + 2;          // [2]
  uint64_t* p_full = s_empty + 2;          // [2]
  uint64_t* o_full = p_full + 2;           // [2]
  uint64_t* o_empty = o_full + 2;          // [2]
  uint64_t* q_full = o_empty + 2;          // [1]
  uint64_t* q_empty = q_full + 1;          // [1]
  uint64_t* fin_full = q_empty + 1;        // [2] WIDE: the softmax warps have published (max, sum) of an item
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(fin_full + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // role of this warp
  const bool is_loader = warp == (WIDE ? 8 : 0), is_mma = warp == (WIDE ? 9 : 1);
  const bool is_softmax = WIDE ? warp < 4 : (warp >= 2 && warp < 6);
  if (threadIdx.x == 0) {
    for (int i = 0; i < ST; ++i) { mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4); mbar_init(&p_full[i], 4);
      mbar_init(&o_full[i], 1); mbar_init(&o_empty[i], WIDE ? 8 : 4);
      mbar_init(&fin_full[i], 4);
    }
    mbar_init(q_full, 4); mbar_init(q_empty, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (is_mma) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // output accumulator buffer, its barrier index and barrier parity for global tile number gj
  auto o_buf = [&](int gj) -> int { return OBUF == 2 ? (gj & 1) : 0; };
  auto o_par = [&](int gj) -> uint32_t { return (uint32_t)(OBUF == 2 ? ((gj >> 1) & 1) : (gj & 1)); };

  const int group = p.Hq / p.Hkv;
  const int total = p.num_items * p.Hkv * p.splits;

  // One role's whole pass over this CTA's work items.  Every role walks the same item list with its own copy of the
  // counters; the loop lives inside the role (not the roles inside one loop) so that each role's code follows its own
  // setmaxnreg and is compiled against that register budget.
  constexpr int R_LOAD = 0, R_MMA = 1, R_SOFTMAX = 2, R_UPPER = 3;
  auto run = [&](auto role_tag) {
  constexpr int ROLE = decltype(role_tag)::value;
  int g = 0;      // tiles processed by this CTA so far (drives stage / phase bookkeeping in every role)
  int item_it = 0;
  for (int w = blockIdx.x; w < total; w += gridDim.x) {
    // ---- decode the work item (identical in every role)
    const int split = w % p.splits;
    const int kh = (w / p.splits) % p.Hkv;
    const int it = w / (p.splits * p.Hkv);
    const int b = p.item_seq ? p.item_seq[it] : it;
    const int q0 = p.item_q0 ? p.item_q0[it] : 0;
    const int r0 = p.q_start[b], qlen = p.q_start[b + 1] - r0;
    const int ctx = p.ctx_len[b];
    int ntok = qlen - q0;
    if (ntok > p.tokens_per_block) ntok = p.tokens_per_block;
    if (ntok <= 0) continue;
    const int nrows = ntok * group;
    // keys visible to the last row of the block
    const int kv_end = ctx - qlen + q0 + ntok;
    const int tiles_all = (kv_end + 127) >> 7;
    const int per = (tiles_all + p.splits - 1) / p.splits;
    const int t0 = split * per;
    const int t1 = min(tiles_all, t0 + per);
    const int n = max(t1 - t0, 0);
    const int slot = p.slots[b];

    if constexpr (ROLE == R_LOAD) {
      // -------------------------------------------------------------- page loader
      const int* bt = p.block_table + (size_t)slot * p.bt_stride;
      const int npages = (kv_end + 15) >> 4;
      for (int i = 0; i < n; ++i) {
        const int gi = g + i, s = gi % ST;
        if (!mbar_wait(&kv_empty[s], ((gi / ST) & 1) ^ 1, abort_flag, p.status)) break;
        if (lane == 0) {
          mbar_expect_tx(&k_full[s], Cfg::TILE_BYTES);
          mbar_expect_tx(&v_full[s], Cfg::TILE_BYTES);
        }
        __syncwarp();
        if (lane < 16) {
          const int pg = lane & 7;
          const int pidx = (t0 + i) * 8 + pg;
          const int page = pidx < npages ? bt[pidx] : 0;          // page 0 is the all-zero scratch page
          const uint8_t* src = p.pool + (size_t)page * p.page_stride + (size_t)kh * p.head_stride;
          if (lane < 8) bulk_load(sK + s * Cfg::TILE_BYTES + pg * Cfg::PAGE_BYTES, src, Cfg::PAGE_BYTES, &k_full[s]);
          else bulk_load(sV + s * Cfg::TILE_BYTES + pg * Cfg::PAGE_BYTES, src + Cfg::PAGE_BYTES, Cfg::PAGE_BYTES, &v_full[s]);
        }
        __syncwarp();
      }
    } else if constexpr (ROLE == R_MMA) {
      // -------------------------------------------------------------- MMA issuer
      if (lane == 0 && n > 0) {
        bool ok = mbar_wait(q_full, item_it & 1, abort_flag, p.status);
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ);
        auto issue_pv = [&](int gj) -> bool {
          const int s = gj % ST, pb = gj & 1;
          if (!mbar_wait(&v_full[s], (gj / ST) & 1, abort_flag, p.status)) return false;
          if (!mbar_wait(&p_full[pb], (gj >> 1) & 1, abort_flag, p.status)) return false;
          const int ob = o_buf(gj);
          if (!mbar_wait(&o_empty[ob], o_par(gj) ^ 1, abort_flag, p.status)) return false;
          tc_fence_after();
          const uint32_t pa = smem_u32(sP + pb * Cfg::P_BYTES), va = smem_u32(sV + s * Cfg::TILE_BYTES);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mma_f8(tmem + 256 + ob * 128, make_smem_desc(pa + ks * 256, 128, 1024, kSwzNone),
                   make_smem_desc(va + ks * 2 * Cfg::PAGE_BYTES, Cfg::PAGE_BYTES, 128, kSwzNone),
                   make_idesc(0, 0, 128, D), ks > 0);
          mma_commit(&o_full[ob]);
          mma_commit(&kv_empty[s]);
          return true;
        };
        for (int i = 0; i < n && ok; ++i) {
          const int gi = g + i, s = gi % ST, sb = gi & 1;
          if (!mbar_wait(&k_full[s], (gi / ST) & 1, abort_flag, p.status)) { ok = false; break; }
          if (!mbar_wait(&s_empty[sb], ((gi >> 1) & 1) ^ 1, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t ka = smem_u32(sK + s * Cfg::TILE_BYTES);
#pragma unroll
          for (int ks = 0; ks < D / 32; ++ks)
            mma_f8(tmem + sb * 128, make_smem_desc(q_addr + ks * 256, 128, 8 * D, kSwzNone),
                   make_smem_desc(ka + ks * 256, 128, 8 * D, kSwzNone), make_idesc(0, 0, 128, 128), ks > 0);
          mma_commit(&s_full[sb]);
          if (i > 0) ok = issue_pv(gi - 1);
        }
        if (ok) ok = issue_pv(g + n - 1);
        if (ok) mma_commit(q_empty);
      }
    } else if constexpr (ROLE == R_UPPER) {
      // -------------------------------------------------------------- output columns 128..255 (head_dim 256 only)
      const int qd = warp & 3;
      const int r = qd * 32 + lane;
      const bool live = r < nrows;
      const int tq = q0 + r / group;
      const int hq = kh * group + r % group;
      float acc[ACC];
#pragma unroll
      for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
      bool ok = true;
      for (int i = 0; i < n && ok; ++i) {
        const int gj = g + i;
        ok = __all_sync(0xffffffffu, mbar_wait(&o_full[0], o_par(gj), abort_flag, p.status));
        if (!ok) break;
        tc_fence_after();
        const float alpha = s_alpha[(gj & 3) * 128 + r];     // written before the row's probabilities were handed over
#pragma unroll
        for (int cch = 0; cch < ACC / 32; ++cch) {
          uint32_t v[32];
          tmem_ld32(tmem + 256 + 128 + cch * 32 + ((uint32_t)(qd * 32) << 16), v);
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 32; ++k) acc[cch * 32 + k] = acc[cch * 32 + k] * alpha + __uint_as_float(v[k]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_empty[0]);
      }
      if (n > 0 && ok) ok = mbar_wait(&fin_full[item_it & 1], (uint32_t)((item_it >> 1) & 1), abort_flag, p.status);
      if (ok && live && n > 0) {
        const float m_fin = s_fin[((item_it & 1) * 128 + r) * 2], l_fin = s_fin[((item_it & 1) * 128 + r) * 2 + 1];
        if (p.splits == 1) {
          const float inv = l_fin > 0.f ? p.v_scale / l_fin : 0.f;
          __nv_bfloat16* orow = p.out + ((size_t)(r0 + tq) * p.Hq + hq) * D + 128;
#pragma unroll
          for (int j = 0; j < ACC; j += 8) {
            uint4 u = make_uint4(pack_bf16x2(acc[j] * inv, acc[j + 1] * inv), pack_bf16x2(acc[j + 2] * inv, acc[j + 3] * inv),
                                 pack_bf16x2(acc[j + 4] * inv, acc[j + 5] * inv), pack_bf16x2(acc[j + 6] * inv, acc[j + 7] * inv));
            *reinterpret_cast<uint4*>(orow + j) = u;
          }
        } else {
          float* po = p.part_o + ((size_t)w * 128 + r) * D + 128;
#pragma unroll
          for (int j = 0; j < ACC; j += 4) *reinterpret_cast<float4*>(po + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
          (void)m_fin;
        }
      }
    } else {
      // -------------------------------------------------------------- softmax + accumulate (one row per thread)
      const int qd = warp & 3;
      const int r = qd * 32 + lane;                       // row of the 128-row block
      const bool live = r < nrows;
      const int tq = q0 + r / group;                      // token within the sequence's rows
      const int hq = kh * group + r % group;
      const int pos_q = ctx - qlen + tq;                  // last visible key position
      float acc[ACC];
#pragma unroll
      for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
      float m_run = -INFINITY, l_run = 0.f, qscale = 1.f;
      if (n > 0) {
        // ---- Q row → e4m3 in the K-major core-matrix layout
        if (!mbar_wait(q_empty, (item_it & 1) ^ 1, abort_flag, p.status)) break;
        const __nv_bfloat16* qrow = p.q + ((size_t)(r0 + tq) * p.Hq + hq) * D;
        float amax = 0.f;
        if (live) {
#pragma unroll
          for (int j = 0; j < D; j += 8) {
            uint4 u = *reinterpret_cast<const uint4*>(qrow + j);
            const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
            for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(bf2f(e[k])));
          }
        }
        qscale = fmaxf(amax, 1e-12f) / 448.f;
        const float qinv = 1.f / qscale;
        uint8_t* qdst = sQ + (r >> 3) * (8 * D) + (r & 7) * 16;
#pragma unroll
        for (int j = 0; j < D; j += 16) {
          uint4 o = make_uint4(0, 0, 0, 0);
          if (live) {
            uint4 u0 = *reinterpret_cast<const uint4*>(qrow + j), u1 = *reinterpret_cast<const uint4*>(qrow + j + 8);
            const __nv_bfloat16* e0 = reinterpret_cast<const __nv_bfloat16*>(&u0);
            const __nv_bfloat16* e1 = reinterpret_cast<const __nv_bfloat16*>(&u1);
            o.x = pack_e4m3x4(bf2f(e0[0]) * qinv, bf2f(e0[1]) * qinv, bf2f(e0[2]) * qinv, bf2f(e0[3]) * qinv);
            o.y = pack_e4m3x4(bf2f(e0[4]) * qinv, bf2f(e0[5]) * qinv, bf2f(e0[6]) * qinv, bf2f(e0[7]) * qinv);
            o.z = pack_e4m3x4(bf2f(e1[0]) * qinv, bf2f(e1[1]) * qinv, bf2f(e1[2]) * qinv, bf2f(e1[3]) * qinv);
            o.w = pack_e4m3x4(bf2f(e1[4]) * qinv, bf2f(e1[5]) * qinv, bf2f(e1[6]) * qinv, bf2f(e1[7]) * qinv);
          }
          *reinterpret_cast<uint4*>(qdst + (j >> 4) * 128) = o;
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(q_full);
      }
      const float c = p.scale_log2 * qscale;              // raw MMA value → log2-domain logit
      float alpha_prev = 1.f;
      bool ok = true;
      auto accumulate = [&](int gj, float alpha) -> bool {
        const int ob = o_buf(gj);
        // tcgen05.ld is warp-collective: the wait's outcome is made warp-uniform before any lane loads
        if (!__all_sync(0xffffffffu, mbar_wait(&o_full[ob], o_par(gj), abort_flag, p.status))) return false;
        tc_fence_after();
#pragma unroll
        for (int cch = 0; cch < ACC / 32; ++cch) {
          uint32_t v[32];
          tmem_ld32(tmem + 256 + ob * 128 + cch * 32 + ((uint32_t)(qd * 32) << 16), v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[cch * 32 + i] = acc[cch * 32 + i] * alpha + __uint_as_float(v[i]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_empty[ob]);
        return true;
      };
      for (int i = 0; i < n && ok; ++i) {
        const int gi = g + i, sb = gi & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&s_full[sb], (gi >> 1) & 1, abort_flag, p.status))) { ok = false; break; }
        tc_fence_after();
        const int k0 = (t0 + i) * 128;
        const int lim = min(pos_q, kv_end - 1) - k0;        // columns <= lim are visible to this row
        const uint32_t s_addr = tmem + sb * 128 + ((uint32_t)(qd * 32) << 16);
        float m_tile = -INFINITY;
        const bool full = lim >= 127;                       // no masking needed for this row in this tile
#pragma unroll 1
        for (int cch = 0; cch < 4; ++cch) {
          uint32_t v[32];
          tmem_ld32(s_addr + cch * 32, v);
          tmem_ld_wait();
          if (full) {
#pragma unroll
            for (int j = 0; j < 32; ++j) m_tile = fmaxf(m_tile, __uint_as_float(v[j]));
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (cch * 32 + j <= lim) m_tile = fmaxf(m_tile, __uint_as_float(v[j]));
          }
        }
        const float m_new = fmaxf(m_run, m_tile * c);
        const float alpha = (m_run == -INFINITY) ? 0.f : ex2(m_run - m_new);
        const float off = (m_new == -INFINITY) ? 0.f : m_new - 8.f;     // P is scaled by 2^8 to use the e4m3 range
        float rs = 0.f;
        uint8_t* pdst = sP + sb * Cfg::P_BYTES + (r >> 3) * 1024 + (r & 7) * 16;
#pragma unroll 1
        for (int cch = 0; cch < 4; ++cch) {
          uint32_t v[32];
          tmem_ld32(s_addr + cch * 32, v);
          tmem_ld_wait();
          float e[32];
          if (full) {
#pragma unroll
            for (int j = 0; j < 32; ++j) { e[j] = ex2(fmaf(__uint_as_float(v[j]), c, -off)); rs += e[j]; }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float x = (cch * 32 + j <= lim) ? ex2(fmaf(__uint_as_float(v[j]), c, -off)) : 0.f;
              e[j] = x;
              rs += x;
            }
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint4 o;
            o.x = pack_e4m3x4(e[h * 16 + 0], e[h * 16 + 1], e[h * 16 + 2], e[h * 16 + 3]);
            o.y = pack_e4m3x4(e[h * 16 + 4], e[h * 16 + 5], e[h * 16 + 6], e[h * 16 + 7]);
            o.z = pack_e4m3x4(e[h * 16 + 8], e[h * 16 + 9], e[h * 16 + 10], e[h * 16 + 11]);
            o.w = pack_e4m3x4(e[h * 16 + 12], e[h * 16 + 13], e[h * 16 + 14], e[h * 16 + 15]);
            *reinterpret_cast<uint4*>(pdst + (cch * 2 + h) * 128) = o;
          }
        }
        l_run = l_run * alpha + rs;
        m_run = m_new;
        if constexpr (WIDE) s_alpha[(gi & 3) * 128 + r] = alpha;   // for the warps that accumulate the other output half
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) { mbar_arrive(&s_empty[sb]); mbar_arrive(&p_full[sb]); }
        if (i > 0) ok = accumulate(gi - 1, alpha_prev);
        alpha_prev = alpha;
      }
      if (ok && n > 0) ok = accumulate(g + n - 1, alpha_prev);
      if constexpr (WIDE) {
        if (n > 0) {           // (also after a failed wait: the other warpgroup's bounded wait then ends at once, via the abort flag)
          s_fin[((item_it & 1) * 128 + r) * 2] = m_run;
          s_fin[((item_it & 1) * 128 + r) * 2 + 1] = l_run;
          __syncwarp();
          if (lane == 0) mbar_arrive(&fin_full[item_it & 1]);
        }
      }
      // ---- write out
      if (ok && live) {
        if (p.splits == 1) {
          const float inv = l_run > 0.f ? p.v_scale / l_run : 0.f;
          __nv_bfloat16* orow = p.out + ((size_t)(r0 + tq) * p.Hq + hq) * D;
#pragma unroll
          for (int j = 0; j < ACC; j += 8) {
            uint4 u = make_uint4(pack_bf16x2(acc[j] * inv, acc[j + 1] * inv), pack_bf16x2(acc[j + 2] * inv, acc[j + 3] * inv),
                                 pack_bf16x2(acc[j + 4] * inv, acc[j + 5] * inv), pack_bf16x2(acc[j + 6] * inv, acc[j + 7] * inv));
            *reinterpret_cast<uint4*>(orow + j) = u;
          }
        } else {
          float* po = p.part_o + ((size_t)w * 128 + r) * D;
#pragma unroll
          for (int j = 0; j < ACC; j += 4) *reinterpret_cast<float4*>(po + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
          p.part_ml[((size_t)w * 128 + r) * 2] = m_run;
          p.part_ml[((size_t)w * 128 + r) * 2 + 1] = l_run;
        }
      }
    }
    g += n;
    if (n > 0) ++item_it;
    if (*abort_flag) break;
  }
  };   // run

  if constexpr (WIDE) {
    // 384 threads start with 168 registers each; the loader / MMA warpgroup hands most of its share to the other two
    if (warp >= 8) {
      reg_dec<64>();
      if (is_loader) run(std::integral_constant<int, R_LOAD>{});
      else if (is_mma) run(std::integral_constant<int, R_MMA>{});
    } else if (warp >= 4) {
      reg_inc<200>();
      run(std::integral_constant<int, R_UPPER>{});
    } else {
      reg_inc<240>();
      run(std::integral_constant<int, R_SOFTMAX>{});
    }
  } else {
    if (is_loader) run(std::integral_constant<int, R_LOAD>{});
    else if (is_mma) run(std::integral_constant<int, R_MMA>{});
    else if (is_softmax) run(std::integral_constant<int, R_SOFTMAX>{});
  }
  tc_fence_before();
  __syncthreads();
  if (is_mma) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// Merge kv-split partials: out = sum_s 2^(m_s - m) acc_s / sum_s 2^(m_s - m) l_s
template <int D>
__global__ void attn_combine_kernel(AttnParams p) {
  const int it = blockIdx.x / p.Hkv, kh = blockIdx.x % p.Hkv;
  const int b = p.item_seq ? p.item_seq[it] : it;
  const int q0 = p.item_q0 ? p.item_q0[it] : 0;
  const int r0 = p.q_start[b], qlen = p.q_start[b + 1] - r0;
  const int group = p.Hq / p.Hkv;
  int ntok = min(qlen - q0, p.tokens_per_block);
  if (ntok <= 0) return;
  const int nrows = ntok * group;
  for (int r = threadIdx.x / 32; r < nrows; r += blockDim.x / 32) {
    const int lane = threadIdx.x & 31;
    float m = -INFINITY;
    for (int s = 0; s < p.splits; ++s) {
      const size_t w = ((size_t)it * p.Hkv + kh) * p.splits + s;
      if (p.part_ml[(w * 128 + r) * 2 + 1] > 0.f) m = fmaxf(m, p.part_ml[(w * 128 + r) * 2]);
    }
    float l = 0.f;
    float o[D / 32];
#pragma unroll
    for (int j = 0; j < D / 32; ++j) o[j] = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const size_t w = ((size_t)it * p.Hkv + kh) * p.splits + s;
      const float ls = p.part_ml[(w * 128 + r) * 2 + 1];
      if (!(ls > 0.f)) continue;
      const float f = exp2f(p.part_ml[(w * 128 + r) * 2] - m);
      l += ls * f;
#pragma unroll
      for (int j = 0; j < D / 32; ++j) o[j] += p.part_o[(w * 128 + r) * D + j * 32 + lane] * f;
    }
    const float inv = l > 0.f ? p.v_scale / l : 0.f;
    const int tq = q0 + r / group, hq = kh * group + r % group;
    __nv_bfloat16* orow = p.out + ((size_t)(r0 + tq) * p.Hq + hq) * D;
#pragma unroll
    for (int j = 0; j < D / 32; ++j) orow[j * 32 + lane] = __float2bfloat16(o[j] * inv);
  }
}

}  // namespace blz

// Scratch needed for `splits` > 1: part_o = items*Hkv*splits*128*D floats, part_ml = items*Hkv*splits*128*2 floats.
BLZ_API int blz_attn_tc(const void* q, void* out, const void* pool, const int* block_table, const int* slots,
                        const int* q_start, const int* ctx_len, const int* item_seq, const int* item_q0, int num_items,
                        int Hq, int Hkv, int D, int bt_stride, long long page_stride, long long head_stride, float scale, float k_scale,
                        float v_scale, int splits, float* part_o, float* part_ml, int max_ctas, cudaStream_t stream) {
  using namespace blz;
  if (num_items <= 0) return 0;
  if ((D != 128 && D != 256) || Hq % Hkv || 128 % (Hq / Hkv) || splits < 1 || (splits > 1 && (!part_o || !part_ml)))
    return (int)cudaErrorInvalidValue;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.pool = (const uint8_t*)pool;
  p.page_stride = page_stride > 0 ? page_stride : (long long)Hkv * 2 * 16 * D;
  p.head_stride = head_stride > 0 ? head_stride : (long long)2 * 16 * D;
  p.block_table = block_table; p.slots = slots; p.q_start = q_start; p.ctx_len = ctx_len;
  p.item_seq = item_seq; p.item_q0 = item_q0; p.part_o = part_o; p.part_ml = part_ml;
  p.num_items = num_items; p.Hq = Hq; p.Hkv = Hkv; p.bt_stride = bt_stride; p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f * k_scale; p.v_scale = v_scale;
  p.tokens_per_block = 128 / (Hq / Hkv);
  p.status = status_word();
  p.min_rows = 0; p.max_rows = 1 << 30; p.row_blocks = 1; p.prof = nullptr;
  static PerDeviceOnce configured, configured_wide;
  {
    cudaError_t e = D == 128 ? configured.smem_limit(attn_tc_kernel<128>, AttnCfg<128>::SMEM)
                             : configured_wide.smem_limit(attn_tc_kernel<256>, AttnCfg<256>::SMEM);
    if (e != cudaSuccess) return (int)e;
  }
  const int total = num_items * Hkv * splits;
  int grid = total < sm_count() ? total : sm_count();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (D == 128) attn_tc_kernel<128><<<grid, AttnCfg<128>::THREADS, AttnCfg<128>::SMEM, stream>>>(p);
  else attn_tc_kernel<256><<<grid, AttnCfg<256>::THREADS, AttnCfg<256>::SMEM, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (splits > 1) {
    if (D == 128) attn_combine_kernel<128><<<num_items * Hkv, 256, 0, stream>>>(p);
    else attn_combine_kernel<256><<<num_items * Hkv, 256, 0, stream>>>(p);
    e = cudaGetLastError();
  }
  return (int)e;
}
