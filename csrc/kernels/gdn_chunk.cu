// Gated DeltaNet over long token runs (prefill), 128 tokens per chunk, on tcgen05.
//
// The recurrence   S <- S e^{g_t};  d_t = beta_t (v_t - S^T k_t);  S <- S + k_t d_t^T;  o_t = S^T q_t      (S is dk x dv)
// is sequential in t.  Over a chunk of C tokens it can be rewritten with matrix products (the WY / UT form):
//     G_i = g_1 + .. + g_i (inside the chunk),  gamma_i = e^{G_i}
//     A   = strictly lower part of  diag(beta) (K K^T) .* e^{G_i - G_j}                      C x C
//     T   = (I + A)^{-1}                                                                      C x C, unit lower triangular
//     U   = T diag(beta) V,      W = T diag(beta gamma) K                                     C x dv, C x dk
//     D   = U - W S0                                  (the d_t of all tokens of the chunk)    C x dv
//     O   = diag(gamma) Q S0 + lower( (Q K^T) .* e^{G_i - G_j} ) D                            C x dv
//     S1  = e^{G_C} S0 + (diag(e^{G_C - G_j}) K)^T D                                          dk x dv
// Every product runs on the tensor core (bf16 operands from shared memory, fp32 accumulators in tensor memory); the
// triangular inverse is computed in fp32 on the CUDA cores (16 x 16 diagonal blocks by substitution, then three levels
// of block merges  T21 = -T22 A21 T11); the state is kept in fp32 in tensor memory for the whole run, transposed
// (S^T: dv on the lanes) so that its bf16 copy for the next chunk's products is a plain row write.  All decay factors
// that appear are e^{G_i - G_j} with j <= i, so they are at most 1.
//
// One CTA per (sequence, value head), 128 threads: thread r owns token r of the chunk and lane r of tensor memory;
// thread 0 also issues the MMAs.  The phases of a chunk run one after the other (no overlap inside a CTA; different
// heads and sequences overlap across SMs).  Every wait is a bounded mbarrier wait.
//
// Operand layout in shared memory: 128 x 128 bf16, K-major, no swizzle, 8 x 8 core matrices of 128 bytes:
//     offset(row, k) = (row / 8) * 2048 + (k / 8) * 128 + (row % 8) * 16 + (k % 8) * 2.
//
// Reference: the reference has the token-by-token kernel only (kernels/src/cuda/gdn_recurrent.cu:27-92) and applies it
// to prompts as well (crates/blaze/src/model.rs:3364-3511); this file is that kernel's chunked counterpart, tested
// against it.
#include "blaze/host.h"
#include "blaze/sm100.cuh"

namespace blz {

struct GdnChunkParams {
  const __nv_bfloat16* conv;   // [T, C] conv + SiLU output, channels [q (Hk*128) | k (Hk*128) | v (Hv*128)]
  const __nv_bfloat16* a_in;   // [T, ld_ab]
  const __nv_bfloat16* b_in;
  long long ld_ab;
  const float* A_log;          // [Hv]
  const float* dt_bias;        // [Hv]
  float* rec_state;            // [slots, Hv, 128 (dk), 128 (dv)] fp32
  __nv_bfloat16* out;          // [T, Hv, 128]
  const int* slots;
  const int* q_start;
  const int* ctx_len;
  const int* no_store;         // optional [B]
  int Hk, Hv;
  int min_rows;                // sequences with fewer new tokens are left to the token-by-token kernel
  int* status;
  long long* prof;             // optional [CTAs][16]: cycles thread 0 spent in each phase, summed over the chunks (diagnostics)
};

constexpr int GC = 128;                       // chunk length = head dims
constexpr int GBUF = GC * GC * 2;             // one bf16 operand buffer
constexpr int GDN_SMEM = 6 * GBUF + 1024 /*align*/ + 3 * GC * 4 + 64;

__device__ __forceinline__ uint32_t op_off(int row, int k) {      // byte offset of element (row, k) in an operand buffer
  return (uint32_t)((row >> 3) * 2048 + (k >> 3) * 128 + (row & 7) * 16 + (k & 7) * 2);
}
// fp32 scratch matrix [128][128] with the column index xor-ed so that a column walk hits different banks
__device__ __forceinline__ int f_idx(int row, int col) { return row * GC + (col ^ ((row & 7) << 2)); }

// Z[rows o_z.., cols c_z..] (S x S) = sign * X (S x S at rx, cx) * Y (S x S at ry, cy), all inside the scratch matrix.
// 128 threads cover 128 / (2 S) independent products at once (pair index p shifts every origin by p * 2 S on both axes).
// CLEAR_Y: afterwards the Y block is set to zero (it was scratch above the diagonal, which later steps read as part of T).
template <int S, bool CLEAR_Y>
__device__ __forceinline__ void tri_product(float* M, int tid, int zr, int zc, int xr, int xc, int yr, int yc, float sign) {
  constexpr int W = S / 2;
  const int pair = tid / (2 * S), i = (tid % (2 * S)) >> 1, c0 = (tid & 1) * W;
  const int o = pair * 2 * S;
  float acc[W];
#pragma unroll
  for (int j = 0; j < W; ++j) acc[j] = 0.f;
  for (int k = 0; k < S; ++k) {
    const float x = M[f_idx(o + xr + i, o + xc + k)];
    const int yrow = o + yr + k;
#pragma unroll
    for (int j = 0; j < W; j += 4) {
      // four consecutive columns stay contiguous under the xor (its low two bits are zero)
      const float4 y = *reinterpret_cast<const float4*>(&M[f_idx(yrow, o + yc + c0 + j)]);
      acc[j] = fmaf(x, y.x, acc[j]); acc[j + 1] = fmaf(x, y.y, acc[j + 1]);
      acc[j + 2] = fmaf(x, y.z, acc[j + 2]); acc[j + 3] = fmaf(x, y.w, acc[j + 3]);
    }
  }
  __syncthreads();        // every thread has read its inputs before any block is rewritten
#pragma unroll
  for (int j = 0; j < W; j += 4) {
    *reinterpret_cast<float4*>(&M[f_idx(o + zr + i, o + zc + c0 + j)]) =
        make_float4(sign * acc[j], sign * acc[j + 1], sign * acc[j + 2], sign * acc[j + 3]);
    if (CLEAR_Y) *reinterpret_cast<float4*>(&M[f_idx(o + yr + i, o + yc + c0 + j)]) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  __syncthreads();
}

__global__ void __launch_bounds__(128, 1) gdn_chunk_kernel(GdnChunkParams p) {
  const int b = blockIdx.x, hv = blockIdx.y;
  const int r0 = p.q_start[b], n = p.q_start[b + 1] - r0;
  if (n < p.min_rows || n <= 0) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int hk = hv / (p.Hv / p.Hk);
  const int Cch = 2 * p.Hk * GC + p.Hv * GC;
  const bool fresh = p.ctx_len[b] - n == 0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bK = smem;                 // K rows            -> later W rows          (with bT: the fp32 scratch matrix)
  uint8_t* bT = smem + GBUF;          // T (scaled) rows   -> later P rows
  uint8_t* bQ = smem + 2 * GBUF;      // Q rows (later scaled by gamma)
  uint8_t* bVT = smem + 3 * GBUF;     // V^T               -> later D^T
  uint8_t* bKT = smem + 4 * GBUF;     // K^T               -> later scaled by e^{G_C - G_j}
  uint8_t* bST = smem + 5 * GBUF;     // S^T rows (bf16 copy of the state)
  float* Mf = reinterpret_cast<float*>(smem);                 // [128][128] fp32 scratch over bK + bT
  float* s_G = reinterpret_cast<float*>(smem + 6 * GBUF);     // [128] cumulative log decay
  float* s_beta = s_G + GC;                                   // [128]
  float* s_w = s_beta + GC;                                   // [128] scan scratch / per-warp sums
  uint64_t* bar = reinterpret_cast<uint64_t*>(s_w + GC);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (tid == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  const uint32_t T_S = tmem + lane_base, T_1 = tmem + 128 + lane_base, T_2 = tmem + 256 + lane_base, T_3 = tmem + 384 + lane_base;
  uint32_t phase = 0;
  bool ok = true;
  long long t_ph[12];
#pragma unroll
  for (int i = 0; i < 12; ++i) t_ph[i] = 0;
  long long t_last = clock64();
  // phase timer (thread 0 only matters): adds the cycles since the last mark to slot i
  auto mark = [&](int i) {
    if (p.prof) {
      const long long t = clock64();
      t_ph[i] += t - t_last;
      t_last = t;
    }
  };

  // issue one product D[128 x 128] (+)= A[128 x 128] * B[128 x 128]^T (both K-major in shared memory)
  auto mma = [&](uint32_t d_col, const uint8_t* A, const uint8_t* B, bool accumulate) {
    const uint32_t a = smem_u32(A), bb = smem_u32(B);
#pragma unroll
    for (int ks = 0; ks < GC / 16; ++ks)
      mma_f16(tmem + d_col, make_smem_desc(a + ks * 256, 128, 2048, kSwzNone), make_smem_desc(bb + ks * 256, 128, 2048, kSwzNone),
              make_idesc(1, 1, 128, 128), (accumulate || ks > 0) ? 1u : 0u);
  };
  // all threads: make shared-memory writes visible to the tensor core, let thread 0 issue, wait for completion
  auto run = [&](auto&& issue) {
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      issue();
      mma_commit(bar);
    }
    ok = __syncthreads_and(mbar_wait(bar, phase, abort_flag, p.status)) != 0;
    phase ^= 1;
    tc_fence_after();
  };

  // ---- state: S^T into tensor memory (fp32) and into bST (bf16); lane = dv index
  {
    const float* st = p.rec_state + (((size_t)p.slots[b] * p.Hv + hv) * GC) * GC;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = fresh ? 0u : __float_as_uint(st[(size_t)(c * 32 + j) * GC + tid]);
      tmem_st32(T_S + c * 32, r);
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 u = make_uint4(pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])),
                             pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                             pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])),
                             pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
        *reinterpret_cast<uint4*>(bST + op_off(tid, c * 32 + j)) = u;
      }
    }
    tmem_st_wait();
  }
  const float Aexp = __expf(p.A_log[hv]);
  const float dtb = p.dt_bias[hv];

  mark(0);
  for (int c0 = 0; c0 < n && ok; c0 += GC) {
    const int L = min(GC, n - c0);
    const bool live = tid < L;
    const size_t row = (size_t)(r0 + c0 + tid);
    // ---- gates and the cumulative log decay (padding rows: no decay, beta = 0, zero q / k / v)
    float g = 0.f, beta = 0.f;
    if (live) {
      const float av = bf2f(p.a_in[row * p.ld_ab + hv]) + dtb;
      const float sp = av > 20.f ? av : log1pf(__expf(av));
      g = -Aexp * sp;
      beta = bf2f(__float2bfloat16(1.f / (1.f + __expf(-bf2f(p.b_in[row * p.ld_ab + hv])))));
    }
    float G = g;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, G, o);
      if ((tid & 31) >= o) G += t;
    }
    if ((tid & 31) == 31) s_w[warp] = G;
    __syncthreads();
    for (int w = 0; w < warp; ++w) G += s_w[w];
    s_G[tid] = G;
    s_beta[tid] = beta;
    __syncthreads();
    const float G_C = s_G[GC - 1];
    // ---- k: L2-normalised -> K rows and K^T; q: normalised and scaled -> Q rows; v -> V^T
    {
      const __nv_bfloat16* src = p.conv + row * Cch + (size_t)p.Hk * GC + (size_t)hk * GC;
      uint4 u[16];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        u[j] = live ? *reinterpret_cast<const uint4*>(src + j * 8) : make_uint4(0, 0, 0, 0);
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u[j]);
#pragma unroll
        for (int q = 0; q < 8; ++q) ss += bf2f(e[q]) * bf2f(e[q]);
      }
      const float kn = rsqrtf(ss + 1e-6f);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u[j]);
        __nv_bfloat16 o8[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          o8[q] = __float2bfloat16(bf2f(e[q]) * kn);
          *reinterpret_cast<__nv_bfloat16*>(bKT + op_off(j * 8 + q, tid)) = o8[q];
        }
        *reinterpret_cast<uint4*>(bK + op_off(tid, j * 8)) = *reinterpret_cast<const uint4*>(o8);
      }
    }
    {
      const __nv_bfloat16* src = p.conv + row * Cch + (size_t)hk * GC;
      uint4 u[16];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        u[j] = live ? *reinterpret_cast<const uint4*>(src + j * 8) : make_uint4(0, 0, 0, 0);
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u[j]);
#pragma unroll
        for (int q = 0; q < 8; ++q) ss += bf2f(e[q]) * bf2f(e[q]);
      }
      const float qn = rsqrtf(ss + 1e-6f) * rsqrtf((float)GC);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u[j]);
        __nv_bfloat16 o8[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) o8[q] = __float2bfloat16(bf2f(e[q]) * qn);
        *reinterpret_cast<uint4*>(bQ + op_off(tid, j * 8)) = *reinterpret_cast<const uint4*>(o8);
      }
    }
    {
      const __nv_bfloat16* src = p.conv + row * Cch + 2 * (size_t)p.Hk * GC + (size_t)hv * GC;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const uint4 u = live ? *reinterpret_cast<const uint4*>(src + j * 8) : make_uint4(0, 0, 0, 0);
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
        for (int q = 0; q < 8; ++q) *reinterpret_cast<__nv_bfloat16*>(bVT + op_off(j * 8 + q, tid)) = e[q];
      }
    }
    mark(1);
    // ---- D1 = K K^T, D2 = Q K^T
    run([&] { mma(128, bK, bK, false); mma(256, bQ, bK, false); });
    if (!ok) break;
    mark(2);
    // ---- A = strictly lower( beta_i D1_ij e^{G_i - G_j} ) into the fp32 scratch (over bK + bT: K rows are no longer needed)
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(T_1 + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int col = c * 32 + j;
        Mf[f_idx(tid, col)] = col < tid ? beta * __uint_as_float(r[j]) * __expf(G - s_G[col]) : 0.f;
      }
    }
    __syncthreads();
    mark(3);
    // ---- T = (I + A)^{-1} in place.  Diagonal 16 x 16 blocks by substitution: thread (block bb, column cc) solves one column.
    {
      const int bb = tid >> 4, cc = tid & 15, o = bb * 16;
      float x[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float acc = (i == cc) ? 1.f : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (j < i) acc -= Mf[f_idx(o + i, o + j)] * x[j];          // x[j] is zero above the diagonal (j < cc)
        x[i] = i >= cc ? acc : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 16; ++i) Mf[f_idx(o + i, o + cc)] = x[i];
      __syncthreads();
    }
    // merges: T21 = -T22 (A21 T11); the product A21 T11 is parked in the (otherwise unused) upper-right block
    tri_product<16, false>(Mf, tid, 0, 16, 16, 0, 0, 0, 1.f);
    tri_product<16, true>(Mf, tid, 16, 0, 16, 16, 0, 16, -1.f);
    tri_product<32, false>(Mf, tid, 0, 32, 32, 0, 0, 0, 1.f);
    tri_product<32, true>(Mf, tid, 32, 0, 32, 32, 0, 32, -1.f);
    tri_product<64, false>(Mf, tid, 0, 64, 64, 0, 0, 0, 1.f);
    tri_product<64, true>(Mf, tid, 64, 0, 64, 64, 0, 64, -1.f);
    mark(4);
    // ---- row tid of T into registers (columns above the diagonal are scratch: masked), then the scratch is free again
    float trow[GC];
#pragma unroll
    for (int j = 0; j < GC; ++j) trow[j] = j <= tid ? Mf[f_idx(tid, j)] : 0.f;
    __syncthreads();
    // ---- U = (T diag(beta)) V  -> T_1
    auto write_T = [&](bool with_gamma) {
#pragma unroll
      for (int j = 0; j < GC; j += 8) {
        float s[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) s[q] = trow[j + q] * s_beta[j + q] * (with_gamma ? __expf(s_G[j + q]) : 1.f);
        *reinterpret_cast<uint4*>(bT + op_off(tid, j)) =
            make_uint4(pack_bf16x2(s[0], s[1]), pack_bf16x2(s[2], s[3]), pack_bf16x2(s[4], s[5]), pack_bf16x2(s[6], s[7]));
      }
    };
    write_T(false);
    mark(5);
    run([&] { mma(128, bT, bVT, false); });
    if (!ok) break;
    // ---- W = (T diag(beta gamma)) K  -> T_3
    write_T(true);
    run([&] { mma(384, bT, bKT, false); });
    if (!ok) break;
    mark(6);
    // ---- W rows -> bK; P = lower( D2 .* e^{G_i - G_j} ) rows -> bT; Q rows scaled by gamma_i; K^T columns by e^{G_C - G_j}
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(T_3 + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        *reinterpret_cast<uint4*>(bK + op_off(tid, c * 32 + j)) =
            make_uint4(pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                       pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])), pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
      tmem_ld32(T_2 + c * 32, r);
      tmem_ld_wait();
      float pv[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int col = c * 32 + j;
        pv[j] = col <= tid ? __uint_as_float(r[j]) * __expf(G - s_G[col]) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        *reinterpret_cast<uint4*>(bT + op_off(tid, c * 32 + j)) =
            make_uint4(pack_bf16x2(pv[j], pv[j + 1]), pack_bf16x2(pv[j + 2], pv[j + 3]), pack_bf16x2(pv[j + 4], pv[j + 5]),
                       pack_bf16x2(pv[j + 6], pv[j + 7]));
    }
    {
      const float gam = __expf(G), kap = __expf(G_C - G);
#pragma unroll
      for (int j = 0; j < GC; j += 8) {
        uint4 u = *reinterpret_cast<uint4*>(bQ + op_off(tid, j));
        __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&u);
#pragma unroll
        for (int q = 0; q < 8; ++q) e[q] = __float2bfloat16(bf2f(e[q]) * gam);
        *reinterpret_cast<uint4*>(bQ + op_off(tid, j)) = u;
      }
#pragma unroll 4
      for (int d = 0; d < GC; ++d) {
        __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(bKT + op_off(d, tid));
        *e = __float2bfloat16(bf2f(*e) * kap);
      }
    }
    mark(7);
    // ---- D5 = W S0 -> T_3;  O = (gamma Q) S0 -> T_2
    run([&] { mma(384, bK, bST, false); mma(256, bQ, bST, false); });
    if (!ok) break;
    mark(8);
    // ---- D = U - D5 -> D^T (bf16) over V^T;  state in tensor memory scaled by e^{G_C}
    {
      const float dec = __expf(G_C);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t u[32], w[32];
        tmem_ld32(T_1 + c * 32, u);
        tmem_ld32(T_3 + c * 32, w);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j)
          *reinterpret_cast<__nv_bfloat16*>(bVT + op_off(c * 32 + j, tid)) = __float2bfloat16(__uint_as_float(u[j]) - __uint_as_float(w[j]));
        tmem_ld32(T_S + c * 32, u);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) u[j] = __float_as_uint(__uint_as_float(u[j]) * dec);
        tmem_st32(T_S + c * 32, u);
      }
      tmem_st_wait();
    }
    mark(9);
    // ---- O += P D;   S^T += D^T (K scaled)   (A = D^T [dv x tokens], B = scaled K^T [dk x tokens])
    run([&] { mma(256, bT, bVT, true); mma(0, bVT, bKT, true); });
    if (!ok) break;
    mark(10);
    // ---- outputs of the chunk; bf16 copy of the new state for the next chunk's products
    const bool last = c0 + GC >= n;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(T_2 + c * 32, r);
      tmem_ld_wait();
      if (live) {
        __nv_bfloat16* dst = p.out + (row * p.Hv + hv) * GC + c * 32;
#pragma unroll
        for (int j = 0; j < 32; j += 8)
          *reinterpret_cast<uint4*>(dst + j) =
              make_uint4(pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                         pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])), pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
      }
      tmem_ld32(T_S + c * 32, r);
      tmem_ld_wait();
      if (!last) {
#pragma unroll
        for (int j = 0; j < 32; j += 8)
          *reinterpret_cast<uint4*>(bST + op_off(tid, c * 32 + j)) =
              make_uint4(pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                         pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])), pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
      } else if (!(p.no_store != nullptr && p.no_store[b])) {
        float* st = p.rec_state + (((size_t)p.slots[b] * p.Hv + hv) * GC) * GC;
#pragma unroll
        for (int j = 0; j < 32; ++j) st[(size_t)(c * 32 + j) * GC + tid] = __uint_as_float(r[j]);
      }
    }
    __syncthreads();
    mark(11);
  }
  if (p.prof && tid == 0) {
#pragma unroll
    for (int i = 0; i < 12; ++i) p.prof[(size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 16 + i] = t_ph[i];
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}


// =====================================================================================================================
// The same algorithm as two kernels.  Everything of a chunk that does not depend on the incoming state (A, T, U, W, the
// masked decayed Q K^T, gamma-scaled Q, decay-scaled K^T) is independent between chunks: `gdn_prep_kernel` computes it
// for all chunks of all sequences at once (one CTA per chunk and head, so a long prompt fills the GPU) and leaves five
// 32 KB operand images per chunk in a workspace, already in the shared-memory operand layout.  `gdn_scan_kernel` then
// walks the chunks of a sequence with the state in tensor memory: per chunk five bulk copies, four products and two
// register passes, about a seventh of the fused kernel's time per chunk.
// Workspace: [chunk id][head][5][128 x 128 bf16]: 0 = W, 1 = gamma-scaled Q, 2 = U, 3 = P, 4 = decay-scaled K^T; and
// chunk_decay[chunk id][head] = e^{G_C}.  Chunk ids count the chunks of the sequences this kernel pair handles, in batch order.

struct GdnSplitParams {
  GdnChunkParams c;
  uint8_t* ws;                 // operand images
  float* chunk_decay;          // [chunks][Hv]
  int B;
};

// chunk id of the first chunk of sequence b (sequences with fewer than min_rows new tokens own no chunk)
__device__ __forceinline__ int first_chunk_of(const GdnChunkParams& p, int b, int tid, float* scratch) {
  int mine = 0;
  for (int i = tid; i < b; i += 128) {
    const int n = p.q_start[i + 1] - p.q_start[i];
    if (n >= p.min_rows && n > 0) mine += (n + GC - 1) / GC;
  }
  int* si = reinterpret_cast<int*>(scratch);
  si[tid] = mine;
  __syncthreads();
  for (int o = 64; o > 0; o >>= 1) {
    if (tid < o) si[tid] += si[tid + o];
    __syncthreads();
  }
  const int r = si[0];
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(128, 1) gdn_prep_kernel(GdnSplitParams sp) {
  const GdnChunkParams& p = sp.c;
  const int b = blockIdx.x, hv = blockIdx.y, ch = blockIdx.z;
  const int r0 = p.q_start[b], n = p.q_start[b + 1] - r0;
  const int c0 = ch * GC;
  if (n < p.min_rows || n <= 0 || c0 >= n) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int hk = hv / (p.Hv / p.Hk);
  const int Cch = 2 * p.Hk * GC + p.Hv * GC;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bK = smem;                 // K rows -> W rows            (with bT: the fp32 scratch matrix)
  uint8_t* bT = smem + GBUF;          // T (scaled) rows -> U rows
  uint8_t* bQ = smem + 2 * GBUF;      // Q rows -> gamma-scaled
  uint8_t* bVT = smem + 3 * GBUF;     // V^T -> P rows
  uint8_t* bKT = smem + 4 * GBUF;     // K^T -> decay-scaled
  float* Mf = reinterpret_cast<float*>(smem);
  float* s_G = reinterpret_cast<float*>(smem + 5 * GBUF);
  float* s_beta = s_G + GC;
  float* s_w = s_beta + GC;
  uint64_t* bar = reinterpret_cast<uint64_t*>(s_w + GC);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int chunk_id = first_chunk_of(p, b, tid, s_w) + ch;
  if (tid == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  const uint32_t T_1 = tmem + 128 + lane_base, T_2 = tmem + 256 + lane_base, T_3 = tmem + 384 + lane_base;
  uint32_t phase = 0;
  bool ok = true;
  auto mma = [&](uint32_t d_col, const uint8_t* A, const uint8_t* Bm, bool accumulate) {
    const uint32_t a = smem_u32(A), bb = smem_u32(Bm);
#pragma unroll
    for (int ks = 0; ks < GC / 16; ++ks)
      mma_f16(tmem + d_col, make_smem_desc(a + ks * 256, 128, 2048, kSwzNone), make_smem_desc(bb + ks * 256, 128, 2048, kSwzNone),
              make_idesc(1, 1, 128, 128), (accumulate || ks > 0) ? 1u : 0u);
  };
  auto run = [&](auto&& issue) {
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      issue();
      mma_commit(bar);
    }
    ok = __syncthreads_and(mbar_wait(bar, phase, abort_flag, p.status)) != 0;
    phase ^= 1;
    tc_fence_after();
  };
  const float Aexp = __expf(p.A_log[hv]);
  const float dtb = p.dt_bias[hv];
  const int L = min(GC, n - c0);
  const bool live = tid < L;
  const size_t row = (size_t)(r0 + c0 + tid);
  float g = 0.f, beta = 0.f;
  if (live) {
    const float av = bf2f(p.a_in[row * p.ld_ab + hv]) + dtb;
    const float spl = av > 20.f ? av : log1pf(__expf(av));
    g = -Aexp * spl;
    beta = bf2f(__float2bfloat16(1.f / (1.f + __expf(-bf2f(p.b_in[row * p.ld_ab + hv])))));
  }
  float G = g;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, G, o);
    if ((tid & 31) >= o) G += t;
  }
  if ((tid & 31) == 31) s_w[warp] = G;
  __syncthreads();
  for (int w = 0; w < warp; ++w) G += s_w[w];
  s_G[tid] = G;
  s_beta[tid] = beta;
  __syncthreads();
  const float G_C = s_G[GC - 1];
  {
    const __nv_bfloat16* src = p.conv + row * Cch + (size_t)p.Hk * GC + (size_t)hk * GC;
    uint4 u[16];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      u[j] = live ? *reinterpret_cast<const uint4*>(src + j * 8) : make_uint4(0, 0, 0, 0);
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u[j]);
#pragma unroll
      for (int q = 0; q < 8; ++q) ss += bf2f(e[q]) * bf2f(e[q]);
    }
    const float kn = rsqrtf(ss + 1e-6f);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u[j]);
      __nv_bfloat16 o8[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        o8[q] = __float2bfloat16(bf2f(e[q]) * kn);
        *reinterpret_cast<__nv_bfloat16*>(bKT + op_off(j * 8 + q, tid)) = o8[q];
      }
      *reinterpret_cast<uint4*>(bK + op_off(tid, j * 8)) = *reinterpret_cast<const uint4*>(o8);
    }
  }
  {
    const __nv_bfloat16* src = p.conv + row * Cch + (size_t)hk * GC;
    uint4 u[16];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      u[j] = live ? *reinterpret_cast<const uint4*>(src + j * 8) : make_uint4(0, 0, 0, 0);
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u[j]);
#pragma unroll
      for (int q = 0; q < 8; ++q) ss += bf2f(e[q]) * bf2f(e[q]);
    }
    const float qn = rsqrtf(ss + 1e-6f) * rsqrtf((float)GC);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u[j]);
      __nv_bfloat16 o8[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) o8[q] = __float2bfloat16(bf2f(e[q]) * qn);
      *reinterpret_cast<uint4*>(bQ + op_off(tid, j * 8)) = *reinterpret_cast<const uint4*>(o8);
    }
  }
  {
    const __nv_bfloat16* src = p.conv + row * Cch + 2 * (size_t)p.Hk * GC + (size_t)hv * GC;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint4 u = live ? *reinterpret_cast<const uint4*>(src + j * 8) : make_uint4(0, 0, 0, 0);
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
      for (int q = 0; q < 8; ++q) *reinterpret_cast<__nv_bfloat16*>(bVT + op_off(j * 8 + q, tid)) = e[q];
    }
  }
  run([&] { mma(128, bK, bK, false); mma(256, bQ, bK, false); });
  if (ok) {
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(T_1 + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int col = c * 32 + j;
        Mf[f_idx(tid, col)] = col < tid ? beta * __uint_as_float(r[j]) * __expf(G - s_G[col]) : 0.f;
      }
    }
    __syncthreads();
    {
      const int bb = tid >> 4, cc = tid & 15, o = bb * 16;
      float x[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float acc = (i == cc) ? 1.f : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (j < i) acc -= Mf[f_idx(o + i, o + j)] * x[j];
        x[i] = i >= cc ? acc : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 16; ++i) Mf[f_idx(o + i, o + cc)] = x[i];
      __syncthreads();
    }
    tri_product<16, false>(Mf, tid, 0, 16, 16, 0, 0, 0, 1.f);
    tri_product<16, true>(Mf, tid, 16, 0, 16, 16, 0, 16, -1.f);
    tri_product<32, false>(Mf, tid, 0, 32, 32, 0, 0, 0, 1.f);
    tri_product<32, true>(Mf, tid, 32, 0, 32, 32, 0, 32, -1.f);
    tri_product<64, false>(Mf, tid, 0, 64, 64, 0, 0, 0, 1.f);
    tri_product<64, true>(Mf, tid, 64, 0, 64, 64, 0, 64, -1.f);
  }
  float trow[GC];
#pragma unroll
  for (int j = 0; j < GC; ++j) trow[j] = (ok && j <= tid) ? Mf[f_idx(tid, j)] : 0.f;
  __syncthreads();
  auto write_T = [&](bool with_gamma) {
#pragma unroll
    for (int j = 0; j < GC; j += 8) {
      float s[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) s[q] = trow[j + q] * s_beta[j + q] * (with_gamma ? __expf(s_G[j + q]) : 1.f);
      *reinterpret_cast<uint4*>(bT + op_off(tid, j)) =
          make_uint4(pack_bf16x2(s[0], s[1]), pack_bf16x2(s[2], s[3]), pack_bf16x2(s[4], s[5]), pack_bf16x2(s[6], s[7]));
    }
  };
  if (ok) {
    write_T(false);
    run([&] { mma(128, bT, bVT, false); });        // U -> T_1
  }
  if (ok) {
    write_T(true);
    run([&] { mma(384, bT, bKT, false); });        // W -> T_3
  }
  if (ok) {
    // W rows -> bK, U rows -> bT, P rows -> bVT (V^T is no longer needed), Q rows scaled by gamma, K^T columns by e^{G_C - G_j}
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(T_3 + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        *reinterpret_cast<uint4*>(bK + op_off(tid, c * 32 + j)) =
            make_uint4(pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                       pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])), pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
      tmem_ld32(T_1 + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        *reinterpret_cast<uint4*>(bT + op_off(tid, c * 32 + j)) =
            make_uint4(pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                       pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])), pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
      tmem_ld32(T_2 + c * 32, r);
      tmem_ld_wait();
      float pv[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int col = c * 32 + j;
        pv[j] = col <= tid ? __uint_as_float(r[j]) * __expf(G - s_G[col]) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        *reinterpret_cast<uint4*>(bVT + op_off(tid, c * 32 + j)) =
            make_uint4(pack_bf16x2(pv[j], pv[j + 1]), pack_bf16x2(pv[j + 2], pv[j + 3]), pack_bf16x2(pv[j + 4], pv[j + 5]),
                       pack_bf16x2(pv[j + 6], pv[j + 7]));
    }
    {
      const float gam = __expf(G), kap = __expf(G_C - G);
#pragma unroll
      for (int j = 0; j < GC; j += 8) {
        uint4 u = *reinterpret_cast<uint4*>(bQ + op_off(tid, j));
        __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&u);
#pragma unroll
        for (int q = 0; q < 8; ++q) e[q] = __float2bfloat16(bf2f(e[q]) * gam);
        *reinterpret_cast<uint4*>(bQ + op_off(tid, j)) = u;
      }
#pragma unroll 4
      for (int d = 0; d < GC; ++d) {
        __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(bKT + op_off(d, tid));
        *e = __float2bfloat16(bf2f(*e) * kap);
      }
    }
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      uint8_t* dst = sp.ws + ((size_t)chunk_id * p.Hv + hv) * 5 * GBUF;
      bulk_store(dst, bK, GBUF);
      bulk_store(dst + GBUF, bQ, GBUF);
      bulk_store(dst + 2 * GBUF, bT, GBUF);
      bulk_store(dst + 3 * GBUF, bVT, GBUF);
      bulk_store(dst + 4 * GBUF, bKT, GBUF);
      tma_store_commit();
      tma_store_wait_all();
      sp.chunk_decay[(size_t)chunk_id * p.Hv + hv] = __expf(G_C);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

__global__ void __launch_bounds__(128, 1) gdn_scan_kernel(GdnSplitParams sp) {
  const GdnChunkParams& p = sp.c;
  const int b = blockIdx.x, hv = blockIdx.y;
  const int r0 = p.q_start[b], n = p.q_start[b + 1] - r0;
  if (n < p.min_rows || n <= 0) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const bool fresh = p.ctx_len[b] - n == 0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bK = smem;                 // W rows
  uint8_t* bT = smem + GBUF;          // P rows
  uint8_t* bQ = smem + 2 * GBUF;      // gamma-scaled Q rows
  uint8_t* bVT = smem + 3 * GBUF;     // U rows -> D^T
  uint8_t* bKT = smem + 4 * GBUF;     // decay-scaled K^T
  uint8_t* bST = smem + 5 * GBUF;     // S^T rows (bf16 copy of the state)
  float* s_w = reinterpret_cast<float*>(smem + 6 * GBUF);
  uint64_t* bar = reinterpret_cast<uint64_t*>(s_w + GC);
  uint64_t* bar_ld = bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_ld + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int chunk0 = first_chunk_of(p, b, tid, s_w);
  if (tid == 0) {
    mbar_init(bar, 1);
    mbar_init(bar_ld, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  const uint32_t T_S = tmem + lane_base, T_2 = tmem + 256 + lane_base, T_3 = tmem + 384 + lane_base;
  uint32_t phase = 0, ld_phase = 0;
  bool ok = true;
  auto mma = [&](uint32_t d_col, const uint8_t* A, const uint8_t* Bm, bool accumulate) {
    const uint32_t a = smem_u32(A), bb = smem_u32(Bm);
#pragma unroll
    for (int ks = 0; ks < GC / 16; ++ks)
      mma_f16(tmem + d_col, make_smem_desc(a + ks * 256, 128, 2048, kSwzNone), make_smem_desc(bb + ks * 256, 128, 2048, kSwzNone),
              make_idesc(1, 1, 128, 128), (accumulate || ks > 0) ? 1u : 0u);
  };
  auto run = [&](auto&& issue) {
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      issue();
      mma_commit(bar);
    }
    ok = __syncthreads_and(mbar_wait(bar, phase, abort_flag, p.status)) != 0;
    phase ^= 1;
    tc_fence_after();
  };
  // the chunk's five operand images; issued by thread 0 once every thread is done with the buffers
  auto load_chunk = [&](int chunk_id) {
    if (tid == 0) {
      const uint8_t* src = sp.ws + ((size_t)chunk_id * p.Hv + hv) * 5 * GBUF;
      mbar_expect_tx(bar_ld, 5 * GBUF);
      bulk_load(bK, src, GBUF, bar_ld);
      bulk_load(bQ, src + GBUF, GBUF, bar_ld);
      bulk_load(bVT, src + 2 * GBUF, GBUF, bar_ld);
      bulk_load(bT, src + 3 * GBUF, GBUF, bar_ld);
      bulk_load(bKT, src + 4 * GBUF, GBUF, bar_ld);
    }
  };
  load_chunk(chunk0);
  {
    const float* st = p.rec_state + (((size_t)p.slots[b] * p.Hv + hv) * GC) * GC;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = fresh ? 0u : __float_as_uint(st[(size_t)(c * 32 + j) * GC + tid]);
      tmem_st32(T_S + c * 32, r);
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        *reinterpret_cast<uint4*>(bST + op_off(tid, c * 32 + j)) =
            make_uint4(pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                       pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])), pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
    }
    tmem_st_wait();
  }
  const int nch = (n + GC - 1) / GC;
  for (int ci = 0; ci < nch && ok; ++ci) {
    const int c0 = ci * GC;
    const int L = min(GC, n - c0);
    const bool live = tid < L;
    const size_t row = (size_t)(r0 + c0 + tid);
    ok = __syncthreads_and(mbar_wait(bar_ld, ld_phase, abort_flag, p.status)) != 0;
    ld_phase ^= 1;
    if (!ok) break;
    // ---- D5 = W S0 -> T_3;  O = (gamma Q) S0 -> T_2 ; meanwhile this thread's U row goes to registers
    uint4 urow[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) urow[j] = *reinterpret_cast<const uint4*>(bVT + op_off(tid, j * 8));
    run([&] { mma(384, bK, bST, false); mma(256, bQ, bST, false); });
    if (!ok) break;
    {
      const float dec = sp.chunk_decay[(size_t)(chunk0 + ci) * p.Hv + hv];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t w[32], u[32];
        tmem_ld32(T_3 + c * 32, w);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&urow[c * 4 + (j >> 3)]);
          *reinterpret_cast<__nv_bfloat16*>(bVT + op_off(c * 32 + j, tid)) = __float2bfloat16(bf2f(e[j & 7]) - __uint_as_float(w[j]));
        }
        tmem_ld32(T_S + c * 32, u);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) u[j] = __float_as_uint(__uint_as_float(u[j]) * dec);
        tmem_st32(T_S + c * 32, u);
      }
      tmem_st_wait();
    }
    // ---- O += P D;   S^T += D^T (K scaled)
    run([&] { mma(256, bT, bVT, true); mma(0, bVT, bKT, true); });
    if (!ok) break;
    const bool last = ci + 1 >= nch;
    if (!last) load_chunk(chunk0 + ci + 1);      // every product that read the buffers has completed
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(T_2 + c * 32, r);
      tmem_ld_wait();
      if (live) {
        __nv_bfloat16* dst = p.out + (row * p.Hv + hv) * GC + c * 32;
#pragma unroll
        for (int j = 0; j < 32; j += 8)
          *reinterpret_cast<uint4*>(dst + j) =
              make_uint4(pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                         pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])), pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
      }
      tmem_ld32(T_S + c * 32, r);
      tmem_ld_wait();
      if (!last) {
#pragma unroll
        for (int j = 0; j < 32; j += 8)
          *reinterpret_cast<uint4*>(bST + op_off(tid, c * 32 + j)) =
              make_uint4(pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                         pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])), pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
      } else if (!(p.no_store != nullptr && p.no_store[b])) {
        float* st = p.rec_state + (((size_t)p.slots[b] * p.Hv + hv) * GC) * GC;
#pragma unroll
        for (int j = 0; j < 32; ++j) st[(size_t)(c * 32 + j) * GC + tid] = __uint_as_float(r[j]);
      }
    }
    __syncthreads();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace blz

namespace { thread_local long long* g_gdn_prof = nullptr; }
// Diagnostics: the NEXT blz_gdn_chunk call on this thread records, per CTA (index head * sequences + sequence) in prof[..][16],
// the cycles thread 0 spent in: 0 set-up + state load, 1 gates + operand loads, 2 K K^T / Q K^T, 3 A, 4 inverse, 5 T rows,
// 6 U and W products, 7 W / P / scaling passes, 8 W S0 and Q S0, 9 D and state decay, 10 P D and state update, 11 outputs.
BLZ_API int blz_gdn_chunk_profile(void* prof) { g_gdn_prof = reinterpret_cast<long long*>(prof); return 0; }

// Gated delta rule over every sequence of the batch that has at least `min_rows` new tokens (the others are left to
// blz_gdn_recurrent, which takes the complementary `max_rows`).  Head dims 128 / 128.  Arguments as blz_gdn_recurrent.
BLZ_API int blz_gdn_chunk(const void* conv, const void* a_in, const void* b_in, long long ld_ab, const float* A_log,
                          const float* dt_bias, float* rec_state, void* out, const int* slots, const int* q_start,
                          const int* ctx_len, const int* no_store, int B, int Hk, int Hv, int DK, int DV, int min_rows,
                          cudaStream_t s) {
  using namespace blz;
  if (B == 0) return 0;
  if (DK != 128 || DV != 128 || Hv % Hk || !out) return (int)cudaErrorInvalidValue;
  GdnChunkParams p;
  p.conv = (const __nv_bfloat16*)conv; p.a_in = (const __nv_bfloat16*)a_in; p.b_in = (const __nv_bfloat16*)b_in;
  p.ld_ab = ld_ab; p.A_log = A_log; p.dt_bias = dt_bias; p.rec_state = rec_state; p.out = (__nv_bfloat16*)out;
  p.slots = slots; p.q_start = q_start; p.ctx_len = ctx_len; p.no_store = no_store; p.Hk = Hk; p.Hv = Hv;
  p.min_rows = min_rows < 1 ? 1 : min_rows;
  p.status = status_word();
  p.prof = g_gdn_prof;
  g_gdn_prof = nullptr;
  static PerDeviceOnce configured;
  cudaError_t e = configured.smem_limit(gdn_chunk_kernel, GDN_SMEM);
  if (e != cudaSuccess) return (int)e;
  gdn_chunk_kernel<<<dim3(B, Hv), 128, GDN_SMEM, s>>>(p);
  return (int)cudaGetLastError();
}

// Workspace bytes blz_gdn_chunk_split needs for `chunks` chunks (sum over its sequences of ceil(new tokens / 128)) and Hv heads.
BLZ_API long long blz_gdn_chunk_ws_bytes(int chunks, int Hv) { return (long long)chunks * Hv * (5LL * blz::GBUF + 4); }

// The chunked rule as two kernels (see gdn_prep_kernel): ws holds blz_gdn_chunk_ws_bytes(chunks, Hv) bytes, max_q is the longest
// run of the batch.  Other arguments as blz_gdn_chunk.
BLZ_API int blz_gdn_chunk_split(const void* conv, const void* a_in, const void* b_in, long long ld_ab, const float* A_log,
                                const float* dt_bias, float* rec_state, void* out, const int* slots, const int* q_start,
                                const int* ctx_len, const int* no_store, int B, int Hk, int Hv, int DK, int DV, int min_rows,
                                int max_q, int chunks, void* ws, cudaStream_t s) {
  using namespace blz;
  if (B == 0 || chunks <= 0) return 0;
  if (DK != 128 || DV != 128 || Hv % Hk || !out || !ws || max_q < 1) return (int)cudaErrorInvalidValue;
  GdnSplitParams sp;
  GdnChunkParams& p = sp.c;
  p.conv = (const __nv_bfloat16*)conv; p.a_in = (const __nv_bfloat16*)a_in; p.b_in = (const __nv_bfloat16*)b_in;
  p.ld_ab = ld_ab; p.A_log = A_log; p.dt_bias = dt_bias; p.rec_state = rec_state; p.out = (__nv_bfloat16*)out;
  p.slots = slots; p.q_start = q_start; p.ctx_len = ctx_len; p.no_store = no_store; p.Hk = Hk; p.Hv = Hv;
  p.min_rows = min_rows < 1 ? 1 : min_rows;
  p.status = status_word();
  p.prof = nullptr;
  sp.ws = reinterpret_cast<uint8_t*>(ws);
  sp.chunk_decay = reinterpret_cast<float*>(sp.ws + (size_t)chunks * Hv * 5 * GBUF);
  sp.B = B;
  constexpr int PREP_SMEM = 5 * GBUF + 1024 + 3 * GC * 4 + 64;
  constexpr int SCAN_SMEM = 6 * GBUF + 1024 + GC * 4 + 64;
  static PerDeviceOnce c1, c2;
  cudaError_t e = c1.smem_limit(gdn_prep_kernel, PREP_SMEM);
  if (e != cudaSuccess) return (int)e;
  e = c2.smem_limit(gdn_scan_kernel, SCAN_SMEM);
  if (e != cudaSuccess) return (int)e;
  gdn_prep_kernel<<<dim3(B, Hv, (max_q + GC - 1) / GC), 128, PREP_SMEM, s>>>(sp);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  gdn_scan_kernel<<<dim3(B, Hv), 128, SCAN_SMEM, s>>>(sp);
  return (int)cudaGetLastError();
}
