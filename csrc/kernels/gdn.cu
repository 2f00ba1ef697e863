// Gated DeltaNet (linear-attention) layer kernels:
//   conv      : causal depthwise conv (kernel <= 8) + SiLU over variable-length sequences with a per-sequence state of the
//               last k-1 inputs (reference: kernels/src/cuda/ops_basic.cu gdn_conv_kernel :319)
//   recurrent : the gated delta rule, token by token, with the gates computed in the kernel
//               g = -exp(A_log) * softplus(a + dt_bias), beta = bf16(sigmoid(b))      (ops_basic.cu gdn_gate :301)
//               S <- S * exp(g);  delta = (v - S^T k) * beta;  S <- S + k delta^T;  o = S^T q
//               with q, k L2-normalised and q scaled by dk^-1/2               (kernels/src/cuda/gdn_recurrent.cu:27-92)
//   gated norm: per-head RMSNorm of o times silu(z)                           (ops_basic.cu gated_rmsnorm_kernel :70)
// State layout: conv_state [rows, C, k-1] bf16, rec_state [rows, Hv, dk, dv] fp32; rows are sequence slots.
#include "blaze/host.h"
#include "blaze/sm100.cuh"

namespace blz {

// grid (ceil(C / 128), B); thread = channel; walks the sequence's tokens in order
template <int KW>
__global__ void gdn_conv_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, __nv_bfloat16* __restrict__ y,
                                __nv_bfloat16* __restrict__ conv_state, const __nv_bfloat16* __restrict__ w,
                                const int* __restrict__ slots, const int* __restrict__ q_start, const int* __restrict__ ctx_len,
                                const int* __restrict__ no_store, int C, int max_rows) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= C) return;
  const int r0 = q_start[b], n = q_start[b + 1] - r0;
  if (n <= 0 || n > max_rows) return;
  const bool fresh = ctx_len[b] - n == 0;
  __nv_bfloat16* st = conv_state + ((size_t)slots[b] * C + c) * (KW - 1);
  float h[KW];
  float wt[KW];
#pragma unroll
  for (int j = 0; j < KW - 1; ++j) h[j] = fresh ? 0.f : bf2f(st[j]);
#pragma unroll
  for (int j = 0; j < KW; ++j) wt[j] = bf2f(w[(size_t)c * KW + j]);
  for (int t = 0; t < n; ++t) {
    h[KW - 1] = bf2f(x[(size_t)(r0 + t) * ldx + c]);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < KW; ++j) acc += h[j] * wt[j];
    const float r = bf2f(__float2bfloat16(acc));
    y[(size_t)(r0 + t) * C + c] = __float2bfloat16(r / (1.f + __expf(-r)));
#pragma unroll
    for (int j = 0; j < KW - 1; ++j) h[j] = h[j + 1];
  }
  if (no_store != nullptr && no_store[b]) return;      // speculative rows: the state advances when they are replayed
#pragma unroll
  for (int j = 0; j < KW - 1; ++j) st[j] = __float2bfloat16(h[j]);
}

// Long token runs (prompts): the same convolution with the tokens spread over the grid.  grid (ceil(C / 128), B, segments):
// segment z handles tokens [z * SEG, (z + 1) * SEG) of the sequence; the k-1 inputs before its first token come from the input
// itself (or from the state for the run's first tokens); the CTA that holds the run's last token writes the new state.
template <int KW>
__global__ void gdn_conv_par_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, __nv_bfloat16* __restrict__ y,
                                    __nv_bfloat16* __restrict__ conv_state, const __nv_bfloat16* __restrict__ w,
                                    const int* __restrict__ slots, const int* __restrict__ q_start, const int* __restrict__ ctx_len,
                                    const int* __restrict__ no_store, int C, int seg, int min_rows) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= C) return;
  const int r0 = q_start[b], n = q_start[b + 1] - r0;
  if (n < min_rows) return;                        // short runs belong to the sequential kernel
  const int t0 = blockIdx.z * seg, t1 = min(n, t0 + seg);
  if (t0 >= n) return;
  const bool fresh = ctx_len[b] - n == 0;
  __nv_bfloat16* st = conv_state + ((size_t)slots[b] * C + c) * (KW - 1);
  float h[KW];
  float wt[KW];
#pragma unroll
  for (int j = 0; j < KW - 1; ++j) {
    const int t = t0 - (KW - 1) + j;              // input position of history slot j (negative: before this run)
    h[j] = t >= 0 ? bf2f(x[(size_t)(r0 + t) * ldx + c]) : (fresh ? 0.f : bf2f(st[KW - 1 + t]));
  }
#pragma unroll
  for (int j = 0; j < KW; ++j) wt[j] = bf2f(w[(size_t)c * KW + j]);
  for (int t = t0; t < t1; ++t) {
    h[KW - 1] = bf2f(x[(size_t)(r0 + t) * ldx + c]);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < KW; ++j) acc += h[j] * wt[j];
    const float r = bf2f(__float2bfloat16(acc));
    y[(size_t)(r0 + t) * C + c] = __float2bfloat16(r / (1.f + __expf(-r)));
#pragma unroll
    for (int j = 0; j < KW - 1; ++j) h[j] = h[j + 1];
  }
  if (t1 == n && !(no_store != nullptr && no_store[b])) {
#pragma unroll
    for (int j = 0; j < KW - 1; ++j) st[j] = __float2bfloat16(h[j]);
  }
}

// grid (B, Hv, DV / 32), 128 threads: thread = (dv column c = tid % 32, dk quarter qt = tid / 32); the state slice
// [DK][32] sits in registers (DK / 4 values per thread).
template <int DK>
__global__ void __launch_bounds__(128) gdn_recurrent_kernel(
    const __nv_bfloat16* __restrict__ conv, const __nv_bfloat16* __restrict__ a_in, const __nv_bfloat16* __restrict__ b_in,
    long long ld_ab, const float* __restrict__ A_log, const float* __restrict__ dt_bias, float* __restrict__ rec_state,
    __nv_bfloat16* __restrict__ out, const int* __restrict__ slots, const int* __restrict__ q_start,
    const int* __restrict__ ctx_len, const int* __restrict__ no_store, int Hk, int Hv, int DV, int max_rows) {
  constexpr int PER = DK / 4;
  const int b = blockIdx.x, hv = blockIdx.y, slice = blockIdx.z;
  const int tid = threadIdx.x, c = tid & 31, qt = tid >> 5;
  const int r0 = q_start[b], n = q_start[b + 1] - r0;
  if (n <= 0 || n > max_rows) return;          // longer runs belong to the chunked kernel
  const bool fresh = ctx_len[b] - n == 0;
  const int hk = hv / (Hv / Hk);
  const int C = 2 * Hk * DK + Hv * DV;                      // conv channels: [q | k | v]
  const int col = slice * 32 + c;
  float* st = rec_state + (((size_t)slots[b] * Hv + hv) * DK) * DV;
  float S[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) S[i] = fresh ? 0.f : st[(size_t)(qt * PER + i) * DV + col];
  __shared__ float s_q[DK], s_k[DK], s_red[2][4][32], s_nrm[2][4];
  const float Aexp = __expf(A_log[hv]);
  const float dtb = dt_bias[hv];
  for (int t = 0; t < n; ++t) {
    const size_t row = (size_t)(r0 + t);
    // ---- L2-normalise q and k of the key head (DK <= 128: one element per thread)
    float qv = 0.f, kv = 0.f;
    if (tid < DK) {
      qv = bf2f(conv[row * C + (size_t)hk * DK + tid]);
      kv = bf2f(conv[row * C + (size_t)Hk * DK + (size_t)hk * DK + tid]);
    }
    const float qs = warp_sum(qv * qv), ks = warp_sum(kv * kv);
    if (c == 0) { s_nrm[0][qt] = qs; s_nrm[1][qt] = ks; }
    __syncthreads();
    const float qn = rsqrtf(s_nrm[0][0] + s_nrm[0][1] + s_nrm[0][2] + s_nrm[0][3] + 1e-6f) * rsqrtf((float)DK);
    const float kn = rsqrtf(s_nrm[1][0] + s_nrm[1][1] + s_nrm[1][2] + s_nrm[1][3] + 1e-6f);
    if (tid < DK) { s_q[tid] = qv * qn; s_k[tid] = kv * kn; }
    const float av = bf2f(a_in[row * ld_ab + hv]) + dtb;
    const float sp = av > 20.f ? av : log1pf(__expf(av));
    const float decay = __expf(-Aexp * sp);
    const float beta = bf2f(__float2bfloat16(1.f / (1.f + __expf(-bf2f(b_in[row * ld_ab + hv])))));
    const float v = bf2f(conv[row * C + 2 * (size_t)Hk * DK + (size_t)hv * DV + col]);
    __syncthreads();
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) { S[i] *= decay; part += S[i] * s_k[qt * PER + i]; }
    s_red[0][qt][c] = part;
    __syncthreads();
    const float kvS = s_red[0][0][c] + s_red[0][1][c] + s_red[0][2][c] + s_red[0][3][c];
    const float delta = (v - kvS) * beta;
    float po = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) { S[i] += s_k[qt * PER + i] * delta; po += S[i] * s_q[qt * PER + i]; }
    s_red[1][qt][c] = po;
    __syncthreads();
    if (qt == 0 && out != nullptr)
      out[(row * Hv + hv) * DV + col] = __float2bfloat16(s_red[1][0][c] + s_red[1][1][c] + s_red[1][2][c] + s_red[1][3][c]);
  }
  if (no_store != nullptr && no_store[b]) return;
#pragma unroll
  for (int i = 0; i < PER; ++i) st[(size_t)(qt * PER + i) * DV + col] = S[i];
}

// one warp per (token, head): y = rmsnorm(o) * w * gate(z), gate = silu, or sigmoid with flag bit 1 (a checkpoint's
// output_gate_type); flag bit 0: w is stored as w - 1
__global__ void gated_rmsnorm_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ z, long long ldz,
                                     const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int rows, int Hv, int DV,
                                     float eps, int flags) {
  const bool zero_centered = flags & 1, sigmoid_gate = flags & 2;
  const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (wid >= rows * Hv) return;
  const int t = wid / Hv, h = wid % Hv;
  const __nv_bfloat16* src = o + ((size_t)t * Hv + h) * DV;
  const __nv_bfloat16* zz = z + (size_t)t * ldz + (size_t)h * DV;
  float ss = 0.f;
  for (int i = lane; i < DV; i += 32) { const float f = bf2f(src[i]); ss += f * f; }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / DV + eps);
  for (int i = lane; i < DV; i += 32) {
    const float g = bf2f(zz[i]);
    const float wf = bf2f(w[i]) + (zero_centered ? 1.f : 0.f);
    const float sg = 1.f / (1.f + __expf(-g));
    y[((size_t)t * Hv + h) * DV + i] = __float2bfloat16(bf2f(src[i]) * rstd * wf * (sigmoid_gate ? sg : g * sg));
  }
}

}  // namespace blz

using namespace blz;
typedef __nv_bfloat16 bf16;

// no_store (both kernels, optional [B]): 1 = read the sequence's state but leave it as it was (speculative rows).
// blz_gdn_recurrent: out may be null (state advance only, used when accepted rows are replayed).
// max_q: the longest token run of the batch (host knowledge).  Runs of at least 64 tokens are convolved with the tokens
// spread over the grid (64-token segments), the others by one thread per channel walking the run.
static int gdn_conv_impl(const void* x, long long ldx, void* y, void* conv_state, const void* w, const int* slots,
                         const int* q_start, const int* ctx_len, const int* no_store, int B, int C, int kw, int max_q,
                         cudaStream_t s) {
  if (B == 0) return 0;
  constexpr int SEG = 64, LONG = 64;
  const bool par = max_q >= LONG;
  dim3 grid((C + 127) / 128, B);
  dim3 grid_par((C + 127) / 128, B, par ? (max_q + SEG - 1) / SEG : 1);
#define BLZ_CONV(K)                                                                                                         \
  do {                                                                                                                      \
    if (par)                                                                                                                \
      gdn_conv_par_kernel<K><<<grid_par, 128, 0, s>>>((const bf16*)x, ldx, (bf16*)y, (bf16*)conv_state, (const bf16*)w, slots, \
                                                      q_start, ctx_len, no_store, C, SEG, LONG);                            \
    if (!par || B > 1)                                                                                                      \
      gdn_conv_kernel<K><<<grid, 128, 0, s>>>((const bf16*)x, ldx, (bf16*)y, (bf16*)conv_state, (const bf16*)w, slots,      \
                                              q_start, ctx_len, no_store, C, par ? LONG - 1 : 0x7fffffff);                  \
  } while (0)
  switch (kw) {
    case 2: BLZ_CONV(2); break;
    case 3: BLZ_CONV(3); break;
    case 4: BLZ_CONV(4); break;
    case 8: BLZ_CONV(8); break;
    default: return (int)cudaErrorInvalidValue;
  }
#undef BLZ_CONV
  return (int)cudaGetLastError();
}
BLZ_API int blz_gdn_conv(const void* x, long long ldx, void* y, void* conv_state, const void* w, const int* slots,
                         const int* q_start, const int* ctx_len, const int* no_store, int B, int C, int kw, cudaStream_t s) {
  return gdn_conv_impl(x, ldx, y, conv_state, w, slots, q_start, ctx_len, no_store, B, C, kw, 0, s);
}
BLZ_API int blz_gdn_conv_runs(const void* x, long long ldx, void* y, void* conv_state, const void* w, const int* slots,
                              const int* q_start, const int* ctx_len, const int* no_store, int B, int C, int kw, int max_q,
                              cudaStream_t s) {
  return gdn_conv_impl(x, ldx, y, conv_state, w, slots, q_start, ctx_len, no_store, B, C, kw, max_q, s);
}

static int gdn_recurrent_impl(const void* conv, const void* a_in, const void* b_in, long long ld_ab, const float* A_log,
                              const float* dt_bias, float* rec_state, void* out, const int* slots, const int* q_start,
                              const int* ctx_len, const int* no_store, int B, int Hk, int Hv, int DK, int DV, int max_rows,
                              cudaStream_t s);
BLZ_API int blz_gdn_recurrent(const void* conv, const void* a_in, const void* b_in, long long ld_ab, const float* A_log,
                              const float* dt_bias, float* rec_state, void* out, const int* slots, const int* q_start,
                              const int* ctx_len, const int* no_store, int B, int Hk, int Hv, int DK, int DV, cudaStream_t s) {
  return gdn_recurrent_impl(conv, a_in, b_in, ld_ab, A_log, dt_bias, rec_state, out, slots, q_start, ctx_len, no_store, B, Hk, Hv,
                            DK, DV, 0x7fffffff, s);
}
// as above, for the sequences with at most max_rows new tokens (the chunked kernel takes the others)
BLZ_API int blz_gdn_recurrent_upto(const void* conv, const void* a_in, const void* b_in, long long ld_ab, const float* A_log,
                                   const float* dt_bias, float* rec_state, void* out, const int* slots, const int* q_start,
                                   const int* ctx_len, const int* no_store, int B, int Hk, int Hv, int DK, int DV, int max_rows,
                                   cudaStream_t s) {
  return gdn_recurrent_impl(conv, a_in, b_in, ld_ab, A_log, dt_bias, rec_state, out, slots, q_start, ctx_len, no_store, B, Hk, Hv,
                            DK, DV, max_rows, s);
}
static int gdn_recurrent_impl(const void* conv, const void* a_in, const void* b_in, long long ld_ab, const float* A_log,
                              const float* dt_bias, float* rec_state, void* out, const int* slots, const int* q_start,
                              const int* ctx_len, const int* no_store, int B, int Hk, int Hv, int DK, int DV, int max_rows,
                              cudaStream_t s) {
  if (B == 0) return 0;
  if (DK != 128 || DV % 32 || Hv % Hk) return (int)cudaErrorInvalidValue;
  dim3 grid(B, Hv, DV / 32);
  gdn_recurrent_kernel<128><<<grid, 128, 0, s>>>((const bf16*)conv, (const bf16*)a_in, (const bf16*)b_in, ld_ab, A_log, dt_bias,
                                                 rec_state, (bf16*)out, slots, q_start, ctx_len, no_store, Hk, Hv, DV, max_rows);
  return (int)cudaGetLastError();
}

// flags: bit 0 = weights stored as w - 1, bit 1 = multiply by sigmoid(z) instead of silu(z)
BLZ_API int blz_gated_rmsnorm(const void* o, const void* z, long long ldz, const void* w, void* y, int rows, int Hv, int DV,
                              float eps, int flags, cudaStream_t s) {
  if (rows == 0) return 0;
  const int warps = rows * Hv;
  gated_rmsnorm_kernel<<<(warps + 7) / 8, 256, 0, s>>>((const bf16*)o, (const bf16*)z, ldz, (const bf16*)w, (bf16*)y, rows, Hv, DV,
                                                       eps, flags);
  return (int)cudaGetLastError();
}
