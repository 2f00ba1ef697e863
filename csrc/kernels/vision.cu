// Vision-tower (ViT encoder) kernels around the tcgen05 GEMMs: LayerNorm with bias, tanh-GELU, 2-D rotary on the packed
// qkv rows, and a non-causal attention kernel for one image's patch tokens.
//
// The encoder runs once per image (a few thousand tokens, head_dim 64..128, 72 for Qwen3-VL), so attention is a plain
// flash-style CUDA-core kernel: one thread per query row keeps q and the output row in registers, the block streams
// K/V tiles through shared memory and every thread reads the same K element at the same time (a broadcast).
// The four projections of a block go through the bf16 tensor-core GEMM with the bias in its epilogue.
//
// Reference: kernels/src/cuda/vision.cu (layernorm :25, embed_pos :72, qkv_rope :102, attention_kernel :174,
// bias_residual :319, bias_act :331).
#include "blaze/host.h"
#include "blaze/sm100.cuh"

namespace blz {

// ---------------------------------------------------------------------------------------------- LayerNorm
// One warp per row; x, y bf16 [T, H]; w, b fp32-or-bf16 given as bf16.
__global__ void vit_layernorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                     const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, int T, int H, float eps) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= T) return;
  const __nv_bfloat16* xr = x + (size_t)row * H;
  float s = 0.f;
  for (int i = lane; i < H; i += 32) s += bf2f(xr[i]);
  const float mean = warp_sum(s) / H;
  float v = 0.f;
  for (int i = lane; i < H; i += 32) { const float d = bf2f(xr[i]) - mean; v += d * d; }
  const float rstd = rsqrtf(warp_sum(v) / H + eps);
  __nv_bfloat16* yr = y + (size_t)row * H;
  for (int i = lane; i < H; i += 32)
    yr[i] = __float2bfloat16((bf2f(xr[i]) - mean) * rstd * bf2f(w[i]) + (b ? bf2f(b[i]) : 0.f));
}

// ---------------------------------------------------------------------------------------------- GELU (tanh form), in place
__global__ void vit_gelu_kernel(__nv_bfloat16* x, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = bf2f(x[i]);
    x[i] = __float2bfloat16(0.5f * v * (1.f + tanhf(0.7978845608f * (v + 0.044715f * v * v * v))));
  }
}

// ---------------------------------------------------------------------------------------------- rotary on q and k
// qkv bf16 [T, 3H]; cos/sin fp32 [T, D/2]; pairs (i, i + D/2) of every head of q and k.
__global__ void vit_rope_kernel(__nv_bfloat16* qkv, const float* __restrict__ cs, const float* __restrict__ sn, int T, int H,
                                int heads) {
  const int D = H / heads, half = D / 2;
  const size_t total = (size_t)T * 2 * heads * half;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int i = idx % half;
    const int hd = (idx / half) % heads;
    const int which = (idx / ((size_t)half * heads)) % 2;
    const int t = idx / ((size_t)half * heads * 2);
    __nv_bfloat16* v = qkv + (size_t)t * 3 * H + (size_t)which * H + hd * D;
    const float c = cs[(size_t)t * half + i], s = sn[(size_t)t * half + i];
    const float a = bf2f(v[i]), b = bf2f(v[i + half]);
    v[i] = __float2bfloat16(a * c - b * s);
    v[i + half] = __float2bfloat16(b * c + a * s);
  }
}

// ---------------------------------------------------------------------------------------------- attention
// qkv bf16 [T, 3H] (q | k | v), tokens [t0, t1) attend to each other (one image); out bf16 [T, H].
// grid (ceil((t1 - t0) / 128), heads), block 128: one query row per thread.
template <int D>
__global__ void __launch_bounds__(128) vit_attention_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ out,
                                                            int t0, int t1, int H, float scale_log2) {
  constexpr int KT = 32;                      // keys per shared-memory tile
  __shared__ float sk[KT][D];
  __shared__ float sv[KT][D];
  const int head = blockIdx.y;
  const int tq = t0 + blockIdx.x * 128 + threadIdx.x;
  const bool live = tq < t1;
  float q[D], acc[D];
#pragma unroll
  for (int i = 0; i < D; ++i) {
    q[i] = live ? bf2f(qkv[(size_t)tq * 3 * H + head * D + i]) * scale_log2 : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int k0 = t0; k0 < t1; k0 += KT) {
    const int n = min(KT, t1 - k0);
    __syncthreads();
    for (int e = threadIdx.x; e < KT * D; e += 128) {
      const int r = e / D, c = e % D;
      const bool ok = r < n;
      sk[r][c] = ok ? bf2f(qkv[(size_t)(k0 + r) * 3 * H + H + head * D + c]) : 0.f;
      sv[r][c] = ok ? bf2f(qkv[(size_t)(k0 + r) * 3 * H + 2 * H + head * D + c]) : 0.f;
    }
    __syncthreads();
    float s[KT];
    float tile_max = -INFINITY;
#pragma unroll
    for (int r = 0; r < KT; ++r) {
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < D; ++i) d = fmaf(q[i], sk[r][i], d);
      s[r] = r < n ? d : -INFINITY;
      tile_max = fmaxf(tile_max, s[r]);
    }
    const float m_new = fmaxf(m, tile_max);
    const float corr = exp2f(m - m_new);
    l *= corr;
#pragma unroll
    for (int i = 0; i < D; ++i) acc[i] *= corr;
#pragma unroll
    for (int r = 0; r < KT; ++r) {
      const float p = exp2f(s[r] - m_new);
      l += p;
#pragma unroll
      for (int i = 0; i < D; ++i) acc[i] = fmaf(p, sv[r][i], acc[i]);
    }
    m = m_new;
  }
  if (live) {
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < D; ++i) out[(size_t)tq * H + head * D + i] = __float2bfloat16(acc[i] * inv);
  }
}

}  // namespace blz

using namespace blz;
typedef __nv_bfloat16 bf16;

BLZ_API int blz_vit_layernorm(const void* x, const void* w, const void* b, void* y, int T, int H, float eps, cudaStream_t s) {
  if (T <= 0) return 0;
  vit_layernorm_kernel<<<(T + 7) / 8, 256, 0, s>>>((const bf16*)x, (const bf16*)w, (const bf16*)b, (bf16*)y, T, H, eps);
  return (int)cudaGetLastError();
}

BLZ_API int blz_vit_gelu(void* x, long long n, cudaStream_t s) {
  if (n <= 0) return 0;
  const long long blocks = (n + 255) / 256;
  vit_gelu_kernel<<<(int)(blocks > 8192 ? 8192 : blocks), 256, 0, s>>>((bf16*)x, (size_t)n);
  return (int)cudaGetLastError();
}

BLZ_API int blz_vit_rope(void* qkv, const float* cs, const float* sn, int T, int H, int heads, cudaStream_t s) {
  if (T <= 0) return 0;
  if (heads <= 0 || H % heads || (H / heads) % 2) return (int)cudaErrorInvalidValue;
  const long long total = (long long)T * heads * (H / heads);
  const long long blocks = (total + 255) / 256;
  vit_rope_kernel<<<(int)(blocks > 8192 ? 8192 : blocks), 256, 0, s>>>((bf16*)qkv, cs, sn, T, H, heads);
  return (int)cudaGetLastError();
}

// head_dim in {32, 64, 72, 80, 96, 128}
BLZ_API int blz_vit_attention(const void* qkv, void* out, int t0, int t1, int H, int heads, cudaStream_t s) {
  if (t1 <= t0) return 0;
  if (heads <= 0 || H % heads) return (int)cudaErrorInvalidValue;
  const int D = H / heads;
  const dim3 grid((t1 - t0 + 127) / 128, heads);
  const float sl2 = 1.4426950408889634f / sqrtf((float)D);
#define BLZ_VA(DD) vit_attention_kernel<DD><<<grid, 128, 0, s>>>((const bf16*)qkv, (bf16*)out, t0, t1, H, sl2)
  switch (D) {
    case 32: BLZ_VA(32); break;
    case 64: BLZ_VA(64); break;
    case 72: BLZ_VA(72); break;
    case 80: BLZ_VA(80); break;
    case 96: BLZ_VA(96); break;
    case 128: BLZ_VA(128); break;
    default: return (int)cudaErrorInvalidValue;
  }
#undef BLZ_VA
  return (int)cudaGetLastError();
}
