// Bandwidth-bound fused ops around the GEMMs:
//   embedding gather; residual-add + RMSNorm (+ NVFP4 / MXFP8 row quantisation for the next GEMM);
//   SwiGLU (+ quantisation); per-head q/k RMSNorm + NeoX rotary + gate split + FP8 paged-KV write in the
//   tcgen05 attention layout; sigmoid gate; argmax with lowest-index ties; row gather.
//
// Same math as the reference's kernels/src/cuda/ops_basic.cu (rmsnorm_kernel :42, attn_prep_kernel :102,
// mul_sigmoid :161, silu_mul :166, argmax_kernel :249, gather_rows :346), kernels/src/cuda/nvfp4_gemm.cu
// quant_rows_kernel :33, kernels/src/cuda/nvfp4_kv.cu kv_store_dense_kernel :188 and embed.cu:6 — fused so
// that each activation makes one trip through HBM between GEMMs.
#include "blaze/host.h"
#include "blaze/sm100.cuh"

namespace blz {

// ---------------------------------------------------------------------------------------------- helpers
__device__ __forceinline__ float block_reduce(float v, float* sh, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float r = is_max ? -INFINITY : 0.f;
  for (int i = 0; i < nw; ++i) r = is_max ? fmaxf(r, sh[i]) : r + sh[i];
  return r;
}

__device__ __forceinline__ uint8_t f2e4m3(float x) {
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float e4m32f(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
// round to E2M1 code (sign bit 3); nearest, ties to the even code, saturating at 6
__device__ __forceinline__ uint32_t f2e2m1(float x) {
  const float a = fminf(fabsf(x), 6.0f);
  uint32_t c = (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.0f);
  return c | ((__float_as_uint(x) >> 31) << 3);
}
// byte offset of scale (row, col) in the 128x4-tiled scale array with `col_tiles` tiles per row tile
__device__ __forceinline__ size_t sf_offset(int row, int col, int col_tiles) {
  return ((size_t)(row >> 7) * col_tiles + (col >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (col & 3);
}

// ---------------------------------------------------------------------------------------------- embedding
__global__ void embed_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ tokens,
                             __nv_bfloat16* __restrict__ out, int H, int vocab) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)tok * H);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// ---------------------------------------------------------------------------------------------- RMSNorm (+quant)
// QUANT: 0 none (bf16 out), 1 NVFP4 (packed + tiled e4m3 scales + per-row fp32 scale), 2 MXFP8 (e4m3 + tiled e8m0)
template <int QUANT>
__global__ void rmsnorm_kernel(__nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ residual,
                               const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                               uint8_t* __restrict__ q_out, uint8_t* __restrict__ sf_out, float* __restrict__ row_scale,
                               int H, float eps, int zero_centered, int sf_col_tiles, int zero_src) {
  extern __shared__ __align__(16) uint8_t dyn[];
  __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(dyn);     // the (x + residual) row, then the normed row
  __shared__ float red[32];
  const int t = blockIdx.x;
  __nv_bfloat16* xr = x + (size_t)t * H;
  __nv_bfloat16* rr = residual ? residual + (size_t)t * H : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 u = *reinterpret_cast<const uint4*>(xr + i);
    if (zero_src) *reinterpret_cast<uint4*>(xr + i) = make_uint4(0, 0, 0, 0);   // hand the accumulation buffer back zeroed
    __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&u);
    if (rr) {
      uint4 ur = *reinterpret_cast<const uint4*>(rr + i);
      const __nv_bfloat16* er = reinterpret_cast<const __nv_bfloat16*>(&ur);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = __float2bfloat16(bf2f(e[j]) + bf2f(er[j]));
      *reinterpret_cast<uint4*>(rr + i) = u;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { float f = bf2f(e[j]); ss += f * f; }
    *reinterpret_cast<uint4*>(row + i) = u;
  }
  ss = block_reduce(ss, red, false);
  const float rstd = rsqrtf(ss / H + eps);
  float amax = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 u = *reinterpret_cast<uint4*>(row + i);
    uint4 uw = *reinterpret_cast<const uint4*>(w + i);
    __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&u);
    const __nv_bfloat16* ew = reinterpret_cast<const __nv_bfloat16*>(&uw);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float wf = bf2f(ew[j]) + (zero_centered ? 1.f : 0.f);
      e[j] = __float2bfloat16(bf2f(e[j]) * rstd * wf);
      amax = fmaxf(amax, fabsf(bf2f(e[j])));
    }
    if (QUANT == 0) *reinterpret_cast<uint4*>(out + (size_t)t * H + i) = u;
    else *reinterpret_cast<uint4*>(row + i) = u;
  }
  if (QUANT == 0) return;
  if (QUANT == 1) {
    amax = block_reduce(amax, red, true);
    const float g = fmaxf(amax / (6.f * 448.f), 1e-30f);
    if (threadIdx.x == 0) row_scale[t] = g;
    __syncthreads();
    for (int b = threadIdx.x; b < H / 16; b += blockDim.x) {
      float v[16];
      float bm = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) { v[j] = bf2f(row[b * 16 + j]); bm = fmaxf(bm, fabsf(v[j])); }
      const uint8_t sf = f2e4m3(bm / 6.f / g);
      const float denom = e4m32f(sf) * g;
      const float inv = denom > 0.f ? 1.f / denom : 0.f;
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) lo |= f2e2m1(denom > 0.f ? v[j] / denom : 0.f) << (4 * j);
#pragma unroll
      for (int j = 0; j < 8; ++j) hi |= f2e2m1(denom > 0.f ? v[8 + j] / denom : 0.f) << (4 * j);
      (void)inv;
      *reinterpret_cast<uint2*>(q_out + (size_t)t * (H / 2) + b * 8) = make_uint2(lo, hi);
      sf_out[sf_offset(t, b, sf_col_tiles)] = sf;
    }
  } else {
    __syncthreads();
    for (int b = threadIdx.x; b < H / 32; b += blockDim.x) {
      float v[32];
      float bm = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) { v[j] = bf2f(row[b * 32 + j]); bm = fmaxf(bm, fabsf(v[j])); }
      bm = fmaxf(bm, 1.17549435e-38f);
      int ex = (int)ceilf(log2f(bm / 448.f));
      ex = max(-127, min(127, ex));
      const float inv = exp2f((float)-ex);
      uint32_t pk[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        pk[j] = f2e4m3(v[4 * j] * inv) | (f2e4m3(v[4 * j + 1] * inv) << 8) | (f2e4m3(v[4 * j + 2] * inv) << 16) |
                (f2e4m3(v[4 * j + 3] * inv) << 24);
      uint4* dst = reinterpret_cast<uint4*>(q_out + (size_t)t * H + b * 32);
      dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
      sf_out[sf_offset(t, b, sf_col_tiles)] = (uint8_t)(ex + 127);
    }
  }
}

// ---------------------------------------------------------------------------------------------- SwiGLU (+quant)
// gu [T, 2I] = [gate | up];  MODE 0: out bf16 [T, I];  MODE 1: NVFP4;  MODE 2: MXFP8.  Optional plain-row input
// (gate_up == nullptr is invalid).  `src_is_act`: quantise `gu` itself ([T, I], no SwiGLU) — used for attention output.
template <int MODE>
__global__ void swiglu_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                              uint8_t* __restrict__ q_out, uint8_t* __restrict__ sf_out, float* __restrict__ row_scale,
                              int I, int src_is_act, int sf_col_tiles, const int* __restrict__ row_list) {
  extern __shared__ __align__(16) uint8_t dyn[];
  __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(dyn);
  __shared__ float red[32];
  // row_list (optional): the rows to process, one per CTA, -1 = none (routed expert rows in their padded row space)
  const int t = row_list ? row_list[blockIdx.x] : (int)blockIdx.x;
  if (t < 0) return;
  const __nv_bfloat16* g = gu + (size_t)t * (src_is_act ? I : 2 * I);
  const __nv_bfloat16* u = g + I;
  float amax = 0.f;
  for (int i = threadIdx.x * 8; i < I; i += blockDim.x * 8) {
    uint4 ug = *reinterpret_cast<const uint4*>(g + i);
    __nv_bfloat16* eg = reinterpret_cast<__nv_bfloat16*>(&ug);
    if (!src_is_act) {
      uint4 uu = *reinterpret_cast<const uint4*>(u + i);
      const __nv_bfloat16* eu = reinterpret_cast<const __nv_bfloat16*>(&uu);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float a = bf2f(eg[j]);
        eg[j] = __float2bfloat16(a / (1.f + __expf(-a)) * bf2f(eu[j]));
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(bf2f(eg[j])));
    if (MODE == 0) *reinterpret_cast<uint4*>(out + (size_t)t * I + i) = ug;
    else *reinterpret_cast<uint4*>(row + i) = ug;
  }
  if (MODE == 0) return;
  if (MODE == 1) {
    amax = block_reduce(amax, red, true);
    const float gs = fmaxf(amax / (6.f * 448.f), 1e-30f);
    if (threadIdx.x == 0) row_scale[t] = gs;
    __syncthreads();
    for (int b = threadIdx.x; b < I / 16; b += blockDim.x) {
      float v[16];
      float bm = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) { v[j] = bf2f(row[b * 16 + j]); bm = fmaxf(bm, fabsf(v[j])); }
      const uint8_t sf = f2e4m3(bm / 6.f / gs);
      const float denom = e4m32f(sf) * gs;
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) lo |= f2e2m1(denom > 0.f ? v[j] / denom : 0.f) << (4 * j);
#pragma unroll
      for (int j = 0; j < 8; ++j) hi |= f2e2m1(denom > 0.f ? v[8 + j] / denom : 0.f) << (4 * j);
      *reinterpret_cast<uint2*>(q_out + (size_t)t * (I / 2) + b * 8) = make_uint2(lo, hi);
      sf_out[sf_offset(t, b, sf_col_tiles)] = sf;
    }
  } else {
    __syncthreads();
    for (int b = threadIdx.x; b < I / 32; b += blockDim.x) {
      float v[32];
      float bm = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) { v[j] = bf2f(row[b * 32 + j]); bm = fmaxf(bm, fabsf(v[j])); }
      bm = fmaxf(bm, 1.17549435e-38f);
      int ex = (int)ceilf(log2f(bm / 448.f));
      ex = max(-127, min(127, ex));
      const float inv = exp2f((float)-ex);
      uint32_t pk[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        pk[j] = f2e4m3(v[4 * j] * inv) | (f2e4m3(v[4 * j + 1] * inv) << 8) | (f2e4m3(v[4 * j + 2] * inv) << 16) |
                (f2e4m3(v[4 * j + 3] * inv) << 24);
      uint4* dst = reinterpret_cast<uint4*>(q_out + (size_t)t * I + b * 32);
      dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
      sf_out[sf_offset(t, b, sf_col_tiles)] = (uint8_t)(ex + 127);
    }
  }
}

// ---------------------------------------------------------------------------------------------- register-resident rows
// Fast path of the two row kernels above for widths up to 6 chunks of 8 elements per thread: the row never touches
// shared memory, every load of a thread is issued before the first use, and the quantiser works on the registers
// (a 16-element NVFP4 block is two neighbouring threads, a 32-element MXFP8 block four).
__device__ __forceinline__ uint32_t pack_e2m1x8(const float (&v)[8], float inv) {
  uint32_t r;
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n"
      "}"
      : "=r"(r)
      : "f"(v[0] * inv), "f"(v[1] * inv), "f"(v[2] * inv), "f"(v[3] * inv), "f"(v[4] * inv), "f"(v[5] * inv), "f"(v[6] * inv),
        "f"(v[7] * inv));
  return r;
}
__device__ __forceinline__ uint32_t pack_e4m3x4_f(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// Quantise this thread's 8 elements [e0, e0+8) of row t.  Every lane of the warp must call it (shuffles); `valid` gates the stores.
template <int QUANT>
__device__ __forceinline__ void quant_store8(const uint4& packed, bool valid, int t, int e0, int W, float g, uint8_t* q_out,
                                             uint8_t* sf_out, int ct) {
  const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&packed);
  float v[8];
  float bm = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) { v[j] = valid ? bf2f(e[j]) : 0.f; bm = fmaxf(bm, fabsf(v[j])); }
  bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
  if (QUANT == 1) {
    const uint8_t sf = f2e4m3(bm / 6.f / g);
    const float denom = e4m32f(sf) * g;
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    const uint32_t codes = pack_e2m1x8(v, inv);
    if (valid) {
      *reinterpret_cast<uint32_t*>(q_out + (size_t)t * (W / 2) + e0 / 2) = codes;
      if ((e0 & 15) == 0) sf_out[sf_offset(t, e0 >> 4, ct)] = sf;
    }
  } else {
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
    bm = fmaxf(bm, 1.17549435e-38f);
    int ex = (int)ceilf(log2f(bm / 448.f));
    ex = max(-127, min(127, ex));
    const float inv = exp2f((float)-ex);
    if (valid) {
      *reinterpret_cast<uint2*>(q_out + (size_t)t * W + e0) =
          make_uint2(pack_e4m3x4_f(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv),
                     pack_e4m3x4_f(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv));
      if ((e0 & 31) == 0) sf_out[sf_offset(t, e0 >> 5, ct)] = (uint8_t)(ex + 127);
    }
  }
}

template <int QUANT, int CH>
__global__ void __launch_bounds__(512) rmsnorm_reg_kernel(__nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ residual,
                                                            const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                                            uint8_t* __restrict__ q_out, uint8_t* __restrict__ sf_out,
                                                            float* __restrict__ row_scale, int H, float eps, int zero_centered,
                                                            int sf_col_tiles, int zero_src) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[32];
  const int t = blockIdx.x;
  __nv_bfloat16* xr = x + (size_t)t * H;
  __nv_bfloat16* rr = residual ? residual + (size_t)t * H : nullptr;
  uint4 u[CH], ur[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 8;
    u[c] = ur[c] = make_uint4(0, 0, 0, 0);
    if (i < H) {
      u[c] = *reinterpret_cast<const uint4*>(xr + i);
      if (rr) ur[c] = *reinterpret_cast<const uint4*>(rr + i);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 8;
    __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&u[c]);
    if (i < H) {
      if (zero_src) *reinterpret_cast<uint4*>(xr + i) = make_uint4(0, 0, 0, 0);
      if (rr) {
        const __nv_bfloat16* er = reinterpret_cast<const __nv_bfloat16*>(&ur[c]);
#pragma unroll
        for (int j = 0; j < 8; ++j) e[j] = __float2bfloat16(bf2f(e[j]) + bf2f(er[j]));
        *reinterpret_cast<uint4*>(rr + i) = u[c];
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { const float f = bf2f(e[j]); ss += f * f; }
  }
  ss = block_reduce(ss, red, false);
  const float rstd = rsqrtf(ss / H + eps);
  float amax = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 8;
    __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&u[c]);
    const uint4 uw = i < H ? *reinterpret_cast<const uint4*>(w + i) : make_uint4(0, 0, 0, 0);   // the weight row stays in L1/L2
    const __nv_bfloat16* ew = reinterpret_cast<const __nv_bfloat16*>(&uw);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float wf = bf2f(ew[j]) + (zero_centered ? 1.f : 0.f);
      e[j] = __float2bfloat16(bf2f(e[j]) * rstd * wf);
      amax = fmaxf(amax, fabsf(bf2f(e[j])));
    }
    if (QUANT == 0 && i < H) *reinterpret_cast<uint4*>(out + (size_t)t * H + i) = u[c];
  }
  if (QUANT == 0) return;
  float g = 1.f;
  if (QUANT == 1) {
    amax = block_reduce(amax, red, true);
    g = fmaxf(amax / (6.f * 448.f), 1e-30f);
    if (threadIdx.x == 0) row_scale[t] = g;
  }
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 8;
    quant_store8<QUANT>(u[c], i < H, t, i, H, g, q_out, sf_out, sf_col_tiles);
  }
}

template <int MODE, int CH>
__global__ void __launch_bounds__(512) swiglu_reg_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                                           uint8_t* __restrict__ q_out, uint8_t* __restrict__ sf_out,
                                                           float* __restrict__ row_scale, int I, int src_is_act, int sf_col_tiles,
                                                           const int* __restrict__ row_list) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[32];
  // row_list (optional): the rows to process, one per CTA, -1 = none (routed expert rows in their padded row space)
  const int t = row_list ? row_list[blockIdx.x] : (int)blockIdx.x;
  if (t < 0) return;
  const __nv_bfloat16* g = gu + (size_t)t * (src_is_act ? I : 2 * I);
  const __nv_bfloat16* up = g + I;
  uint4 a[CH], b[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 8;
    a[c] = b[c] = make_uint4(0, 0, 0, 0);
    if (i < I) {
      a[c] = *reinterpret_cast<const uint4*>(g + i);
      if (!src_is_act) b[c] = *reinterpret_cast<const uint4*>(up + i);
    }
  }
  float amax = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 8;
    __nv_bfloat16* eg = reinterpret_cast<__nv_bfloat16*>(&a[c]);
    const __nv_bfloat16* eu = reinterpret_cast<const __nv_bfloat16*>(&b[c]);
    if (!src_is_act) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float x = bf2f(eg[j]);
        eg[j] = __float2bfloat16(x / (1.f + __expf(-x)) * bf2f(eu[j]));
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(bf2f(eg[j])));
    if (MODE == 0 && i < I) *reinterpret_cast<uint4*>(out + (size_t)t * I + i) = a[c];
  }
  if (MODE == 0) return;
  float gs = 1.f;
  if (MODE == 1) {
    amax = block_reduce(amax, red, true);
    gs = fmaxf(amax / (6.f * 448.f), 1e-30f);
    if (threadIdx.x == 0) row_scale[t] = gs;
  }
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 8;
    quant_store8<MODE>(a[c], i < I, t, i, I, gs, q_out, sf_out, sf_col_tiles);
  }
}

// Rows of at most 1024 activations (expert intermediates): several rows per CTA, `tpr` threads each (a multiple of 32, so
// a warp never spans two rows), instead of one mostly idle 256-thread CTA per row.  Entry r of the launch handles row
// row_list[r] (or r); -1 and entries beyond n_rows are skipped.
template <int MODE>
__global__ void __launch_bounds__(256) swiglu_rows_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                                            uint8_t* __restrict__ q_out, uint8_t* __restrict__ sf_out,
                                                            float* __restrict__ row_scale, int I, int src_is_act, int sf_col_tiles,
                                                            const int* __restrict__ row_list, int n_rows, int tpr) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[8];
  const int sub = threadIdx.x / tpr, in_row = threadIdx.x - sub * tpr;
  const int r = blockIdx.x * (blockDim.x / tpr) + sub;
  int t = -1;
  if (r < n_rows) t = row_list ? row_list[r] : r;
  const bool live = t >= 0;
  const int i = in_row * 8;
  const bool valid = live && i < I;
  uint4 a = make_uint4(0, 0, 0, 0), b = a;
  if (valid) {
    const __nv_bfloat16* g = gu + (size_t)t * (src_is_act ? I : 2 * I);
    a = *reinterpret_cast<const uint4*>(g + i);
    if (!src_is_act) b = *reinterpret_cast<const uint4*>(g + I + i);
  }
  __nv_bfloat16* eg = reinterpret_cast<__nv_bfloat16*>(&a);
  const __nv_bfloat16* eu = reinterpret_cast<const __nv_bfloat16*>(&b);
  float amax = 0.f;
  if (!src_is_act) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float x = bf2f(eg[j]);
      eg[j] = __float2bfloat16(x / (1.f + __expf(-x)) * bf2f(eu[j]));
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(bf2f(eg[j])));
  if (MODE == 0) {
    if (valid) *reinterpret_cast<uint4*>(out + (size_t)t * I + i) = a;
    return;
  }
  float gs = 1.f;
  if (MODE == 1) {
    // the row's largest magnitude: over the warp, then over the row's warps
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    float m = 0.f;
    for (int k = 0; k < (tpr >> 5); ++k) m = fmaxf(m, red[((sub * tpr) >> 5) + k]);
    gs = fmaxf(m / (6.f * 448.f), 1e-30f);
    if (live && in_row == 0) row_scale[t] = gs;
  }
  quant_store8<MODE>(a, valid, live ? t : 0, i, I, gs, q_out, sf_out, sf_col_tiles);
}

// ---------------------------------------------------------------------------------------------- attention prep
// One CTA per token; its warps walk the token's heads.  Heads 0..Hq-1 are query heads, then Hkv key heads, then Hkv
// value heads.  qkv row layout: [q heads (x2 when gated: q | gate per head)] [k heads] [v heads].  The rotary
// sine/cosine pairs of the token are computed once into shared memory and reused by every q and k head.
template <int D>
__global__ void __launch_bounds__(512) attn_prep_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                                 __nv_bfloat16* __restrict__ gate_out, uint8_t* __restrict__ kv_pool,
                                 const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                                 const float* __restrict__ inv_freq, const __nv_bfloat16* __restrict__ q_norm_w,
                                 const __nv_bfloat16* __restrict__ k_norm_w, int T, int Hq, int Hkv, int rot_dim,
                                 float eps, float rope_scale, int gated, int zero_centered, float k_scale_inv,
                                 float v_scale_inv, long long page_stride, long long head_stride, int rotate,
                                 long long pos_stride, int mrope0, int mrope1) {
  pdl_trigger();
  pdl_wait();
  constexpr int VPL = D / 32;
  __shared__ float2 cs[D / 2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const int heads = Hq + 2 * Hkv;
  const int half = rot_dim / 2;
  {
    // M-RoPE (pos_stride > 0): positions is [3, T]; frequency i follows the temporal stream below mrope0, the height stream
    // below mrope1, the width stream above (reference: attn_prep_kernel<MROPE>, kernels/src/cuda/ops_basic.cu:102)
    const float p0 = (float)positions[t];
    const float p1 = pos_stride > 0 ? (float)positions[pos_stride + t] : p0;
    const float p2 = pos_stride > 0 ? (float)positions[2 * pos_stride + t] : p0;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float pos = pos_stride > 0 ? (i < mrope0 ? p0 : (i < mrope1 ? p1 : p2)) : p0;
      float s, c;
      sincosf(pos * inv_freq[i], &s, &c);
      cs[i] = make_float2(c * rope_scale, s * rope_scale);
    }
  }
  __syncthreads();
  const int qw = Hq * D * (gated ? 2 : 1);
  const size_t row_w = (size_t)qw + 2 * (size_t)Hkv * D;
  const __nv_bfloat16* row = qkv + t * row_w;
  const int lanes_half = half / VPL;          // partner lane distance (power of two)
  const int slot = slot_mapping[t];
  float nwq[VPL], nwk[VPL];
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    nwq[j] = q_norm_w ? bf2f(q_norm_w[lane * VPL + j]) + (zero_centered ? 1.f : 0.f) : 0.f;
    nwk[j] = k_norm_w ? bf2f(k_norm_w[lane * VPL + j]) + (zero_centered ? 1.f : 0.f) : 0.f;
  }
  for (int h = warp; h < heads; h += nwarps) {
    const __nv_bfloat16* src;
    int kind;  // 0 q, 1 k, 2 v
    if (h < Hq) { kind = 0; src = row + (size_t)h * D * (gated ? 2 : 1); }
    else if (h < Hq + Hkv) { kind = 1; src = row + qw + (size_t)(h - Hq) * D; }
    else { kind = 2; src = row + qw + (size_t)Hkv * D + (size_t)(h - Hq - Hkv) * D; }
    if (kind != 0 && slot < 0) continue;
    __align__(16) __nv_bfloat16 raw[VPL];
    if constexpr (VPL == 4) *reinterpret_cast<uint2*>(raw) = *reinterpret_cast<const uint2*>(src + lane * 4);
    else if constexpr (VPL == 8) *reinterpret_cast<uint4*>(raw) = *reinterpret_cast<const uint4*>(src + lane * 8);
    else *reinterpret_cast<uint32_t*>(raw) = *reinterpret_cast<const uint32_t*>(src + lane * 2);
    float v[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) v[j] = bf2f(raw[j]);
    if (kind == 0 && gated) {
      __nv_bfloat16* gdst = gate_out + ((size_t)t * Hq + h) * D + lane * VPL;
      if constexpr (VPL == 4) *reinterpret_cast<uint2*>(gdst) = *reinterpret_cast<const uint2*>(src + D + lane * 4);
      else if constexpr (VPL == 8) *reinterpret_cast<uint4*>(gdst) = *reinterpret_cast<const uint4*>(src + D + lane * 8);
      else *reinterpret_cast<uint32_t*>(gdst) = *reinterpret_cast<const uint32_t*>(src + D + lane * 2);
    }
    if (kind < 2) {
      if (kind == 0 ? q_norm_w != nullptr : k_norm_w != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < VPL; ++j) ss += v[j] * v[j];
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / D + eps);
#pragma unroll
        for (int j = 0; j < VPL; ++j) v[j] = bf2f(__float2bfloat16(v[j] * rstd * (kind == 0 ? nwq[j] : nwk[j])));
      }
      // NeoX rotary over the first rot_dim dims: pairs (i, i + half)
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const int i = lane * VPL + j;
        const float other = __shfl_xor_sync(0xffffffffu, v[j], lanes_half);
        if (i < rot_dim) {
          const float2 c = cs[i < half ? i : i - half];
          v[j] = i < half ? v[j] * c.x - other * c.y : v[j] * c.x + other * c.y;
        }
      }
      // Optional randomised Hadamard rotation of q and k (the same orthogonal map on both keeps q.k; it spreads
      // outliers over the head before the key is rounded to e4m3): sign flip by a fixed hash of the element index,
      // then a Walsh-Hadamard transform over the D elements the warp holds, scaled by 1/sqrt(D).
      if (rotate) {
#pragma unroll
        for (int j = 0; j < VPL; ++j)
          if (((uint32_t)(lane * VPL + j) * 2654435761u >> 15) & 1u) v[j] = -v[j];
#pragma unroll
        for (int st = 1; st < VPL; st <<= 1) {
#pragma unroll
          for (int j = 0; j < VPL; ++j)
            if (!(j & st)) { const float a = v[j], b = v[j | st]; v[j] = a + b; v[j | st] = a - b; }
        }
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
          for (int j = 0; j < VPL; ++j) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], m);
            v[j] = (lane & m) ? other - v[j] : v[j] + other;
          }
        }
        const float sc = rsqrtf((float)D);
#pragma unroll
        for (int j = 0; j < VPL; ++j) v[j] *= sc;
      }
    }
    if (kind == 0) {
      __align__(16) __nv_bfloat16 o[VPL];
#pragma unroll
      for (int j = 0; j < VPL; ++j) o[j] = __float2bfloat16(v[j]);
      __nv_bfloat16* dst = q_out + ((size_t)t * Hq + h) * D + lane * VPL;
      if constexpr (VPL == 4) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(o);
      else if constexpr (VPL == 8) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
      else *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(o);
      continue;
    }
    const int page = slot >> 4, tp = slot & 15;
    const int kh = kind == 1 ? h - Hq : h - Hq - Hkv;
    uint8_t* blk = kv_pool + (size_t)page * page_stride + (size_t)kh * head_stride;
    if (kind == 1) {
      // the lane's VPL dims are consecutive bytes of one 16-byte core-matrix row
      __align__(8) uint8_t b[VPL];
#pragma unroll
      for (int j = 0; j < VPL; ++j) b[j] = f2e4m3(bf2f(__float2bfloat16(v[j])) * k_scale_inv);
      const int i0 = lane * VPL;
      uint8_t* dst = blk + (tp >> 3) * 8 * D + (i0 >> 4) * 128 + (tp & 7) * 16 + (i0 & 15);
      if constexpr (VPL == 4) *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(b);
      else if constexpr (VPL == 8) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(b);
      else *reinterpret_cast<uint16_t*>(dst) = *reinterpret_cast<const uint16_t*>(b);
    } else {
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const int i = lane * VPL + j;
        blk[16 * D + i * 16 + tp] = f2e4m3(v[j] * v_scale_inv);
      }
    }
  }
}

__global__ void mul_sigmoid_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] = __float2bfloat16(bf2f(x[i]) / (1.f + __expf(-bf2f(gate[i]))));
}
__global__ void add_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* out, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(bf2f(a[i]) + bf2f(b[i]));
}
// out[t, :] = a[t, :] + b[t, :] * bf16(sigmoid(gate_logit[t]))
__global__ void add_sigmoid_scaled_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, const __nv_bfloat16* gl,
                                          __nv_bfloat16* out, int H) {
  const int t = blockIdx.x;
  const float s = bf2f(__float2bfloat16(1.f / (1.f + __expf(-bf2f(gl[t])))));
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[(size_t)t * H + i] = __float2bfloat16(bf2f(a[(size_t)t * H + i]) + bf2f(b[(size_t)t * H + i]) * s);
}
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ rows,
                                   __nv_bfloat16* __restrict__ out, int H) {
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)rows[blockIdx.x] * H);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// argmax over fp32 rows, lowest index wins ties; writes int64 ids (and optionally the max value)
__global__ void argmax_kernel(const float* __restrict__ logits, long long* __restrict__ out, float* __restrict__ out_val,
                              int V, long long ld, int index_offset) {
  pdl_trigger();
  pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  const float* row = logits + (size_t)blockIdx.x * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float x = row[i];
    if (x > best || (x == best && i < bi)) { best = x; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) {
      out[blockIdx.x] = (long long)(bi == 0x7fffffff ? 0 : bi) + index_offset;
      if (out_val) out_val[blockIdx.x] = best;
    }
  }
}

// Reduce the per-tile (value, column) pairs of the greedy head: one warp per row, ties to the lower column.
__global__ void argmax_parts_kernel(const float* __restrict__ val, const int* __restrict__ idx, int tiles, int M,
                                    long long* __restrict__ out, float* __restrict__ out_val, int index_offset) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int t = lane; t < tiles; t += 32) {
    const float v = val[(size_t)t * M + row];
    const int i = idx[(size_t)t * M + row];
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if (lane == 0) {
    out[row] = (long long)bi + index_offset;
    if (out_val) out_val[row] = bv;
  }
}

}  // namespace blz

using namespace blz;
typedef __nv_bfloat16 bf16;

static void configure_once() {
  static bool attr = false;
  if (attr) return;
  cudaFuncSetAttribute(swiglu_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  cudaFuncSetAttribute(swiglu_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  cudaFuncSetAttribute(rmsnorm_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  cudaFuncSetAttribute(rmsnorm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  cudaFuncSetAttribute(rmsnorm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  attr = true;
}

// threads and chunks per thread of the register-resident row kernels; chunks == 0: width not covered
// Few rows (a decode step) cannot fill the GPU with 256-thread CTAs: they get up to 512 threads per row, which shortens
// each row's dependency chain; BLAZE_ROW_THREADS=256 restores one shape for all.
static inline void reg_shape(int W, int T, int* threads, int* chunks) {
  static int wide_rows = -1;
  if (wide_rows < 0) { const char* e = getenv("BLAZE_ROW_THREADS"); wide_rows = (e && atoi(e) == 256) ? 0 : 1; }
  *threads = W <= 12288 ? 256 : 512;
  if (wide_rows && T <= 1024 && W >= 4096) *threads = 512;
  const int ch = (W + *threads * 8 - 1) / (*threads * 8);
  *chunks = (W % 32 == 0 && ch <= 6) ? ch : 0;
}

#define BLZ_CH_SWITCH(ch, CALL)                                                                    \
  switch (ch) {                                                                                     \
    case 1: CALL(1); break; case 2: CALL(2); break; case 3: CALL(3); break; case 4: CALL(4); break; \
    case 5: CALL(5); break; default: CALL(6); break;                                                \
  }

static inline int norm_threads(int H) {
  int t = H / 8;
  t = (t + 31) / 32 * 32;
  return t < 32 ? 32 : (t > 1024 ? 1024 : t);
}

BLZ_API int blz_embed(const void* table, const int* tokens, void* out, int T, int H, int vocab, cudaStream_t s) {
  if (H % 8) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  launch_pdl(embed_kernel, dim3(T), dim3(256), 0, s, (const bf16*)table, tokens, (bf16*)out, H, vocab);
  return (int)cudaGetLastError();
}

// quant: 0 → bf16 `out`; 1 → NVFP4 (q_out [T, H/2], sf_out tiled, row_scale [T]); 2 → MXFP8 (q_out [T, H], sf_out tiled)
BLZ_API int blz_rmsnorm(void* x, void* residual, const void* w, void* out, void* q_out, void* sf_out,
                        float* row_scale, int T, int H, float eps, int zero_centered, int quant, int zero_src, cudaStream_t s) {
  if (H % 32 || T < 0) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  configure_once();
  const int thr = norm_threads(H);
  const size_t sm = (size_t)H * 2;
  const int ct = quant == 1 ? (H + 63) / 64 : (H + 127) / 128;
  int rt, ch;
  reg_shape(H, T, &rt, &ch);
  if (ch) {
#define BLZ_RN(C)                                                                                                              \
  if (quant == 0) launch_pdl(rmsnorm_reg_kernel<0, C>, dim3(T), dim3(rt), 0, s, (bf16*)x, (bf16*)residual, (const bf16*)w, (bf16*)out, (uint8_t*)nullptr, (uint8_t*)nullptr, (float*)nullptr, H, eps, zero_centered, 0, zero_src); \
  else if (quant == 1) launch_pdl(rmsnorm_reg_kernel<1, C>, dim3(T), dim3(rt), 0, s, (bf16*)x, (bf16*)residual, (const bf16*)w, (bf16*)nullptr, (uint8_t*)q_out, (uint8_t*)sf_out, row_scale, H, eps, zero_centered, ct, zero_src); \
  else launch_pdl(rmsnorm_reg_kernel<2, C>, dim3(T), dim3(rt), 0, s, (bf16*)x, (bf16*)residual, (const bf16*)w, (bf16*)nullptr, (uint8_t*)q_out, (uint8_t*)sf_out, row_scale, H, eps, zero_centered, ct, zero_src)
    BLZ_CH_SWITCH(ch, BLZ_RN)
#undef BLZ_RN
    return (int)cudaGetLastError();
  }
  if (quant == 0)
    rmsnorm_kernel<0><<<T, thr, sm, s>>>((bf16*)x, (bf16*)residual, (const bf16*)w, (bf16*)out, nullptr, nullptr, nullptr, H, eps, zero_centered, 0, zero_src);
  else if (quant == 1)
    rmsnorm_kernel<1><<<T, thr, sm, s>>>((bf16*)x, (bf16*)residual, (const bf16*)w, nullptr, (uint8_t*)q_out, (uint8_t*)sf_out, row_scale, H, eps, zero_centered, ct, zero_src);
  else
    rmsnorm_kernel<2><<<T, thr, sm, s>>>((bf16*)x, (bf16*)residual, (const bf16*)w, nullptr, (uint8_t*)q_out, (uint8_t*)sf_out, row_scale, H, eps, zero_centered, ct, zero_src);
  return (int)cudaGetLastError();
}

// mode as `quant` above; src_is_act = 1 quantises the [T, I] input as is (no SwiGLU).  blz_swiglu_live: T entries of row_list
// name the rows to process (-1 = skip): the live rows of the routed experts' padded row space.
static int swiglu_impl(const void* gu, void* out, void* q_out, void* sf_out, float* row_scale, int T, int I,
                       int mode, int src_is_act, const int* row_list, cudaStream_t s);
BLZ_API int blz_swiglu(const void* gu, void* out, void* q_out, void* sf_out, float* row_scale, int T, int I,
                       int mode, int src_is_act, cudaStream_t s) {
  return swiglu_impl(gu, out, q_out, sf_out, row_scale, T, I, mode, src_is_act, nullptr, s);
}
BLZ_API int blz_swiglu_live(const void* gu, void* out, void* q_out, void* sf_out, float* row_scale, int T, int I,
                            int mode, int src_is_act, const int* row_list, cudaStream_t s) {
  return swiglu_impl(gu, out, q_out, sf_out, row_scale, T, I, mode, src_is_act, row_list, s);
}
static int swiglu_impl(const void* gu, void* out, void* q_out, void* sf_out, float* row_scale, int T, int I,
                       int mode, int src_is_act, const int* row_list, cudaStream_t s) {
  if (I % 32 || T < 0) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  const int thr = norm_threads(I);
  const size_t sm = (size_t)I * 2;
  const int ct = mode == 1 ? (I + 63) / 64 : (I + 127) / 128;
  configure_once();
  {
    const int tpr = (I / 8 + 31) / 32 * 32, rows_per = tpr <= 128 ? 256 / tpr : 1;
    if (I <= 1024 && rows_per >= 2) {
      const dim3 grid((T + rows_per - 1) / rows_per), block(rows_per * tpr);
      if (mode == 0) launch_pdl(swiglu_rows_kernel<0>, grid, block, 0, s, (const bf16*)gu, (bf16*)out, (uint8_t*)nullptr, (uint8_t*)nullptr, (float*)nullptr, I, src_is_act, 0, row_list, T, tpr);
      else if (mode == 1) launch_pdl(swiglu_rows_kernel<1>, grid, block, 0, s, (const bf16*)gu, (bf16*)nullptr, (uint8_t*)q_out, (uint8_t*)sf_out, row_scale, I, src_is_act, ct, row_list, T, tpr);
      else launch_pdl(swiglu_rows_kernel<2>, grid, block, 0, s, (const bf16*)gu, (bf16*)nullptr, (uint8_t*)q_out, (uint8_t*)sf_out, row_scale, I, src_is_act, ct, row_list, T, tpr);
      return (int)cudaGetLastError();
    }
  }
  int rt, ch;
  reg_shape(I, T, &rt, &ch);
  if (ch) {
#define BLZ_SW(C)                                                                                                              \
  if (mode == 0) launch_pdl(swiglu_reg_kernel<0, C>, dim3(T), dim3(rt), 0, s, (const bf16*)gu, (bf16*)out, (uint8_t*)nullptr, (uint8_t*)nullptr, (float*)nullptr, I, src_is_act, 0, row_list); \
  else if (mode == 1) launch_pdl(swiglu_reg_kernel<1, C>, dim3(T), dim3(rt), 0, s, (const bf16*)gu, (bf16*)nullptr, (uint8_t*)q_out, (uint8_t*)sf_out, row_scale, I, src_is_act, ct, row_list); \
  else launch_pdl(swiglu_reg_kernel<2, C>, dim3(T), dim3(rt), 0, s, (const bf16*)gu, (bf16*)nullptr, (uint8_t*)q_out, (uint8_t*)sf_out, row_scale, I, src_is_act, ct, row_list)
    BLZ_CH_SWITCH(ch, BLZ_SW)
#undef BLZ_SW
    return (int)cudaGetLastError();
  }
  if (mode == 0) swiglu_kernel<0><<<T, thr, 0, s>>>((const bf16*)gu, (bf16*)out, nullptr, nullptr, nullptr, I, src_is_act, 0, row_list);
  else if (mode == 1) swiglu_kernel<1><<<T, thr, sm, s>>>((const bf16*)gu, nullptr, (uint8_t*)q_out, (uint8_t*)sf_out, row_scale, I, src_is_act, ct, row_list);
  else swiglu_kernel<2><<<T, thr, sm, s>>>((const bf16*)gu, nullptr, (uint8_t*)q_out, (uint8_t*)sf_out, row_scale, I, src_is_act, ct, row_list);
  return (int)cudaGetLastError();
}

BLZ_API int blz_attn_prep(const void* qkv, void* q_out, void* gate_out, void* kv_pool, const int* positions,
                          const int* slot_mapping, const float* inv_freq, const void* q_norm_w, const void* k_norm_w,
                          int T, int Hq, int Hkv, int D, int rot_dim, float eps, float rope_scale, int gated,
                          int zero_centered, float k_scale, float v_scale, long long page_stride, long long head_stride,
                          int rotate, long long pos_stride, int mrope0, int mrope1, cudaStream_t s) {
  if (T == 0) return 0;
  const int half = rot_dim / 2, vpl = D / 32;
  if ((D != 64 && D != 128 && D != 256) || rot_dim > D || half % vpl || ((half / vpl) & (half / vpl - 1)) || half / vpl > 16)
    return (int)cudaErrorInvalidValue;
  // decode-sized steps: more warps per token shorten the per-token chain (launch bound of the kernel: 512 threads)
  int wpb = (Hq + 2 * Hkv) >= 8 ? 8 : (Hq + 2 * Hkv);
  { static int wide = -1; if (wide < 0) { const char* e = getenv("BLAZE_ROW_THREADS"); wide = (e && atoi(e) == 256) ? 0 : 1; }
    if (wide && T <= 1024 && (Hq + 2 * Hkv) >= 16) wpb = 16; }
  const int grid = T;
#define BLZ_PREP(DD)                                                                                                 \
  launch_pdl(attn_prep_kernel<DD>, dim3(grid), dim3(wpb * 32), 0, s, (const bf16*)qkv, (bf16*)q_out, (bf16*)gate_out,  \
             (uint8_t*)kv_pool, positions, slot_mapping, inv_freq, (const bf16*)q_norm_w, (const bf16*)k_norm_w, T, Hq, \
             Hkv, rot_dim, eps, rope_scale, gated, zero_centered, 1.f / k_scale, 1.f / v_scale,                         \
             page_stride > 0 ? page_stride : (long long)Hkv * 2 * 16 * D, head_stride > 0 ? head_stride : (long long)2 * 16 * D, \
             rotate, pos_stride, mrope0, mrope1)
  if (D == 64) BLZ_PREP(64); else if (D == 128) BLZ_PREP(128); else BLZ_PREP(256);
#undef BLZ_PREP
  return (int)cudaGetLastError();
}

namespace blz {
// Copy the K and V rows of KV slot src[m] to slot dst[m] in every KV head of one layer's pool (page layout of the
// attention kernels: K as 8-row x 16-byte core matrices, V transposed).  Used after a draft tree has been verified: the
// accepted path's rows move down to consecutive positions.  Moves seg[i] .. seg[i+1]-1 belong to sequence i and run in
// list order inside one CTA (a later move may overwrite the source of an earlier one: row 2 -> 1, then row 5 -> 2);
// different sequences never share a slot.  Reference: blz_move_rows (kernels/src/cuda/tree.cu :142).
__global__ void kv_move_rows_kernel(uint8_t* pool, const int* __restrict__ src, const int* __restrict__ dst,
                                    const int* __restrict__ seg, int D, long long page_stride, long long head_stride) {
  for (int m = seg[blockIdx.x]; m < seg[blockIdx.x + 1]; ++m) {
    const int s = src[m], d = dst[m];
    if (s != d && s >= 0 && d >= 0) {
      const uint8_t* sb = pool + (size_t)(s >> 4) * page_stride + (size_t)blockIdx.y * head_stride;
      uint8_t* db = pool + (size_t)(d >> 4) * page_stride + (size_t)blockIdx.y * head_stride;
      const int st = s & 15, dt = d & 15;
      for (int c = threadIdx.x; c < D / 16; c += blockDim.x)
        *reinterpret_cast<uint4*>(db + (dt >> 3) * 8 * D + c * 128 + (dt & 7) * 16) =
            *reinterpret_cast<const uint4*>(sb + (st >> 3) * 8 * D + c * 128 + (st & 7) * 16);
      for (int i = threadIdx.x; i < D; i += blockDim.x) db[16 * D + i * 16 + dt] = sb[16 * D + i * 16 + st];
    }
    __syncthreads();
  }
}

}  // namespace blz
BLZ_API int blz_kv_move_rows(void* pool, const int* src, const int* dst, const int* seg, int num_seqs, int Hkv, int D,
                             long long page_stride, long long head_stride, cudaStream_t s) {
  if (num_seqs <= 0) return 0;
  if (D % 16 || Hkv <= 0 || page_stride <= 0 || head_stride <= 0 || page_stride % 16 || head_stride % 16)
    return (int)cudaErrorInvalidValue;
  blz::kv_move_rows_kernel<<<dim3(num_seqs, Hkv), 128, 0, s>>>((uint8_t*)pool, src, dst, seg, D, page_stride, head_stride);
  return (int)cudaGetLastError();
}

BLZ_API int blz_mul_sigmoid(void* x, const void* gate, long long n, cudaStream_t s) {
  if (n == 0) return 0;
  mul_sigmoid_kernel<<<(int)((n + 1023) / 1024 > 4096 ? 4096 : (n + 1023) / 1024), 256, 0, s>>>((bf16*)x, (const bf16*)gate, (size_t)n);
  return (int)cudaGetLastError();
}
BLZ_API int blz_add(const void* a, const void* b, void* out, long long n, cudaStream_t s) {
  if (n == 0) return 0;
  add_kernel<<<(int)((n + 1023) / 1024 > 4096 ? 4096 : (n + 1023) / 1024), 256, 0, s>>>((const bf16*)a, (const bf16*)b, (bf16*)out, (size_t)n);
  return (int)cudaGetLastError();
}
BLZ_API int blz_add_sigmoid_scaled(const void* a, const void* b, const void* gl, void* out, int T, int H, cudaStream_t s) {
  if (T == 0) return 0;
  add_sigmoid_scaled_kernel<<<T, 256, 0, s>>>((const bf16*)a, (const bf16*)b, (const bf16*)gl, (bf16*)out, H);
  return (int)cudaGetLastError();
}
BLZ_API int blz_gather_rows(const void* x, const int* rows, void* out, int R, int H, cudaStream_t s) {
  if (R == 0) return 0;
  if (H % 8) return (int)cudaErrorInvalidValue;
  gather_rows_kernel<<<R, 256, 0, s>>>((const bf16*)x, rows, (bf16*)out, H);
  return (int)cudaGetLastError();
}
BLZ_API int blz_argmax(const float* logits, long long* out, float* out_val, int R, int V, long long ld, int index_offset,
                       cudaStream_t s) {
  if (R == 0) return 0;
  launch_pdl(argmax_kernel, dim3(R), dim3(1024), 0, s, logits, out, out_val, V, ld, index_offset);
  return (int)cudaGetLastError();
}

BLZ_API int blz_argmax_parts(const float* val, const int* idx, int tiles, int M, long long* out, float* out_val, int index_offset,
                             cudaStream_t s) {
  if (M <= 0 || tiles <= 0) return 0;
  return (int)launch_pdl(argmax_parts_kernel, dim3((M + 7) / 8), dim3(256), 0, s, val, idx, tiles, M, out, out_val, index_offset);
}
