// Collectives over NVLink peer memory, issued from inside the kernels (no library call on the hot path):
//
//   * all-reduce of a bf16 buffer that lives in symmetric memory: every rank reduces 1/world of the rows and
//     broadcasts its slice — through the NVSwitch (`multimem.ld_reduce` / `multimem.st`) when a multicast mapping
//     exists, else through plain peer loads / stores in rank order (identical bits on every rank);
//   * the same reduction fused with the residual add and the next RMSNorm, optionally quantising the normed rows
//     to NVFP4 / MXFP8 for the following GEMM, so that what crosses NVLink on the way back is the 4/8-bit
//     activation, and the residual stream stays sharded by rows (sequence-parallel between the two collectives).
//
// Rank synchronisation is a flag barrier in symmetric memory: release stores to the peers' pads, acquire loads on the
// own pad, a monotonically increasing epoch kept in device memory (so captured CUDA graphs replay correctly), and a
// bounded spin that records an error in the status word instead of hanging.
//
// Reference counterparts: kernels/src/cuda/host_allreduce.cu — host_ar_kernel :171 (sums through pinned host slots
// in rank order), host_ar_rmsnorm_kernel :280 (all-reduce + residual + RMSNorm in one kernel), wait_for :105 (300 s
// spin then __trap); crates/blaze/src/model.rs reduce_norm :2555.
#include "blaze/host.h"
#include "blaze/sm100.cuh"

namespace blz {

static constexpr int kMaxWorld = 8;
static constexpr int kMaxBlocks = 512;

struct CommParams {
  void* peer_in[kMaxWorld];       // partial sums of every rank (symmetric buffer A)
  void* peer_out[kMaxWorld];      // result buffer of every rank (symmetric buffer B; may equal A)
  void* peer_sf[kMaxWorld];       // scale-factor result buffer of every rank
  void* peer_rs[kMaxWorld];       // per-row scale result buffer of every rank
  uint32_t* peer_pad[kMaxWorld];  // flag pads, [kMaxBlocks][kMaxWorld] uint32 each
  void* mc_in;                    // multicast views of the same buffers (null without NVLS)
  void* mc_out;
  void* mc_sf;
  void* mc_rs;
  uint32_t* epoch;                // [kMaxBlocks] local, monotonically increasing
  long long spin_limit;           // clock ticks a flag wait may take before it gives up
  int rank, world;
  int* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Block-level barrier across ranks: block b of every rank meets block b of every other rank.
// Every kernel uses two barrier epochs (entry = base + 1, exit = base + 2) and advances the stored epoch by two at
// entry, so a rank that gave up on a wait stays in step with its peers on the next kernel.
// Returns false (after recording kErrFlagTimeout) when a peer does not show up within the spin limit.
__device__ __forceinline__ bool rank_barrier(const CommParams& c, int* ok_smem, int phase) {
  __syncthreads();
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) {
    if (phase == 0) {
      s_epoch = c.epoch[blockIdx.x] + 1;
      c.epoch[blockIdx.x] = s_epoch + 1;
    } else {
      s_epoch = c.epoch[blockIdx.x];
    }
    *ok_smem = 1;
  }
  __threadfence_system();
  __syncthreads();
  const uint32_t e = s_epoch;
  if (threadIdx.x < c.world) {
    const int peer = threadIdx.x;
    st_release_sys(c.peer_pad[peer] + (size_t)blockIdx.x * kMaxWorld + c.rank, e);
    const uint32_t* mine = c.peer_pad[c.rank] + (size_t)blockIdx.x * kMaxWorld + peer;
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys(mine) - e) < 0) {
      if (clock64() - t0 > c.spin_limit) {
        atomicCAS(c.status, kOk, kErrFlagTimeout);
        *ok_smem = 0;
        break;
      }
    }
  }
  __syncthreads();
  return *ok_smem != 0;
}

// ------------------------------------------------------------------------------------------ multimem helpers
__device__ __forceinline__ uint4 mm_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void mm_st_v4(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void mm_st_v2(void* mc, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1,%2};" ::"l"(mc), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void mm_st_b32(void* mc, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

// sum of the 8 bf16 at byte offset `off` over all ranks, in rank order, fp32 accumulation
template <bool MC>
__device__ __forceinline__ void reduce8(const CommParams& c, size_t off, float (&f)[8]) {
  if constexpr (MC) {
    uint4 v = mm_ld_reduce_bf16x8(reinterpret_cast<const uint8_t*>(c.mc_in) + off);
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = bf2f(e[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = 0.f;
    for (int r = 0; r < c.world; ++r) {
      uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(c.peer_in[r]) + off);
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += bf2f(e[j]);
    }
  }
}
template <bool MC>
__device__ __forceinline__ void bcast16(const CommParams& c, void* const* peers, void* mc, size_t off, uint4 v) {
  if constexpr (MC) {
    mm_st_v4(reinterpret_cast<uint8_t*>(mc) + off, v);
  } else {
    for (int r = 0; r < c.world; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(peers[r]) + off) = v;
  }
}
template <bool MC>
__device__ __forceinline__ void bcast8(const CommParams& c, void* const* peers, void* mc, size_t off, uint2 v) {
  if constexpr (MC) {
    mm_st_v2(reinterpret_cast<uint8_t*>(mc) + off, v);
  } else {
    for (int r = 0; r < c.world; ++r) *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(peers[r]) + off) = v;
  }
}
template <bool MC>
__device__ __forceinline__ void bcast4(const CommParams& c, void* const* peers, void* mc, size_t off, uint32_t v) {
  if constexpr (MC) {
    mm_st_b32(reinterpret_cast<uint8_t*>(mc) + off, v);
  } else {
    for (int r = 0; r < c.world; ++r) *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(peers[r]) + off) = v;
  }
}

// ------------------------------------------------------------------------------------------ all-reduce
// n16 = number of 16-byte vectors.  Rank r reduces vectors [r*per, (r+1)*per) and broadcasts them into peer_out.
template <bool MC>
__global__ void __launch_bounds__(512) allreduce_kernel(CommParams c, size_t n16) {
  __shared__ int ok;
  if (!rank_barrier(c, &ok, 0)) return;
  const size_t per = (n16 + c.world - 1) / c.world;
  const size_t lo = (size_t)c.rank * per, hi = min(n16, lo + per);
  for (size_t i = lo + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += (size_t)gridDim.x * blockDim.x) {
    float f[8];
    reduce8<MC>(c, i * 16, f);
    uint4 o = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
    bcast16<MC>(c, c.peer_out, c.mc_out, i * 16, o);
  }
  rank_barrier(c, &ok, 1);
}

// ------------------------------------------------------------------------------------------ all-reduce + residual + RMSNorm (+quant)
__device__ __forceinline__ uint8_t f2e4m3_c(float x) { return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3); }
__device__ __forceinline__ float e4m32f_c(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
__device__ __forceinline__ uint32_t f2e2m1_c(float x) {
  const float a = fminf(fabsf(x), 6.0f);
  uint32_t k = (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.0f);
  return k | ((__float_as_uint(x) >> 31) << 3);
}
__device__ __forceinline__ float block_reduce_c(float v, float* sh, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float r = is_max ? -INFINITY : 0.f;
  for (int i = 0; i < nw; ++i) r = is_max ? fmaxf(r, sh[i]) : r + sh[i];
  return r;
}

// Rows are dealt to ranks in contiguous slices: rank r owns rows [r*rows_per, (r+1)*rows_per).  The owner sums the
// partial rows of all ranks, adds its slice of the residual stream (`residual` is LOCAL, [rows_per, H], updated in
// place), normalises, and broadcasts the result row: bf16 (QUANT 0), NVFP4 (1) or MXFP8 (2) into every rank's
// output buffers.  With `norm_w == nullptr` the summed (+ residual) row itself is broadcast (final layer).
template <bool MC, int QUANT>
__global__ void __launch_bounds__(1024) allreduce_norm_kernel(CommParams c, __nv_bfloat16* residual,
                                                              const __nv_bfloat16* __restrict__ norm_w, int T, int H,
                                                              int rows_per, float eps, int zero_centered, int sf_col_tiles) {
  extern __shared__ __align__(16) uint8_t dyn[];
  __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(dyn);
  __shared__ float red[32];
  __shared__ int ok;
  if (!rank_barrier(c, &ok, 0)) return;
  const int lo = c.rank * rows_per, hi = min(T, lo + rows_per);
  for (int t = lo + blockIdx.x; t < hi; t += gridDim.x) {
    __nv_bfloat16* rr = residual ? residual + (size_t)(t - lo) * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float f[8];
      reduce8<MC>(c, ((size_t)t * H + i) * 2, f);
      uint4 u;
      __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&u);
      if (rr) {
        uint4 ur = *reinterpret_cast<const uint4*>(rr + i);
        const __nv_bfloat16* er = reinterpret_cast<const __nv_bfloat16*>(&ur);
#pragma unroll
        for (int j = 0; j < 8; ++j) e[j] = __float2bfloat16(bf2f(__float2bfloat16(f[j])) + bf2f(er[j]));
        *reinterpret_cast<uint4*>(rr + i) = u;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) e[j] = __float2bfloat16(f[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float x = bf2f(e[j]); ss += x * x; }
      *reinterpret_cast<uint4*>(row + i) = u;
    }
    float rstd = 1.f;
    if (norm_w) {
      ss = block_reduce_c(ss, red, false);
      rstd = rsqrtf(ss / H + eps);
    } else {
      __syncthreads();
    }
    float amax = 0.f;
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      uint4 u = *reinterpret_cast<uint4*>(row + i);
      __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&u);
      if (norm_w) {
        uint4 uw = *reinterpret_cast<const uint4*>(norm_w + i);
        const __nv_bfloat16* ew = reinterpret_cast<const __nv_bfloat16*>(&uw);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          e[j] = __float2bfloat16(bf2f(e[j]) * rstd * (bf2f(ew[j]) + (zero_centered ? 1.f : 0.f)));
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(bf2f(e[j])));
      if (QUANT == 0) bcast16<MC>(c, c.peer_out, c.mc_out, ((size_t)t * H + i) * 2, u);
      else *reinterpret_cast<uint4*>(row + i) = u;
    }
    if (QUANT == 1) {
      amax = block_reduce_c(amax, red, true);
      const float g = fmaxf(amax / (6.f * 448.f), 1e-30f);
      if (threadIdx.x == 0) bcast4<MC>(c, c.peer_rs, c.mc_rs, (size_t)t * 4, __float_as_uint(g));
      // one thread per 64 elements: four 16-element blocks → 32 packed bytes and the 4 scale bytes of one tile column
      for (int b4 = threadIdx.x; b4 < H / 64; b4 += blockDim.x) {
        uint32_t sfw = 0;
        uint32_t pk[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float v[16];
          float bm = 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) { v[j] = bf2f(row[b4 * 64 + q * 16 + j]); bm = fmaxf(bm, fabsf(v[j])); }
          const uint8_t sf = f2e4m3_c(bm / 6.f / g);
          const float denom = e4m32f_c(sf) * g;
          uint32_t lo4 = 0, hi4 = 0;
#pragma unroll
          for (int j = 0; j < 8; ++j) lo4 |= f2e2m1_c(denom > 0.f ? v[j] / denom : 0.f) << (4 * j);
#pragma unroll
          for (int j = 0; j < 8; ++j) hi4 |= f2e2m1_c(denom > 0.f ? v[8 + j] / denom : 0.f) << (4 * j);
          pk[q * 2] = lo4; pk[q * 2 + 1] = hi4;
          sfw |= (uint32_t)sf << (8 * q);
        }
        const size_t qoff = (size_t)t * (H / 2) + (size_t)b4 * 32;
        bcast16<MC>(c, c.peer_out, c.mc_out, qoff, make_uint4(pk[0], pk[1], pk[2], pk[3]));
        bcast16<MC>(c, c.peer_out, c.mc_out, qoff + 16, make_uint4(pk[4], pk[5], pk[6], pk[7]));
        const size_t soff = ((size_t)(t >> 7) * sf_col_tiles + b4) * 512 + (t & 31) * 16 + ((t >> 5) & 3) * 4;
        bcast4<MC>(c, c.peer_sf, c.mc_sf, soff, sfw);
      }
    } else if (QUANT == 2) {
      __syncthreads();
      // one thread per 128 elements: four 32-element blocks → 128 e4m3 bytes and 4 e8m0 scale bytes
      for (int b4 = threadIdx.x; b4 < H / 128; b4 += blockDim.x) {
        uint32_t sfw = 0;
#pragma unroll 1
        for (int q = 0; q < 4; ++q) {
          float v[32];
          float bm = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) { v[j] = bf2f(row[b4 * 128 + q * 32 + j]); bm = fmaxf(bm, fabsf(v[j])); }
          bm = fmaxf(bm, 1.17549435e-38f);
          int ex = (int)ceilf(log2f(bm / 448.f));
          ex = max(-127, min(127, ex));
          const float inv = exp2f((float)-ex);
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            w[j] = f2e4m3_c(v[4 * j] * inv) | (f2e4m3_c(v[4 * j + 1] * inv) << 8) | (f2e4m3_c(v[4 * j + 2] * inv) << 16) |
                   (f2e4m3_c(v[4 * j + 3] * inv) << 24);
          const size_t qoff = (size_t)t * H + (size_t)b4 * 128 + q * 32;
          bcast16<MC>(c, c.peer_out, c.mc_out, qoff, make_uint4(w[0], w[1], w[2], w[3]));
          bcast16<MC>(c, c.peer_out, c.mc_out, qoff + 16, make_uint4(w[4], w[5], w[6], w[7]));
          sfw |= (uint32_t)(ex + 127) << (8 * q);
        }
        const size_t soff = ((size_t)(t >> 7) * sf_col_tiles + b4) * 512 + (t & 31) * 16 + ((t >> 5) & 3) * 4;
        bcast4<MC>(c, c.peer_sf, c.mc_sf, soff, sfw);
      }
    }
    __syncthreads();
  }
  rank_barrier(c, &ok, 1);
}

}  // namespace blz

using namespace blz;

// A communicator is a plain struct filled from Python (pointers obtained from the symmetric-memory rendezvous).
struct BlzComm {
  CommParams p;
};

// timeout_ms: how long a rank waits for its peers inside a kernel before it records an error and moves on.
BLZ_API void* blz_comm_create(int rank, int world, void* const* pads, void* epoch, int timeout_ms) {
  if (world < 1 || world > kMaxWorld) return nullptr;
  BlzComm* c = new BlzComm();
  memset(&c->p, 0, sizeof(c->p));
  c->p.rank = rank; c->p.world = world;
  for (int r = 0; r < world; ++r) c->p.peer_pad[r] = reinterpret_cast<uint32_t*>(pads[r]);
  c->p.epoch = reinterpret_cast<uint32_t*>(epoch);
  c->p.status = status_word();
  c->p.spin_limit = (long long)(timeout_ms > 0 ? timeout_ms : 10000) * 1900000LL;
  return c;
}
BLZ_API void blz_comm_destroy(void* h) { delete reinterpret_cast<BlzComm*>(h); }
BLZ_API int blz_comm_pad_bytes() { return kMaxBlocks * kMaxWorld * 4; }
BLZ_API int blz_comm_epoch_bytes() { return kMaxBlocks * 4; }

static void fill(CommParams& p, int world, void* const* in, void* const* out, void* const* sf, void* const* rs, void* mc_in,
                 void* mc_out, void* mc_sf, void* mc_rs) {
  for (int r = 0; r < world; ++r) {
    p.peer_in[r] = in ? in[r] : nullptr;
    p.peer_out[r] = out ? out[r] : nullptr;
    p.peer_sf[r] = sf ? sf[r] : nullptr;
    p.peer_rs[r] = rs ? rs[r] : nullptr;
  }
  p.mc_in = mc_in; p.mc_out = mc_out; p.mc_sf = mc_sf; p.mc_rs = mc_rs;
}

// In: per-rank pointers to the partial sums (bf16, `nbytes` each, a multiple of 16).  Out: per-rank result pointers
// (may alias In).  mc_* non-null selects the NVSwitch multimem path.
BLZ_API int blz_comm_allreduce(void* h, void* const* in, void* const* out, void* mc_in, void* mc_out, long long nbytes,
                               int blocks, cudaStream_t s) {
  BlzComm* c = reinterpret_cast<BlzComm*>(h);
  if (!c || nbytes % 16 || blocks < 1 || blocks > kMaxBlocks) return (int)cudaErrorInvalidValue;
  CommParams p = c->p;
  fill(p, p.world, in, out, nullptr, nullptr, mc_in, mc_out, nullptr, nullptr);
  if (mc_in && mc_out) allreduce_kernel<true><<<blocks, 512, 0, s>>>(p, (size_t)nbytes / 16);
  else allreduce_kernel<false><<<blocks, 512, 0, s>>>(p, (size_t)nbytes / 16);
  return (int)cudaGetLastError();
}

// Fused all-reduce + residual + RMSNorm (+ quantise).  quant: 0 bf16 rows, 1 NVFP4, 2 MXFP8.
BLZ_API int blz_comm_allreduce_norm(void* h, void* const* in, void* const* out, void* const* sf, void* const* rs, void* mc_in,
                                    void* mc_out, void* mc_sf, void* mc_rs, void* residual, const void* norm_w, int T, int H,
                                    int rows_per, float eps, int zero_centered, int quant, int blocks, cudaStream_t s) {
  BlzComm* c = reinterpret_cast<BlzComm*>(h);
  if (!c || H % 128 || blocks < 1 || blocks > kMaxBlocks || quant < 0 || quant > 2) return (int)cudaErrorInvalidValue;
  CommParams p = c->p;
  fill(p, p.world, in, out, sf, rs, mc_in, mc_out, mc_sf, mc_rs);
  const bool mc = mc_in && mc_out && (quant == 0 || mc_sf) && (quant != 1 || mc_rs);
  int thr = (H / 8 + 31) / 32 * 32;
  thr = thr > 1024 ? 1024 : thr;
  const size_t sm = (size_t)H * 2;
  const int ct = quant == 1 ? (H + 63) / 64 : (H + 127) / 128;
  __nv_bfloat16* res = reinterpret_cast<__nv_bfloat16*>(residual);
  const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(norm_w);
#define BLZ_ARN(MCV, Q)                                                                                              \
  {                                                                                                                  \
    static bool done = false;                                                                                        \
    if (!done) { cudaFuncSetAttribute(allreduce_norm_kernel<MCV, Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); done = true; } \
    allreduce_norm_kernel<MCV, Q><<<blocks, thr, sm, s>>>(p, res, w, T, H, rows_per, eps, zero_centered, ct);          \
  }
  if (mc) { if (quant == 0) BLZ_ARN(true, 0) else if (quant == 1) BLZ_ARN(true, 1) else BLZ_ARN(true, 2) }
  else { if (quant == 0) BLZ_ARN(false, 0) else if (quant == 1) BLZ_ARN(false, 1) else BLZ_ARN(false, 2) }
#undef BLZ_ARN
  return (int)cudaGetLastError();
}
