// Collectives over NVLink peer memory, issued from inside the kernels (no library call on the hot path):
//
//   * all-reduce of a bf16 buffer that lives in symmetric memory: every rank reduces 1/world of the rows and
//     broadcasts its slice — through the NVSwitch (`multimem.ld_reduce` / `multimem.st`) when a multicast mapping
//     exists, else through plain peer loads / stores in rank order (identical bits on every rank);
//   * the same reduction fused with the residual add and the next RMSNorm, optionally quantising the normed rows
//     to NVFP4 / MXFP8 for the following GEMM, so that what crosses NVLink on the way back is the 4/8-bit
//     activation, and the residual stream stays sharded by rows (sequence-parallel between the two collectives).
//
// Rank synchronisation is a flag barrier in symmetric memory: relaxed system-scope stores to the peers' pads after one
// system fence, relaxed polls of the own pad, a monotonically increasing epoch kept in device memory (so captured CUDA graphs replay correctly), and a
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
  uint32_t* peer_sig[kMaxWorld];  // arrival counters of every rank, [kMaxWorld] uint32 each (slot = source rank)
  uint32_t* sig_expect;           // local: the count a consumer of a signalling kernel's result must wait for
  long long* prof;                // optional [8] nanosecond stamps of block 0 (entry, after each phase); null = off
  // reduce-scatter by push: the partial rows this rank owns arrive in its LOCAL slot buffer [world][rows_per][H] (stored
  // there by every rank's GEMM epilogue), announced by flag [source rank] reaching the value in *slot_epoch
  const __nv_bfloat16* slots;     // null = the partial sums are in peer_in / mc_in and a rank barrier opens the kernel
  const uint32_t* slot_flags;     // [world] local
  const uint32_t* slot_epoch;     // local word, advanced by this rank's own producing GEMM
};

__device__ __forceinline__ void stamp(const CommParams& c, int k) {
  if (c.prof && blockIdx.x == 0 && threadIdx.x == 0) {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    c.prof[k] = t;
  }
}


__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Block-level barrier across ranks: block b of every rank meets block b of every other rank.
// Every kernel uses two barrier epochs (entry = base + 1, exit = base + 2) and advances the stored epoch by two at
// entry, so a rank that gave up on a wait stays in step with its peers on the next kernel.
// Returns false (after recording kErrFlagTimeout) when a peer does not show up within the spin limit.
//
// Cost matters here (a decode step runs dozens of these): only the `world` signalling threads touch the fabric.  The
// CTA barrier orders every thread's earlier stores before the signalling threads; at the exit phase those threads
// issue ONE system-scope fence (so the result stores are visible before the flag) and at the entry phase none (there
// is nothing to publish).  Flags are written and polled relaxed; one fence after the wait orders the reads that follow.
// phase 2 = exit without waiting: publish the results and the flag, return at once; whoever consumes the results waits
// for the flags itself (the GEMM that follows does, after it has started fetching its weights).
__device__ __forceinline__ bool rank_barrier(const CommParams& c, int* ok_smem, int phase) {
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
  __syncthreads();
  const uint32_t e = s_epoch;
  if (threadIdx.x < c.world) {
    const int peer = threadIdx.x;
    if (phase >= 1) fence_acq_rel_sys();
    if (phase == 2) {
      // one arrival per block on every peer's counter; the consumer polls `world` words instead of one flag per block
      asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(c.peer_sig[peer] + c.rank), "r"(1u) : "memory");
    } else {
      st_relaxed_sys(c.peer_pad[peer] + (size_t)blockIdx.x * kMaxWorld + c.rank, e);
    }
    const uint32_t* mine = c.peer_pad[c.rank] + (size_t)blockIdx.x * kMaxWorld + peer;
    const long long t0 = clock64();
    while (phase != 2 && (int32_t)(ld_relaxed_sys(mine) - e) < 0) {
      if (clock64() - t0 > c.spin_limit) {
        atomicCAS(c.status, kOk, kErrFlagTimeout);
        *ok_smem = 0;
        break;
      }
    }
    if (phase == 0) fence_acq_rel_sys();
  }
  __syncthreads();
  return *ok_smem != 0;
}

// Entry of a kernel whose inputs were pushed into this rank's slot buffer: no barrier, no traffic - wait (bounded) until every
// source rank's flag has reached the epoch of the reduction.  Keeps the barrier epochs in step for the exit phase.
__device__ __forceinline__ bool wait_slots(const CommParams& c, int* ok_smem) {
  if (threadIdx.x == 0) {
    c.epoch[blockIdx.x] += 2;
    *ok_smem = 1;
  }
  __syncthreads();
  if (threadIdx.x < c.world) {
    const uint32_t want = *c.slot_epoch;
    const uint32_t* f = c.slot_flags + threadIdx.x;
    const long long t0 = clock64();
    while (true) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if ((int32_t)(v - want) >= 0) break;
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
  pdl_trigger();
  pdl_wait();
  stamp(c, 0);
  if (!rank_barrier(c, &ok, 0)) return;
  stamp(c, 1);
  const size_t per = (n16 + c.world - 1) / c.world;
  const size_t lo = (size_t)c.rank * per, hi = min(n16, lo + per);
  for (size_t i = lo + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += (size_t)gridDim.x * blockDim.x) {
    float f[8];
    reduce8<MC>(c, i * 16, f);
    uint4 o = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
    bcast16<MC>(c, c.peer_out, c.mc_out, i * 16, o);
  }
  stamp(c, 3);
  rank_barrier(c, &ok, 1);
  stamp(c, 4);
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
//
// One row per CTA at a time; thread i owns CH chunks of 8 consecutive elements (chunk c covers elements
// (c * blockDim + i) * 8 ...), which stay in registers from the reduction to the quantised stores.  A 16-element NVFP4
// block is two neighbouring threads, a 32-element MXFP8 block four; neighbours pool their packed codes through
// shuffles so that what goes through the switch are 16-byte (codes) and 4-byte (scale tile column) stores.
__device__ __forceinline__ uint32_t pack_e2m1x8_c(const float (&v)[8], float inv) {
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
__device__ __forceinline__ uint32_t pack_e4m3x4_c(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

template <bool MC, int QUANT, int CH>
__global__ void __launch_bounds__(1024) allreduce_norm_kernel(CommParams c, __nv_bfloat16* residual,
                                                              const __nv_bfloat16* __restrict__ norm_w, int T, int H,
                                                              int rows_per, float eps, int zero_centered, int sf_col_tiles,
                                                              int defer_exit) {
  __shared__ float red[32];
  __shared__ int ok;
  pdl_trigger();
  pdl_wait();
  stamp(c, 0);
  if (defer_exit && blockIdx.x == 0 && threadIdx.x == 0) *c.sig_expect += gridDim.x;
  if (c.slots != nullptr) {
    if (!wait_slots(c, &ok)) return;
  } else if (!rank_barrier(c, &ok, 0)) {
    return;
  }
  stamp(c, 1);
  const int lo = c.rank * rows_per, hi = min(T, lo + rows_per);
  const int lane = threadIdx.x & 31;
  for (int t = lo + blockIdx.x; t < hi; t += gridDim.x) {
    __nv_bfloat16* rr = residual ? residual + (size_t)(t - lo) * H : nullptr;
    uint4 u[CH];
    float ss = 0.f;
#pragma unroll
    for (int ch = 0; ch < CH; ++ch) {
      const int i = (ch * blockDim.x + threadIdx.x) * 8;
      u[ch] = make_uint4(0, 0, 0, 0);
      if (i < H) {
        float f[8];
        if (c.slots != nullptr) {
          // the partial rows of every source rank, from local memory, summed in rank order
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = 0.f;
          for (int r = 0; r < c.world; ++r) {
            const uint4 v = *reinterpret_cast<const uint4*>(c.slots + ((size_t)r * rows_per + (t - lo)) * H + i);
            const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] += bf2f(e[j]);
          }
        } else {
          reduce8<MC>(c, ((size_t)t * H + i) * 2, f);
        }
        __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&u[ch]);
        if (rr) {
          const uint4 ur = *reinterpret_cast<const uint4*>(rr + i);
          const __nv_bfloat16* er = reinterpret_cast<const __nv_bfloat16*>(&ur);
#pragma unroll
          for (int j = 0; j < 8; ++j) e[j] = __float2bfloat16(bf2f(__float2bfloat16(f[j])) + bf2f(er[j]));
          *reinterpret_cast<uint4*>(rr + i) = u[ch];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) e[j] = __float2bfloat16(f[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float x = bf2f(e[j]); ss += x * x; }
      }
    }
    float rstd = 1.f;
    if (norm_w) {
      ss = block_reduce_c(ss, red, false);
      rstd = rsqrtf(ss / H + eps);
    }
    stamp(c, 2);
    float amax = 0.f;
#pragma unroll
    for (int ch = 0; ch < CH; ++ch) {
      const int i = (ch * blockDim.x + threadIdx.x) * 8;
      __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&u[ch]);
      if (norm_w && i < H) {
        const uint4 uw = *reinterpret_cast<const uint4*>(norm_w + i);
        const __nv_bfloat16* ew = reinterpret_cast<const __nv_bfloat16*>(&uw);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          e[j] = __float2bfloat16(bf2f(e[j]) * rstd * (bf2f(ew[j]) + (zero_centered ? 1.f : 0.f)));
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(bf2f(e[j])));
      if (QUANT == 0 && i < H) bcast16<MC>(c, c.peer_out, c.mc_out, ((size_t)t * H + i) * 2, u[ch]);
    }
    if (QUANT == 1) {
      amax = block_reduce_c(amax, red, true);
      const float g = fmaxf(amax / (6.f * 448.f), 1e-30f);
      if (threadIdx.x == 0) bcast4<MC>(c, c.peer_rs, c.mc_rs, (size_t)t * 4, __float_as_uint(g));
#pragma unroll
      for (int ch = 0; ch < CH; ++ch) {
        const int i = (ch * blockDim.x + threadIdx.x) * 8;
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u[ch]);
        float v[8];
        float bm = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[j] = bf2f(e[j]); bm = fmaxf(bm, fabsf(v[j])); }
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
        const uint32_t sf = f2e4m3_c(bm / 6.f / g);
        const float denom = e4m32f_c((uint8_t)sf) * g;
        const uint32_t codes = pack_e2m1x8_c(v, denom > 0.f ? 1.f / denom : 0.f);
        // four threads -> 16 bytes of codes (32 elements); eight threads -> the 4 scale bytes of one 64-element tile column
        const uint32_t c1 = __shfl_down_sync(0xffffffffu, codes, 1), c2 = __shfl_down_sync(0xffffffffu, codes, 2),
                       c3 = __shfl_down_sync(0xffffffffu, codes, 3);
        const uint32_t s2 = __shfl_down_sync(0xffffffffu, sf, 2), s4 = __shfl_down_sync(0xffffffffu, sf, 4),
                       s6 = __shfl_down_sync(0xffffffffu, sf, 6);
        if (i < H) {
          if ((lane & 3) == 0) bcast16<MC>(c, c.peer_out, c.mc_out, (size_t)t * (H / 2) + i / 2, make_uint4(codes, c1, c2, c3));
          if ((lane & 7) == 0) {
            const size_t soff = ((size_t)(t >> 7) * sf_col_tiles + (i >> 6)) * 512 + (t & 31) * 16 + ((t >> 5) & 3) * 4;
            bcast4<MC>(c, c.peer_sf, c.mc_sf, soff, sf | (s2 << 8) | (s4 << 16) | (s6 << 24));
          }
        }
      }
    } else if (QUANT == 2) {
#pragma unroll
      for (int ch = 0; ch < CH; ++ch) {
        const int i = (ch * blockDim.x + threadIdx.x) * 8;
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u[ch]);
        float v[8];
        float bm = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[j] = bf2f(e[j]); bm = fmaxf(bm, fabsf(v[j])); }
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
        bm = fmaxf(bm, 1.17549435e-38f);
        int ex = (int)ceilf(log2f(bm / 448.f));
        ex = max(-127, min(127, ex));
        const float inv = exp2f((float)-ex);
        const uint32_t w0 = pack_e4m3x4_c(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
        const uint32_t w1 = pack_e4m3x4_c(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
        const uint32_t n0 = __shfl_down_sync(0xffffffffu, w0, 1), n1 = __shfl_down_sync(0xffffffffu, w1, 1);
        const uint32_t sf = (uint32_t)(ex + 127);
        const uint32_t s4 = __shfl_down_sync(0xffffffffu, sf, 4), s8 = __shfl_down_sync(0xffffffffu, sf, 8),
                       s12 = __shfl_down_sync(0xffffffffu, sf, 12);
        if (i < H) {
          if ((lane & 1) == 0) bcast16<MC>(c, c.peer_out, c.mc_out, (size_t)t * H + i, make_uint4(w0, w1, n0, n1));
          if ((lane & 15) == 0) {
            const size_t soff = ((size_t)(t >> 7) * sf_col_tiles + (i >> 7)) * 512 + (t & 31) * 16 + ((t >> 5) & 3) * 4;
            bcast4<MC>(c, c.peer_sf, c.mc_sf, soff, sf | (s4 << 8) | (s8 << 16) | (s12 << 24));
          }
        }
      }
    }
  }
  stamp(c, 3);
  rank_barrier(c, &ok, defer_exit ? 2 : 1);
  stamp(c, 4);
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
// Arrival counters for kernels that signal instead of waiting: sigs[r] = rank r's counter row (kMaxWorld uint32, zeroed),
// expect = a zeroed local device word.
BLZ_API void blz_comm_set_signals(void* h, void* const* sigs, void* expect) {
  BlzComm* c = reinterpret_cast<BlzComm*>(h);
  if (!c) return;
  for (int r = 0; r < c->p.world; ++r) c->p.peer_sig[r] = reinterpret_cast<uint32_t*>(sigs[r]);
  c->p.sig_expect = reinterpret_cast<uint32_t*>(expect);
}
// Nanosecond stamps of block 0 of every later collective kernel go to `prof` (device memory, 8 x int64); null turns it off.
BLZ_API void blz_comm_set_prof(void* h, void* prof) {
  if (h) reinterpret_cast<BlzComm*>(h)->p.prof = reinterpret_cast<long long*>(prof);
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
  if (mc_in && mc_out) launch_pdl(allreduce_kernel<true>, dim3(blocks), dim3(512), 0, s, p, (size_t)nbytes / 16);
  else launch_pdl(allreduce_kernel<false>, dim3(blocks), dim3(512), 0, s, p, (size_t)nbytes / 16);
  return (int)cudaGetLastError();
}

// Fused all-reduce + residual + RMSNorm (+ quantise).  quant: 0 bf16 rows, 1 NVFP4, 2 MXFP8.
// defer_exit: the kernel signals the peers and returns without waiting for theirs; the consumer of the result must wait
// for this rank's arrival counters to reach the expected count (blz_comm_set_signals, blz_gemm_wait_flags).
static int launch_norm(CommParams& p, bool mc, void* residual, const void* norm_w, int T, int H, int rows_per, float eps,
                       int zero_centered, int quant, int blocks, int defer_exit, cudaStream_t s) {
  if (H % 128 || blocks < 1 || blocks > kMaxBlocks || quant < 0 || quant > 2) return (int)cudaErrorInvalidValue;
  if (defer_exit && !p.sig_expect) return (int)cudaErrorInvalidValue;
  // threads: a multiple of 32 covering H/8 chunks in at most 4 rounds
  int ch = (H / 8 + 1023) / 1024;
  if (ch > 4) return (int)cudaErrorInvalidValue;
  int thr = ((H / 8 + ch - 1) / ch + 31) / 32 * 32;
  const int ct = quant == 1 ? (H + 63) / 64 : (H + 127) / 128;
  __nv_bfloat16* res = reinterpret_cast<__nv_bfloat16*>(residual);
  const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(norm_w);
#define BLZ_ARN3(MCV, Q, C) launch_pdl(allreduce_norm_kernel<MCV, Q, C>, dim3(blocks), dim3(thr), 0, s, p, res, w, T, H, rows_per, eps, zero_centered, ct, defer_exit)
#define BLZ_ARN2(MCV, Q)                                                                  \
  { if (ch == 1) BLZ_ARN3(MCV, Q, 1); else if (ch == 2) BLZ_ARN3(MCV, Q, 2); else if (ch == 3) BLZ_ARN3(MCV, Q, 3); else BLZ_ARN3(MCV, Q, 4); }
  if (mc) { if (quant == 0) BLZ_ARN2(true, 0) else if (quant == 1) BLZ_ARN2(true, 1) else BLZ_ARN2(true, 2) }
  else { if (quant == 0) BLZ_ARN2(false, 0) else if (quant == 1) BLZ_ARN2(false, 1) else BLZ_ARN2(false, 2) }
#undef BLZ_ARN2
#undef BLZ_ARN3
  return (int)cudaGetLastError();
}

BLZ_API int blz_comm_allreduce_norm(void* h, void* const* in, void* const* out, void* const* sf, void* const* rs, void* mc_in,
                                    void* mc_out, void* mc_sf, void* mc_rs, void* residual, const void* norm_w, int T, int H,
                                    int rows_per, float eps, int zero_centered, int quant, int blocks, int defer_exit,
                                    cudaStream_t s) {
  BlzComm* c = reinterpret_cast<BlzComm*>(h);
  if (!c) return (int)cudaErrorInvalidValue;
  CommParams p = c->p;
  fill(p, p.world, in, out, sf, rs, mc_in, mc_out, mc_sf, mc_rs);
  p.slots = nullptr;
  const bool mc = mc_in && mc_out && (quant == 0 || mc_sf) && (quant != 1 || mc_rs);
  return launch_norm(p, mc, residual, norm_w, T, H, rows_per, eps, zero_centered, quant, blocks, defer_exit, s);
}

// The same reduction + residual + RMSNorm (+ quantise) for partial sums that every rank's GEMM pushed into this rank's slot
// buffer (blz_gemm_push_rs): `slots` = the LOCAL buffer [world][rows_per][H], `flags` = the local flag row [world], `epoch` =
// the local epoch word the producing GEMM advanced.  No entry barrier: the kernel waits (bounded) for the flags.  The results
// are broadcast as in blz_comm_allreduce_norm (out / sf / rs per rank, or their multicast views).
BLZ_API int blz_comm_slots_norm(void* h, const void* slots, const void* flags, const void* epoch, void* const* out,
                                void* const* sf, void* const* rs, void* mc_out, void* mc_sf, void* mc_rs, void* residual,
                                const void* norm_w, int T, int H, int rows_per, float eps, int zero_centered, int quant, int blocks,
                                int defer_exit, cudaStream_t s) {
  BlzComm* c = reinterpret_cast<BlzComm*>(h);
  if (!c || !slots || !flags || !epoch) return (int)cudaErrorInvalidValue;
  CommParams p = c->p;
  fill(p, p.world, nullptr, out, sf, rs, nullptr, mc_out, mc_sf, mc_rs);
  p.slots = reinterpret_cast<const __nv_bfloat16*>(slots);
  p.slot_flags = reinterpret_cast<const uint32_t*>(flags);
  p.slot_epoch = reinterpret_cast<const uint32_t*>(epoch);
  const bool mc = mc_out && (quant == 0 || mc_sf) && (quant != 1 || mc_rs);
  return launch_norm(p, mc, residual, norm_w, T, H, rows_per, eps, zero_centered, quant, blocks, defer_exit, s);
}
