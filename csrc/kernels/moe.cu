// Mixture-of-experts routing and token movement around the grouped tcgen05 GEMM:
//   route   : softmax over all experts → top-k (lowest id wins ties) → optional renormalisation, plus a histogram of
//             the experts this rank holds (reference semantics: kernels/src/cuda/ops_basic.cu router_topk_kernel :196)
//   plan    : prefix sums of the 128-row padded per-expert counts → row offsets and the expert of every M tile
//   scatter : copies each routed token's (quantised) activation row into its expert's row range
//   combine : out[token] = sum_k w[token,k] * y[row_of(token,k)]
// Experts not held by this rank (expert parallelism) are skipped: the result is this rank's partial sum, which the
// fused reduce + norm kernel adds across ranks — tokens are already replicated, so no dispatch traffic is needed.
// The reference instead tiers experts over GPU0 / GPU1 / CPU / SSD behind host mailboxes
// (kernels/src/cuda/moe_narrow.cu plan_kernel :171, combine :484; kernels/src/runtime/hybrid.cpp:282).
#include "blaze/host.h"
#include "blaze/sm100.cuh"

namespace blz {

// One warp per token.  E <= 512, k <= 32.
__global__ void moe_route_kernel(const float* __restrict__ logits, float* __restrict__ topk_w, int* __restrict__ topk_id,
                                 int* __restrict__ counts, int T, int E, int k, int renorm, int first, int local_n) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  constexpr int PER = 16;
  float v[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = j * 32 + lane;
    v[j] = e < E ? logits[(size_t)t * E + e] : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    v[j] = (j * 32 + lane) < E ? __expf(v[j] - mx) : -1.f;      // -1 marks "absent / taken"
    if (v[j] > 0.f) sum += v[j];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int i = 0; i < k; ++i) {
    float best = -1.f;
    int bid = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < PER; ++j)
      if (v[j] > best) { best = v[j]; bid = j * 32 + lane; }     // ascending ids within the lane: first max = lowest id
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bid, o);
      if (ob > best || (ob == best && oi < bid)) { best = ob; bid = oi; }
    }
    if ((bid & 31) == lane) v[bid >> 5] = -1.f;
    if (lane == i) { my_w = best * inv; my_id = bid; }
    wsum += best * inv;
  }
  if (lane < k) {
    topk_w[(size_t)t * k + lane] = renorm ? my_w / wsum : my_w;
    topk_id[(size_t)t * k + lane] = my_id;
    const int le = my_id - first;
    if (le >= 0 && le < local_n) atomicAdd(&counts[le], 1);
  }
}

// Single block.  offsets[e] = first row of expert e in the padded row space; tile_expert[m_tile] = local expert or -1.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ fill,
                                int* __restrict__ tile_expert, int* __restrict__ tile_rows, int local_n, int max_tiles) {
  __shared__ int s_off[513];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < local_n; ++e) {
      s_off[e] = acc;
      acc += (counts[e] + 127) / 128 * 128;
    }
    s_off[local_n] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < local_n; e += blockDim.x) {
    offsets[e] = s_off[e];
    fill[e] = 0;
  }
  for (int tl = threadIdx.x; tl < max_tiles; tl += blockDim.x) {
    const int row = tl * 128;
    int ex = -1;
    if (row < s_off[local_n]) {
      int lo = 0, hi = local_n - 1;       // last e with s_off[e] <= row
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_off[mid] <= row) lo = mid; else hi = mid - 1;
      }
      ex = lo;
    }
    tile_expert[tl] = ex;
    if (tile_rows) tile_rows[tl] = ex < 0 ? 0 : min(128, counts[ex] - (row - s_off[ex]));     // live rows of the tile
  }
}

// One block per token.  QK: 0 = bf16 rows [T, K]; 1 = NVFP4 (data [T, K/2], tiled e4m3 scales, row scale); 2 = MXFP8.
template <int QK>
__global__ void moe_scatter_kernel(const uint8_t* __restrict__ src, const uint8_t* __restrict__ src_sf,
                                   const float* __restrict__ src_rs, uint8_t* __restrict__ dst, uint8_t* __restrict__ dst_sf,
                                   float* __restrict__ dst_rs, const int* __restrict__ topk_id, const int* __restrict__ offsets,
                                   int* __restrict__ fill, int* __restrict__ row_map, int K, int k, int first, int local_n,
                                   int sf_tiles) {
  const int t = blockIdx.x;
  __shared__ int s_row[32];
  if (threadIdx.x < k) {
    const int le = topk_id[(size_t)t * k + threadIdx.x] - first;
    int row = -1;
    if (le >= 0 && le < local_n) row = offsets[le] + atomicAdd(&fill[le], 1);
    s_row[threadIdx.x] = row;
    row_map[(size_t)t * k + threadIdx.x] = row;
  }
  __syncthreads();
  const int row_bytes = QK == 0 ? K * 2 : (QK == 1 ? K / 2 : K);
  const int sf_cols = QK == 1 ? K / 16 : (QK == 2 ? K / 32 : 0);          // scale bytes per row (multiple of 4)
  for (int j = 0; j < k; ++j) {
    const int row = s_row[j];
    if (row < 0) continue;
    const uint4* s4 = reinterpret_cast<const uint4*>(src + (size_t)t * row_bytes);
    uint4* d4 = reinterpret_cast<uint4*>(dst + (size_t)row * row_bytes);
    for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) d4[i] = s4[i];
    if (QK != 0) {
      for (int c4 = threadIdx.x; c4 < sf_cols / 4; c4 += blockDim.x) {
        const size_t so = ((size_t)(t >> 7) * sf_tiles + c4) * 512 + (t & 31) * 16 + ((t >> 5) & 3) * 4;
        const size_t dofs = ((size_t)(row >> 7) * sf_tiles + c4) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4;
        *reinterpret_cast<uint32_t*>(dst_sf + dofs) = *reinterpret_cast<const uint32_t*>(src_sf + so);
      }
      if (QK == 1 && threadIdx.x == 0) dst_rs[row] = src_rs[t];
    }
  }
}

__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ topk_w,
                                   const int* __restrict__ row_map, __nv_bfloat16* __restrict__ out, int H, int k) {
  const int t = blockIdx.x;
  __shared__ float s_w[32];
  __shared__ int s_row[32];
  if (threadIdx.x < k) {
    s_w[threadIdx.x] = topk_w[(size_t)t * k + threadIdx.x];
    s_row[threadIdx.x] = row_map[(size_t)t * k + threadIdx.x];
  }
  __syncthreads();
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const int row = s_row[j];
      if (row < 0) continue;
      const uint4 u = *reinterpret_cast<const uint4*>(y + (size_t)row * H + i);
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] += s_w[j] * bf2f(e[q]);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * H + i) =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

}  // namespace blz

using namespace blz;

BLZ_API int blz_moe_route(const float* logits, float* topk_w, int* topk_id, int* counts, int T, int E, int k, int renorm,
                          int first, int local_n, cudaStream_t s) {
  if (E > 512 || k > 32 || k < 1 || local_n > 512) return (int)cudaErrorInvalidValue;
  cudaMemsetAsync(counts, 0, sizeof(int) * (local_n > 0 ? local_n : 1), s);
  if (T == 0) return 0;
  moe_route_kernel<<<(T + 3) / 4, 128, 0, s>>>(logits, topk_w, topk_id, counts, T, E, k, renorm, first, local_n);
  return (int)cudaGetLastError();
}

BLZ_API int blz_moe_plan(const int* counts, int* offsets, int* fill, int* tile_expert, int* tile_rows, int local_n,
                         int max_tiles, cudaStream_t s) {
  moe_plan_kernel<<<1, 256, 0, s>>>(counts, offsets, fill, tile_expert, tile_rows, local_n, max_tiles);
  return (int)cudaGetLastError();
}

BLZ_API int blz_moe_scatter(int qk, const void* src, const void* src_sf, const float* src_rs, void* dst, void* dst_sf,
                            float* dst_rs, const int* topk_id, const int* offsets, int* fill, int* row_map, int T, int K, int k,
                            int first, int local_n, cudaStream_t s) {
  if (T == 0) return 0;
  const int sf_tiles = qk == 1 ? (K + 63) / 64 : (K + 127) / 128;
#define BLZ_SC(Q) moe_scatter_kernel<Q><<<T, 128, 0, s>>>((const uint8_t*)src, (const uint8_t*)src_sf, src_rs, (uint8_t*)dst, \
    (uint8_t*)dst_sf, dst_rs, topk_id, offsets, fill, row_map, K, k, first, local_n, sf_tiles)
  if (qk == 0) BLZ_SC(0); else if (qk == 1) BLZ_SC(1); else BLZ_SC(2);
#undef BLZ_SC
  return (int)cudaGetLastError();
}

BLZ_API int blz_moe_combine(const void* y, const float* topk_w, const int* row_map, void* out, int T, int H, int k,
                            cudaStream_t s) {
  if (T == 0) return 0;
  moe_combine_kernel<<<T, 256, 0, s>>>((const __nv_bfloat16*)y, topk_w, row_map, (__nv_bfloat16*)out, H, k);
  return (int)cudaGetLastError();
}
