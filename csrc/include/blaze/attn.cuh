// Shared declarations of the paged-attention kernels (prefill/verify row-block kernel and decode kernel).
#pragma once
#include "blaze/sm100.cuh"

namespace blz {

struct AttnParams {
  const __nv_bfloat16* q;      // [T, Hq, D]
  __nv_bfloat16* out;          // [T, Hq, D]
  const uint8_t* pool;         // blocks of [2, 16*D] bytes (K, V^T) addressed by page * page_stride + head * head_stride
  long long page_stride, head_stride;   // bytes; the storage may be page-major or head-major
  const int* block_table;      // [max_seqs, bt_stride]
  const int* slots;            // [B]
  const int* q_start;          // [B+1]
  const int* ctx_len;          // [B]
  const int* item_seq;         // [items] or null (then item = seq * Hkv... decode mapping)
  const int* item_q0;          // [items] first token (relative to the sequence's rows) of the row block
  float* part_o;               // [items*splits, 128, D] partial outputs (splits > 1)
  float* part_ml;              // [items*splits, 128, 2] partial (max, sum)
  int num_items;               // row-block items (without heads / splits)
  int Hq, Hkv, bt_stride, splits;
  float scale_log2;            // softmax scale * log2(e) * k_scale
  float v_scale;
  int tokens_per_block;        // 128 / group (rows per item = tokens_per_block * group)
  int min_rows, max_rows;      // a sequence is processed iff min_rows <= q_len * group <= max_rows
  int row_blocks;              // decode kernel: row blocks of NMAX rows per (sequence, kv head)
  long long* prof;             // optional [blocks][16] wait-cycle counters (null = off)
  int* status;
  const int* tree_mask = nullptr;   // decode kernel, verify rows: [T] bit j = this row may see the sequence's j-th new token
};


__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}


}  // namespace blz
