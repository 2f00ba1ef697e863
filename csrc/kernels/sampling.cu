// Sampler kernels: the ordered stage chain on fp32 logits for rows whose first filter is top_k <= 64 (the "bounded"
// path), plus log-sum-exp and top-64 export for log-probs.
//
// One CTA (1024 threads) per row.  Steps: allowed-token mask and vocabulary bound → canonical copy semantics (penalties
// then bias, used for log-probs) → the row's stage program (penalties, logit_bias, temperature) applied on the fly →
// top-64 by repeated block arg-max (ties to the lower id) → top_k / top_p / min_p on the sorted candidates →
// inverse-CDF draw with the host-supplied uniform number.  Status -1 = empty support, -2 = NaN / +inf on an allowed token.
// Reference: kernels/src/cuda/sampling_pipeline.cu (initialize :74, transform :106, top64 :137, filter :193, draw :246,
// export_results :270) and kernels/src/cuda/sampling.cu (topk_radix_kernel :58, penalties :196, edits :211, lse :242).
#include "blaze/host.h"
#include "blaze/sm100.cuh"

namespace blz {

struct SamplingRow {
  float temperature, top_p, min_p, draw;
  int top_k;            // <= 64 on this path (<= 0: 64)
  int stage_mask;       // 4 bits per position: stage ids in chain order (1 penalties, 2 bias, 3 temperature, 4 top_k, 5 top_p, 6 min_p)
  int edit_begin, edit_count;    // slice of the edits array
  int want_lse;         // 0 no log-probs, 1 log-prob of the chosen token, 2 also the top-64 alternatives
};

struct Edit { int id; float mul_pos, mul_neg, sub, bias, banned; };

__device__ __forceinline__ void better(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

__global__ void __launch_bounds__(1024) sample_bounded_kernel(const float* __restrict__ logits, long long ld, int V,
                                                              const SamplingRow* __restrict__ rows, const Edit* __restrict__ edits,
                                                              const uint32_t* __restrict__ allowed, int allowed_words,
                                                              long long* __restrict__ out_token, float* __restrict__ out_logprob,
                                                              float* __restrict__ out_lse, float* __restrict__ top_vals,
                                                              int* __restrict__ top_ids,
                                                              int* __restrict__ status, float* __restrict__ work) {
  const int r = blockIdx.x;
  const SamplingRow row = rows[r];
  const float* x = logits + (size_t)r * ld;
  float* w = work + (size_t)r * V;                  // working copy: the chain's view of the logits
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float cand_v[64];
  __shared__ int cand_i[64];
  __shared__ float s_red[32];
  __shared__ int s_flag;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_flag = 0;
  __syncthreads();
  // ---- initialise: mask, vocabulary bound, non-finite check
  const bool do_pen = [&] { for (int s = 0; s < 8; ++s) if (((row.stage_mask >> (4 * s)) & 15) == 1) return true; return false; }();
  const bool do_bias = [&] { for (int s = 0; s < 8; ++s) if (((row.stage_mask >> (4 * s)) & 15) == 2) return true; return false; }();
  bool do_temp = false;
  for (int s = 0; s < 8; ++s) if (((row.stage_mask >> (4 * s)) & 15) == 3) do_temp = true;
  int any_ok = 0;
  for (int i = tid; i < V; i += blockDim.x) {
    bool ok = true;
    if (allowed) ok = (allowed[(size_t)r * allowed_words + (i >> 5)] >> (i & 31)) & 1u;
    float v = x[i];
    if (ok && (isnan(v) || v == INFINITY)) atomicExch(&s_flag, 2);
    if (!ok || !isfinite(v)) v = -INFINITY;
    any_ok |= ok;
    w[i] = v;
  }
  __syncthreads();
  if (s_flag == 2) { if (tid == 0) { status[r] = -2; out_token[r] = -1; } return; }
  // ---- sparse edits (penalties, bias).  The canonical log-prob copy always gets penalties then bias; it is evaluated
  //      lazily below for the exported tokens only.
  for (int e = tid; e < row.edit_count; e += blockDim.x) {
    const Edit ed = edits[row.edit_begin + e];
    if (ed.id < 0 || ed.id >= V) continue;
    float v = w[ed.id];
    if (do_pen) {
      if (ed.banned > 0.f) v = -INFINITY;
      else v = (v > 0.f ? v * ed.mul_pos : v * ed.mul_neg) - ed.sub;
    }
    if (do_bias) v += ed.bias;
    w[ed.id] = v;
  }
  __syncthreads();
  const bool greedy = do_temp && row.temperature == 0.f;
  const float inv_t = (do_temp && row.temperature > 0.f) ? 1.f / row.temperature : 1.f;
  // ---- top-64 by repeated arg-max; every thread keeps the best of its strided slice
  // candidates to collect: the top_k of the chain, or all 64 when the caller also wants log-prob alternatives
  const int k_sel = greedy ? 1 : (row.top_k > 0 && row.top_k < 64 ? row.top_k : 64);
  const int K = row.want_lse >= 2 ? 64 : k_sel;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = tid; i < V; i += blockDim.x) better(best, bi, w[i], i);
  int found = 0;
  for (int k = 0; k < K; ++k) {
    float v = best;
    int id = bi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) better(v, id, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, id, o));
    if (lane == 0) { sv[warp] = v; si[warp] = id; }
    __syncthreads();
    if (warp == 0) {
      v = sv[lane];
      id = si[lane];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) better(v, id, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, id, o));
      if (lane == 0) { cand_v[k] = v; cand_i[k] = id; }
    }
    __syncthreads();
    const int win = cand_i[k];
    if (cand_v[k] == -INFINITY) break;
    found = k + 1;
    if (win != 0x7fffffff && (win % blockDim.x) == tid) {     // the owner rescans its slice without the winner
      w[win] = -INFINITY;
      best = -INFINITY;
      bi = 0x7fffffff;
      for (int i = tid; i < V; i += blockDim.x) better(best, bi, w[i], i);
    }
    __syncthreads();
  }
  if (found == 0) { if (tid == 0) { status[r] = -1; out_token[r] = -1; } return; }
  // ---- filters on the sorted candidates + draw (one thread; <= 64 items)
  if (tid == 0) {
    int n = found < k_sel ? found : k_sel;
    double p[64];
    const double m = (double)cand_v[0] * inv_t;
    auto renorm = [&](int cnt) {
      double s = 0;
      for (int i = 0; i < cnt; ++i) { p[i] = exp((double)cand_v[i] * inv_t - m); s += p[i]; }
      for (int i = 0; i < cnt; ++i) p[i] /= s;
    };
    if (!greedy) {
      for (int s = 0; s < 8; ++s) {
        const int st = (row.stage_mask >> (4 * s)) & 15;
        if (st == 5) {            // top_p: shortest prefix with mass >= p
          renorm(n);
          double c = 0;
          int keep = n;
          for (int i = 0; i < n; ++i) { if (c >= (double)row.top_p) { keep = i; break; } c += p[i]; }
          n = keep < 1 ? 1 : keep;
        } else if (st == 6) {     // min_p
          renorm(n);
          int keep = 0;
          for (int i = 0; i < n; ++i) if (p[i] / p[0] >= (double)row.min_p) keep = i + 1;
          n = keep < 1 ? 1 : keep;
        }
      }
    } else {
      n = 1;
    }
    renorm(n);
    double c = 0;
    int pick = n - 1;
    for (int i = 0; i < n; ++i) { c += p[i]; if ((double)row.draw < c) { pick = i; break; } }
    out_token[r] = cand_i[pick];
    status[r] = 0;
    s_flag = cand_i[pick];
    for (int i = 0; i < 64; ++i) {
      top_vals[(size_t)r * 64 + i] = i < found ? cand_v[i] : -INFINITY;
      top_ids[(size_t)r * 64 + i] = i < found ? cand_i[i] : -1;
    }
  }
  __syncthreads();
  if (!row.want_lse) return;
  // ---- canonical log-prob of the chosen token: log-sum-exp over (logits with penalties then bias)
  const int chosen = s_flag;
  float mx = -INFINITY;
  for (int i = tid; i < V; i += blockDim.x) {
    bool ok = true;
    if (allowed) ok = (allowed[(size_t)r * allowed_words + (i >> 5)] >> (i & 31)) & 1u;
    const float v = ok && isfinite(x[i]) ? x[i] : -INFINITY;
    mx = fmaxf(mx, v);
  }
  mx = warp_max(mx);
  if (lane == 0) s_red[warp] = mx;
  __syncthreads();
  mx = s_red[0];
  for (int i = 1; i < 32; ++i) mx = fmaxf(mx, s_red[i]);
  __syncthreads();
  float sum = 0.f;
  for (int i = tid; i < V; i += blockDim.x) {
    bool ok = true;
    if (allowed) ok = (allowed[(size_t)r * allowed_words + (i >> 5)] >> (i & 31)) & 1u;
    if (ok && isfinite(x[i])) sum += __expf(x[i] - mx);
  }
  sum = warp_sum(sum);
  if (lane == 0) s_red[warp] = sum;
  __syncthreads();
  if (tid == 0) {
    double tot = 0;
    for (int i = 0; i < 32; ++i) tot += s_red[i];
    // correct the sum for the edited ids (few): remove their raw term, add their canonical term
    double canon_chosen = x[chosen];
    for (int e = 0; e < row.edit_count; ++e) {
      const Edit ed = edits[row.edit_begin + e];
      if (ed.id < 0 || ed.id >= V || !isfinite(x[ed.id])) continue;
      double v = x[ed.id];
      tot -= exp(v - (double)mx);
      if (ed.banned > 0.f) v = -INFINITY;
      else v = (v > 0 ? v * ed.mul_pos : v * ed.mul_neg) - ed.sub + ed.bias;
      if (v > -INFINITY) tot += exp(v - (double)mx);
      if (ed.id == chosen) canon_chosen = v;
    }
    const double lse = (double)mx + log(tot);
    out_logprob[r] = (float)(canon_chosen - lse);
    out_lse[r] = (float)lse;
  }
}

}  // namespace blz

// rows: R records of 9 x 4 bytes (see SamplingRow); edits: records of 6 x 4 bytes; allowed: optional bit masks
// [R, allowed_words]; work: R * V floats of scratch.  Outputs: token ids (int64), canonical log-prob of the token, the
// canonical log-sum-exp (rows with want_lse), the top-64 (value, id) pairs of the edited logits, status.
BLZ_API int blz_sample_bounded(const float* logits, long long ld, int R, int V, const void* rows, const void* edits,
                               const void* allowed, int allowed_words, long long* out_token, float* out_logprob, float* out_lse,
                               float* top_vals, int* top_ids, int* status, float* work, cudaStream_t s) {
  if (R == 0) return 0;
  blz::sample_bounded_kernel<<<R, 1024, 0, s>>>(logits, ld, V, (const blz::SamplingRow*)rows, (const blz::Edit*)edits,
                                                (const uint32_t*)allowed, allowed_words, out_token, out_logprob, out_lse, top_vals,
                                                top_ids, status, work);
  return (int)cudaGetLastError();
}
