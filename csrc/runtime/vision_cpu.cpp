// CPU vision tower: fp32 ViT encoder (pre-LN blocks with 2-D rotary attention and a GELU MLP) on a thread pool.
// It is the oracle for the CUDA tower and the timed CPU baseline.
// Reference: kernels/src/cpu/vision_cpu.cpp (thread Pool :44, gemm :201, layernorm :254, bias_act :273, qkv_rope :352,
// attention :392).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

#include "blaze/runtime.h"

extern "C" {
struct BlzVitBlock {
  const float *ln1_w, *ln1_b, *qkv_w, *qkv_b, *proj_w, *proj_b, *ln2_w, *ln2_b, *fc1_w, *fc1_b, *fc2_w, *fc2_b;
};
struct BlzVitWeights {
  int hidden, heads, mlp, depth, patch_dim;
  float eps;
  const float *patch_w, *patch_b;      // [hidden, patch_dim], [hidden]
  const float *pos;                    // [n_tokens, hidden] already interpolated, or null
  const float *rope_cos, *rope_sin;    // [n_tokens, head_dim / 2] or null
  const BlzVitBlock* blocks;           // [depth]
  const float *ln_f_w, *ln_f_b;        // final LayerNorm (or null)
};
}

namespace {

void parallel_for(int n, int threads, const std::function<void(int, int)>& fn) {
  threads = std::max(1, std::min(threads, n));
  if (threads == 1) { fn(0, n); return; }
  std::vector<std::thread> th;
  const int per = (n + threads - 1) / threads;
  for (int t = 0; t < threads; ++t) {
    const int lo = t * per, hi = std::min(n, lo + per);
    if (lo < hi) th.emplace_back(fn, lo, hi);
  }
  for (auto& x : th) x.join();
}

// y[T, N] = x[T, K] · w[N, K]^T + b
void linear(const float* x, const float* w, const float* b, float* y, int T, int N, int K, int threads) {
  parallel_for(T, threads, [&](int lo, int hi) {
    for (int t = lo; t < hi; ++t)
      for (int n = 0; n < N; ++n) {
        float acc = b ? b[n] : 0.f;
        const float* xr = x + (size_t)t * K;
        const float* wr = w + (size_t)n * K;
        for (int k = 0; k < K; ++k) acc += xr[k] * wr[k];
        y[(size_t)t * N + n] = acc;
      }
  });
}

void layernorm(const float* x, const float* w, const float* b, float* y, int T, int H, float eps, int threads) {
  parallel_for(T, threads, [&](int lo, int hi) {
    for (int t = lo; t < hi; ++t) {
      const float* xr = x + (size_t)t * H;
      float mean = 0.f, var = 0.f;
      for (int i = 0; i < H; ++i) mean += xr[i];
      mean /= H;
      for (int i = 0; i < H; ++i) var += (xr[i] - mean) * (xr[i] - mean);
      const float rstd = 1.f / std::sqrt(var / H + eps);
      for (int i = 0; i < H; ++i) y[(size_t)t * H + i] = (xr[i] - mean) * rstd * w[i] + (b ? b[i] : 0.f);
    }
  });
}

inline float gelu_tanh(float x) { return 0.5f * x * (1.f + std::tanh(0.7978845608f * (x + 0.044715f * x * x * x))); }

}  // namespace

extern "C" void blz_vit_forward_cpu(const float* patches, int T, const BlzVitWeights* w, float* out, int threads) {
  const int H = w->hidden, NH = w->heads, D = H / NH, half = D / 2;
  std::vector<float> x((size_t)T * H), h((size_t)T * H), qkv((size_t)T * 3 * H), att((size_t)T * H), mid((size_t)T * w->mlp);
  linear(patches, w->patch_w, w->patch_b, x.data(), T, H, w->patch_dim, threads);
  if (w->pos) for (size_t i = 0; i < x.size(); ++i) x[i] += w->pos[i];
  const float scale = 1.f / std::sqrt((float)D);
  for (int l = 0; l < w->depth; ++l) {
    const BlzVitBlock& b = w->blocks[l];
    layernorm(x.data(), b.ln1_w, b.ln1_b, h.data(), T, H, w->eps, threads);
    linear(h.data(), b.qkv_w, b.qkv_b, qkv.data(), T, 3 * H, H, threads);
    if (w->rope_cos) {
      parallel_for(T, threads, [&](int lo, int hi) {
        for (int t = lo; t < hi; ++t)
          for (int which = 0; which < 2; ++which)
            for (int hd = 0; hd < NH; ++hd) {
              float* v = &qkv[(size_t)t * 3 * H + which * H + hd * D];
              for (int i = 0; i < half; ++i) {
                const float c = w->rope_cos[(size_t)t * half + i], s = w->rope_sin[(size_t)t * half + i];
                const float a = v[i], bb = v[i + half];
                v[i] = a * c - bb * s;
                v[i + half] = bb * c + a * s;
              }
            }
      });
    }
    parallel_for(T * NH, threads, [&](int lo, int hi) {
      std::vector<float> p(T);
      for (int idx = lo; idx < hi; ++idx) {
        const int t = idx / NH, hd = idx % NH;
        const float* q = &qkv[(size_t)t * 3 * H + hd * D];
        float mx = -INFINITY;
        for (int j = 0; j < T; ++j) {
          const float* k = &qkv[(size_t)j * 3 * H + H + hd * D];
          float s = 0.f;
          for (int i = 0; i < D; ++i) s += q[i] * k[i];
          p[j] = s * scale;
          mx = std::max(mx, p[j]);
        }
        float sum = 0.f;
        for (int j = 0; j < T; ++j) { p[j] = std::exp(p[j] - mx); sum += p[j]; }
        float* o = &att[(size_t)t * H + hd * D];
        for (int i = 0; i < D; ++i) o[i] = 0.f;
        for (int j = 0; j < T; ++j) {
          const float* v = &qkv[(size_t)j * 3 * H + 2 * H + hd * D];
          const float pj = p[j] / sum;
          for (int i = 0; i < D; ++i) o[i] += pj * v[i];
        }
      }
    });
    linear(att.data(), b.proj_w, b.proj_b, h.data(), T, H, H, threads);
    for (size_t i = 0; i < x.size(); ++i) x[i] += h[i];
    layernorm(x.data(), b.ln2_w, b.ln2_b, h.data(), T, H, w->eps, threads);
    linear(h.data(), b.fc1_w, b.fc1_b, mid.data(), T, w->mlp, H, threads);
    for (size_t i = 0; i < mid.size(); ++i) mid[i] = gelu_tanh(mid[i]);
    linear(mid.data(), b.fc2_w, b.fc2_b, h.data(), T, H, w->mlp, threads);
    for (size_t i = 0; i < x.size(); ++i) x[i] += h[i];
  }
  if (w->ln_f_w) layernorm(x.data(), w->ln_f_w, w->ln_f_b, out, T, H, w->eps, threads);
  else memcpy(out, x.data(), x.size() * sizeof(float));
}
