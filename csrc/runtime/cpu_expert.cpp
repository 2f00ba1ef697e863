// CPU oracle of one NVFP4 expert (gate_up → SwiGLU → down) in fp32: the reference result for the grouped tcgen05
// GEMM path.  Rows are spread over threads; the inner loops vectorise (AVX2 / FMA flags in the build).
// Reference: kernels/src/cpu/cpu_engine.cpp (worker threads, :425), kernels/src/cpu/expert_avx2.cpp expert_forward :262.
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

#include "blaze/runtime.h"

namespace {
const float kE2M1[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

float e4m3_to_float(uint8_t b) {
  const int sign = b >> 7, exp = (b >> 3) & 15, man = b & 7;
  float v;
  if (exp == 0) v = std::ldexp((float)man, -9);
  else if (exp == 15 && man == 7) v = NAN;
  else v = std::ldexp(1.f + man / 8.f, exp - 7);
  return sign ? -v : v;
}

// w row n of a [N, K] NVFP4 matrix → fp32
void dequant_row(const uint8_t* w, const uint8_t* sf, float alpha, int K, float* out) {
  for (int b = 0; b < K / 16; ++b) {
    const float s = e4m3_to_float(sf[b]) * alpha;
    for (int j = 0; j < 8; ++j) {
      const uint8_t byte = w[b * 8 + j];
      out[b * 16 + 2 * j] = kE2M1[byte & 15] * s;
      out[b * 16 + 2 * j + 1] = kE2M1[byte >> 4] * s;
    }
  }
}
}  // namespace

extern "C" void blz_cpu_expert_nvfp4(const float* x, int rows, int H, int I, const uint8_t* gu_w, const uint8_t* gu_sf,
                                     const float* gu_alpha, const uint8_t* dn_w, const uint8_t* dn_sf, const float* dn_alpha,
                                     float* y, int threads) {
  std::vector<float> Wgu((size_t)2 * I * H), Wdn((size_t)H * I);
  for (int n = 0; n < 2 * I; ++n) dequant_row(gu_w + (size_t)n * (H / 2), gu_sf + (size_t)n * (H / 16), gu_alpha[n], H, &Wgu[(size_t)n * H]);
  for (int n = 0; n < H; ++n) dequant_row(dn_w + (size_t)n * (I / 2), dn_sf + (size_t)n * (I / 16), dn_alpha[n], I, &Wdn[(size_t)n * I]);
  threads = threads < 1 ? 1 : (threads > rows ? (rows > 0 ? rows : 1) : threads);
  auto work = [&](int lo, int hi) {
    std::vector<float> act(I);
    for (int r = lo; r < hi; ++r) {
      const float* xr = x + (size_t)r * H;
      for (int i = 0; i < I; ++i) {
        float g = 0.f, u = 0.f;
        const float* wg = &Wgu[(size_t)i * H];
        const float* wu = &Wgu[(size_t)(I + i) * H];
        for (int k = 0; k < H; ++k) { g += xr[k] * wg[k]; u += xr[k] * wu[k]; }
        act[i] = g / (1.f + std::exp(-g)) * u;
      }
      float* yr = y + (size_t)r * H;
      for (int n = 0; n < H; ++n) {
        float acc = 0.f;
        const float* wd = &Wdn[(size_t)n * I];
        for (int i = 0; i < I; ++i) acc += act[i] * wd[i];
        yr[n] = acc;
      }
    }
  };
  std::vector<std::thread> th;
  const int per = (rows + threads - 1) / threads;
  for (int t = 0; t < threads; ++t) {
    const int lo = t * per, hi = std::min(rows, lo + per);
    if (lo < hi) th.emplace_back(work, lo, hi);
  }
  for (auto& t : th) t.join();
}
