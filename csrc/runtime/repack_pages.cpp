// Weight repack (scale-factor tiling for the tcgen05 block-scaled MMA) and the ref-counted page allocator.
// Reference: kernels/src/cpu/repack.cpp (NVFP4 expert records → "rg16" layout), crates/blaze/src/engine.rs:1083-1164 (pages).
#include <cstring>
#include <mutex>
#include <vector>

#include "blaze/runtime.h"

extern "C" int64_t blz_swizzle_sf_bytes(int64_t rows, int64_t cols) {
  return ((rows + 127) / 128) * ((cols + 3) / 4) * 512;
}

extern "C" void blz_swizzle_sf(const uint8_t* src, int64_t rows, int64_t cols, uint8_t* dst) {
  const int64_t ct = (cols + 3) / 4;
  memset(dst, 0, (size_t)blz_swizzle_sf_bytes(rows, cols));
  for (int64_t r = 0; r < rows; ++r) {
    const uint8_t* s = src + r * cols;
    uint8_t* tile_row = dst + ((r >> 7) * ct) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4;
    for (int64_t c = 0; c < cols; ++c) tile_row[(c >> 2) * 512 + (c & 3)] = s[c];
  }
}

namespace {
struct Pages {
  std::vector<int32_t> free_list;
  std::vector<int32_t> refs;
  std::mutex mu;
};
}  // namespace

extern "C" void* blz_pages_create(int num_pages) {
  Pages* p = new Pages();
  p->refs.assign(num_pages, 0);
  for (int i = num_pages - 1; i >= 1; --i) p->free_list.push_back(i);
  return p;
}
extern "C" void blz_pages_destroy(void* h) { delete reinterpret_cast<Pages*>(h); }
extern "C" int blz_pages_free_count(void* h) {
  Pages* p = reinterpret_cast<Pages*>(h);
  std::lock_guard<std::mutex> lk(p->mu);
  return (int)p->free_list.size();
}
extern "C" int blz_pages_alloc(void* h, int n, int32_t* out) {
  Pages* p = reinterpret_cast<Pages*>(h);
  std::lock_guard<std::mutex> lk(p->mu);
  if ((int)p->free_list.size() < n) return -1;
  for (int i = 0; i < n; ++i) {
    out[i] = p->free_list.back();
    p->free_list.pop_back();
    p->refs[out[i]] = 1;
  }
  return 0;
}
extern "C" void blz_pages_retain(void* h, const int32_t* pages, int n) {
  Pages* p = reinterpret_cast<Pages*>(h);
  std::lock_guard<std::mutex> lk(p->mu);
  for (int i = 0; i < n; ++i) p->refs[pages[i]]++;
}
extern "C" int blz_pages_release(void* h, const int32_t* pages, int n) {
  Pages* p = reinterpret_cast<Pages*>(h);
  std::lock_guard<std::mutex> lk(p->mu);
  int rc = 0;
  for (int i = 0; i < n; ++i) {
    int32_t& r = p->refs[pages[i]];
    if (r <= 0) { rc = -1; continue; }
    if (--r == 0) p->free_list.push_back(pages[i]);
  }
  return rc;
}
