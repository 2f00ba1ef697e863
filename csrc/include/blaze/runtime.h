// C API of the host runtime library (libblaze_runtime.so): safetensors reader, weight repack, page allocator,
// CPU expert oracle, CPU vision tower, log bridge.  Counterparts in the reference: kernels/include/blaze/safetensors.h,
// repack.h, store.h, cpu_expert.h, vision_cpu.h, log.h.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- log bridge: messages from native code reach the Python logger through this callback
typedef void (*blz_log_fn)(int level, const char* msg);
void blz_log_set(blz_log_fn fn);
void blz_log(int level, const char* fmt, ...);

// ---- safetensors directory reader (mmap-free: pread into caller memory, several threads per tensor)
void* blz_st_open(const char* dir, char* err, int err_len);
void blz_st_close(void* h);
int blz_st_count(void* h);
// name / dtype into caller buffers; shape into `shape` (up to 8 dims); returns rank or -1
int blz_st_info(void* h, int index, char* name, int name_len, char* dtype, int dtype_len, int64_t* shape, int64_t* nbytes);
int blz_st_find(void* h, const char* name);
// reads the whole tensor into dst (dst_bytes must equal its size); returns 0 or -errno
int blz_st_read(void* h, int index, void* dst, int64_t dst_bytes, int threads);

// ---- repack
// 1-byte scale matrix [rows, cols] → 128x4 tiles of 512 bytes (byte (r,c) at (r%32)*16 + (r/32)*4 + c inside a tile)
void blz_swizzle_sf(const uint8_t* src, int64_t rows, int64_t cols, uint8_t* dst);
int64_t blz_swizzle_sf_bytes(int64_t rows, int64_t cols);

// ---- page allocator (ref-counted 16-token pages; page 0 reserved)
void* blz_pages_create(int num_pages);
void blz_pages_destroy(void* h);
int blz_pages_free_count(void* h);
int blz_pages_alloc(void* h, int n, int32_t* out);          // 0 ok, -1 not enough pages
void blz_pages_retain(void* h, const int32_t* pages, int n);
int blz_pages_release(void* h, const int32_t* pages, int n);  // -1 when a page is released twice

// ---- CPU expert oracle: y = down(silu(gate(x)) * up(x)) for one NVFP4 expert, fp32 math
// gate_up: packed [2I, K/2] + e4m3 scales [2I, K/16] + per-row alpha [2I]; down: packed [H, I/2] + scales [H, I/16] + alpha [H]
void blz_cpu_expert_nvfp4(const float* x, int rows, int H, int I, const uint8_t* gu_w, const uint8_t* gu_sf, const float* gu_alpha,
                          const uint8_t* dn_w, const uint8_t* dn_sf, const float* dn_alpha, float* y, int threads);

// ---- CPU vision tower (fp32 ViT encoder block stack); see vision_cpu.cpp for the weight struct layout
struct BlzVitWeights;
void blz_vit_forward_cpu(const float* patches, int n_tokens, const struct BlzVitWeights* w, float* out, int threads);

#ifdef __cplusplus
}
#endif
