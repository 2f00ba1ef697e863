// Library-wide host state: status word, TMA descriptor encoder, launch counter.
#include <mutex>

#include "blaze/host.h"

namespace blz {

static int* g_status[64] = {nullptr};
static std::mutex g_mu;

int* status_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status[dev]) {
    cudaMalloc(&g_status[dev], 64 * sizeof(int));
    cudaMemset(g_status[dev], 0, 64 * sizeof(int));
  }
  return g_status[dev];
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encoder() {
  static EncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(p);
  }
  return fn;
}

cudaError_t encode_tmap(CUtensorMap* out, const void* base, int dtype_bytes, uint64_t dim0, uint64_t dim1,
                        uint64_t stride1_bytes, uint32_t box0, uint32_t box1, int swizzle, uint64_t dim2,
                        uint64_t stride2_bytes, uint32_t box2) {
  EncodeTiled fn = encoder();
  if (!fn) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (stride1_bytes & 15)) return cudaErrorInvalidValue;
  CUtensorMapDataType dt = dtype_bytes == 1   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : dtype_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                              : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUtensorMapSwizzle sw = swizzle == 3   ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                                         : CU_TENSOR_MAP_SWIZZLE_NONE;
  cuuint32_t rank = dim2 > 0 ? 3 : 2;
  cuuint64_t dims[3] = {dim0, dim1, dim2 > 0 ? dim2 : 1};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

}  // namespace blz

// Read and clear the status word (0 = no bounded wait ran out since the last call). Synchronises the device.
BLZ_API int blz_status_take() {
  int* d = blz::status_word();
  int h = 0;
  cudaMemcpy(&h, d, sizeof(int), cudaMemcpyDeviceToHost);
  if (h) cudaMemset(d, 0, sizeof(int));
  return h;
}

// Queue a copy of the status word into `host_dst` (pinned host memory) behind the work already on `stream`: the host reads
// it once it has synchronised with the step anyway (when it takes the step's tokens), so watching the word costs no
// synchronisation of its own.
BLZ_API int blz_status_peek_async(int* host_dst, cudaStream_t stream) {
  if (!host_dst) return (int)cudaErrorInvalidValue;
  return (int)cudaMemcpyAsync(host_dst, blz::status_word(), sizeof(int), cudaMemcpyDeviceToHost, stream);
}

BLZ_API void* blz_status_ptr() { return blz::status_word(); }

BLZ_API int blz_version() { return 1; }
