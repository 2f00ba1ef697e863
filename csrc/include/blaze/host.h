// Host-side helpers shared by the kernel launchers: error plumbing, TMA descriptor encoding
// (driver entry point fetched through the runtime, so nothing links against libcuda), the global
// status word that bounded device waits report into.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define BLZ_API extern "C" __attribute__((visibility("default")))

namespace blz {

// returns the device pointer of this device's status word (allocated on first use)
int* status_word();

// Encode a 2-D (or 3-D when dim2 > 0) tiled tensor map. `dtype_bytes`: 1 → UINT8, 2 → BFLOAT16, 4 → FLOAT32.
// `swizzle`: 0 none, 1 32B, 2 64B, 3 128B.
cudaError_t encode_tmap(CUtensorMap* out, const void* base, int dtype_bytes, uint64_t dim0, uint64_t dim1,
                        uint64_t stride1_bytes, uint32_t box0, uint32_t box1, int swizzle, uint64_t dim2 = 0,
                        uint64_t stride2_bytes = 0, uint32_t box2 = 1);

// BLAZE_PDL=0 turns programmatic dependent launch off (every kernel then starts after its predecessor has finished).
inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("BLAZE_PDL");
    on = (e && e[0] == '1') ? 1 : 0;
  }
  return on != 0;
}

// Launch a kernel that follows the pdl_trigger / pdl_wait protocol (sm100.cuh) so that its prologue — and, for the
// GEMMs, the first weight tiles — overlap the tail of the kernel before it on the stream.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// SM count of the current device (cached per device: a process may drive several GPUs).
inline int sm_count() {
  static int n[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!n[dev]) {
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    n[dev] = v;
  }
  return n[dev];
}

// cudaFuncSetAttribute applies to the current device only: remember per device whether a kernel has been configured.
// One instance per kernel instantiation (a function-local static of the launcher).
struct PerDeviceOnce {
  bool done[64] = {false};
  // Sets the dynamic shared-memory limit of `kernel` on the current device the first time it is launched there.
  template <typename K>
  cudaError_t smem_limit(K kernel, int bytes) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done[dev] = true;   // idempotent: two threads racing here both set the same value
    return e;
  }
};

}  // namespace blz
