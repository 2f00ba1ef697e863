// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference: there the host always owns and passes every buffer
// (kernels/include/blaze/*.h take raw pointers for scratch as well).
//
// Who needs it: code that runs where cudaMalloc is forbidden or would deadlock — inside a CUDA-graph capture that was
// started by someone else, inside a stream callback / host function, in a process whose memory pool is owned by another
// runtime and must not grow, or in a latency-critical path that may not take the allocator lock.  The split-KV variant of
// the paged decode attention needs scratch for its per-split partial outputs; `blz_attn_decode` takes that scratch from
// the caller, this variant keeps it inside the library instead.
//
// How: the partial outputs and (max, sum) pairs live in ONE file-scope `static __device__ __align__(256)` array of
// BLZ_ATTN_NOALLOC_SCRATCH_BYTES (16.5 MiB); every GPU that loads the library holds it until the process exits.
// The first call on a device (under a lock, so threads may race to it) looks the array's device address up
// (cudaGetSymbolAddress) and sets the kernel's shared-memory limit for that device; make that first call outside of any
// stream capture.  Later calls on that device only launch.
// The function never calls cudaMalloc / cudaFree or any allocating library routine.
//
// Limits: seqs * kv_heads * row_blocks * splits * 16 rows of 130 floats must fit the array, and row_blocks * 16 must cover
// max_rows; otherwise the call returns cudaErrorInvalidValue and `blz_attn_decode_noalloc_error()` explains what was too large.  All calls share the array:
// it keeps the last call's contents (nothing in it has to start at zero — every slot that is read is written first by
// the same call), and two calls that overlap on the GPU (different streams, or concurrent graphs) race on it.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BLZ_ATTN_NOALLOC_SCRATCH_BYTES (16u * 1024u * 1024u + 512u * 1024u)

// Same arguments and result as blz_attn_decode with nmax = 16, minus the scratch pointers.  page_stride / head_stride:
// bytes between the [2, 16*D] blocks of consecutive pages / kv heads in the pool (0 = page-major [pages, Hkv, 2, 16*D]).
int blz_attn_decode_noalloc(const void* q, void* out, const void* pool, const int* block_table, const int* slots,
                            const int* q_start, const int* ctx_len, int num_seqs, int Hq, int Hkv, int D, int bt_stride,
                            long long page_stride, long long head_stride, float scale, float k_scale, float v_scale, int row_blocks, int min_rows, int max_rows, int splits,
                            int max_ctas, cudaStream_t stream);

// The kernels' waits are bounded; one that runs out records 1 in a status word inside the library instead of hanging, and
// the call's output is then not valid.  This reads and clears that word for the current device (0 = fine, -1 = no call was
// made on this device yet).  It synchronises the device, so call it between steps, not per launch.  Allocates nothing.
int blz_attn_decode_noalloc_status(void);

// Text of the last size / set-up error of this thread ("" when the last call succeeded).
const char* blz_attn_decode_noalloc_error(void);

// Bytes of scratch the given problem needs (to check against BLZ_ATTN_NOALLOC_SCRATCH_BYTES beforehand).
long long blz_attn_decode_noalloc_bytes(int num_seqs, int Hkv, int row_blocks, int splits);

#ifdef __cplusplus
}
#endif
