// Split-KV decode attention with built-in scratch: an entry point that allocates nothing.
//
// This entry point has no counterpart in the reference; it exists for callers that must not allocate
// device memory at all (embedding in another runtime, fixed-memory deployments).
//
// `bonsai_attn_decode` takes three caller-owned scratch buffers (partial accumulators, partial
// max/sum pairs, arrival counters).  `bonsai_attn_decode_static` computes the same result with the
// same kernel but takes none: its scratch lives in one file-scope `static __device__` array of
// fixed size inside the library image, one instance per device.  The entry point never calls
// cudaMalloc, cudaFree or any allocating library routine; the only runtime calls it makes are
// cudaGetDevice, cudaGetSymbolAddress (once per device, result cached), cudaMemsetAsync and the
// kernel launch.
//
// Limits (BONSAI_ATTN_STATIC_* below).  A call is rejected with BONSAI_CUDA_BAD_ARG and a message
// in `err` when
//     batch * nq * nsplit * hd  >  BONSAI_ATTN_STATIC_MAX_ACC_FLOATS   (1 Mi floats = 4 MiB), or
//     batch * nq * nsplit * 2   >  BONSAI_ATTN_STATIC_MAX_ML_FLOATS    (32 Ki floats = 128 KiB), or
//     batch * nkv               >  BONSAI_ATTN_STATIC_MAX_COUNTERS     (4096).
// The max/sum area is sized for the accumulator limit at head dimension 64, the smallest the kernel
// behind this entry accepts, so its limit only binds for head dimensions the kernel rejects anyway.
//
// Rules for callers:
//  * The scratch array is shared by every call on a device.  Two calls whose kernels may overlap
//    (different streams, or different host threads on different streams) race on it; issue all
//    calls for one device on one stream, or order them with events.
//  * The arrival counters must be zero when the kernel starts.  The array is zero at module load
//    and the kernel leaves the counters at zero, and in addition every call clears the counters
//    it is about to use with a cudaMemsetAsync on `stream` ahead of the launch, so a call that
//    follows a failed or aborted launch still starts clean.  The other two areas need no clearing.
//  * The first call on each device resolves the symbol address, which may load the module; make
//    that first call outside any stream capture.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#define BONSAI_ATTN_STATIC_MAX_ACC_FLOATS (1u << 20)
#define BONSAI_ATTN_STATIC_MAX_ML_FLOATS (1u << 15)
#define BONSAI_ATTN_STATIC_MAX_COUNTERS 4096u

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as for bonsai_attn_decode minus the three scratch pointers.  `err` (capacity `err_cap`,
// may be null) receives a NUL-terminated description when the return value is negative.
int bonsai_attn_decode_static(const float* q, const int* positions, const int* block_table, int max_pages, int batch, int nq,
                              int nkv, int hd, int kvt, int page_size, const void* kpool, const void* vpool,
                              const float* kscale, const float* vscale, int nsplit, float* out, int extra_len,
                              cudaStream_t stream, char* err, size_t err_cap);

#ifdef __cplusplus
}
#endif
