// pg_gemm_bf16_tn_noalloc: the bf16 GEMM for callers that must not allocate.
//
// This entry point has no counterpart in the reference engine.
//
// Who needs it: code that runs where device allocation is off limits -- a plugin
// called from inside another runtime's stream callback or allocator hook, a host
// whose memory pool is frozen after start-up (all HBM already handed to weights and
// the KV cache), or an embedder that forbids cudaMalloc/cudaFree on its serving
// threads because those calls synchronise the whole device.  pg_gemm_bf16_tn asks its
// caller for a split-K workspace and tile counters; such a caller has nowhere to get
// them from.  Here that scratch lives in a fixed array inside the library image
// instead, so the call needs only the operands and the output.
//
// Limits and rules:
//  * The scratch is PG_NOALLOC_SCRATCH_BYTES (8 MiB) of device memory per GPU that
//    loads the library, held until the process exits.  The first PG_NOALLOC_COUNTER_BYTES
//    hold one counter per output tile, so a problem may have at most
//    PG_NOALLOC_MAX_TILES (16384) output tiles (tile = 128 weight rows x one token
//    tile); larger problems are refused with PG_ERR_INVALID and a message.  The rest
//    holds split-K partial sums; when it is too small for the preferred split count the
//    kernel runs with fewer splits (same result up to f32 summation order).
//  * The first call on a device looks up the scratch address (cudaGetSymbolAddress, with
//    that device current).  Make that first call outside any stream capture.
//  * All calls on a device share the one array, and it keeps whatever the previous call
//    left there.  Each call clears the counters it needs on `stream` before launching.
//    Two calls that overlap on the GPU (different streams, or graphs replayed
//    concurrently) race on it: serialise them.
//  * Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define PG_NOALLOC_SCRATCH_BYTES (8 << 20)
#define PG_NOALLOC_COUNTER_BYTES (64 << 10)
#define PG_NOALLOC_MAX_TILES (PG_NOALLOC_COUNTER_BYTES / 4)

#ifdef __cplusplus
extern "C" {
#endif

// y[T, M] (bf16, row stride ldy) = x[T, K] (bf16, row stride ldx) * w[M, K]^T (bf16, row
// stride ldw), f32 accumulation.  `status` is a caller-owned device uint32 that the
// kernel sets if a bounded wait expires (0 = clean).  Returns 0 or a negative PG_ERR_*
// code; pg_last_error() has the message.
int pg_gemm_bf16_tn_noalloc(const void* x, const void* w, void* y, int T, int M, int K, long long ldx, long long ldw, long long ldy,
                            void* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
