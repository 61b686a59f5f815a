// Allocation-free entry point of the kernel library.
//
// This declaration has no counterpart in the reference project; it exists for embedders of this library.
//
// Who needs it: hosts that hand every byte of device memory to their own pool at start-up (an inference server
// that pre-reserves its KV cache and activation arena, a plug-in loaded into another framework's process) and
// latency-critical loops that must never hit the driver's allocator. For such callers a cudaMalloc from inside
// a library call can fail outright (nothing is left outside the pool), and even when it succeeds it takes a
// driver lock and may synchronise the device in the middle of a step. The regular entry point mstar_gemm_bf16
// leaves the split-K scratch to the caller (the Python layer allocates it with torch); this variant needs no
// scratch from anyone: it keeps its own inside the library image.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest scratch the entry point will use. Problems whose split-K plan needs more are refused (return -1,
// message from mstar_last_error()); they are not silently run another way.
#define MSTAR_NOALLOC_WORKSPACE_BYTES (16u << 20)   /* fp32 partial tiles */
#define MSTAR_NOALLOC_MAX_TILES 4096                /* one arrival counter per output tile */

// C[M,N] = A[M,K] * B[N,K]^T, bf16 operands and output, fp32 accumulation, no bias / residual / activation. It is
// the same tcgen05 kernel and tile plan as mstar_gemm_bf16, but the split-K partial sums always meet in the
// scratch array, while the regular entry point may sum them through a thread-block cluster with another split
// factor. The two therefore add the same products in a different order: results agree within bf16 rounding of
// the output, not bit for bit.
//
// Scratch lives in a file-scope device array of MSTAR_NOALLOC_WORKSPACE_BYTES (+ counters); every GPU that loads
// the library carries it until the process exits. The entry point calls no cudaMalloc / cudaFree and no
// allocating library routine.
//
// * The first call on each device looks up the array's device address (cudaGetSymbolAddress) and sets the
//   kernel's shared-memory attribute for that device; make that first call before any CUDA stream capture on
//   that device.
// * Device-side waits in this path are bounded like everywhere in the library, but a wait that runs out is NOT
//   reported: the library's status word lives in allocated memory, which this entry point must not create, so the
//   kernel is given none. After such a timeout the output tile is incomplete and the call still returns 0.
// * All calls share the one array. Two calls that can overlap on the GPU (different streams, or a capture
//   replayed concurrently) race on it: serialise them. The counters are cleared on the stream at every call;
//   the partial-tile area is fully rewritten before it is read, so leftovers of earlier calls are harmless.
// * lda / ldb / ldc are in elements; lda and ldb must be multiples of 8 and A, B 16-byte aligned.
// Returns 0 on success, -1 on error (see mstar_last_error()).
int mstar_gemm_bf16_noalloc(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                            void* stream);

#ifdef __cplusplus
}
#endif
