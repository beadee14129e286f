/* Split-K GEMM entry point that allocates nothing.
 *
 * This entry point has no counterpart in the reference library: it exists for
 * callers of this library that are not in a position to allocate device memory
 * at the time they need a GEMM:
 *   - a serving engine that handed the whole device to its own memory pool at
 *     start-up, so that a cudaMalloc from inside a library call would fail or
 *     take memory the engine has promised to its KV cache;
 *   - code on a latency-critical path (a decode step), where the device-wide
 *     synchronisation that cudaMalloc / cudaFree may imply is not acceptable;
 *   - a plug-in whose host framework forbids allocation inside its compute
 *     callbacks.
 * oob_gemm() with splits > 1 keeps its fp32 partial tiles in a workspace that
 * the library allocates (and grows) with cudaMalloc.  The function below runs
 * the same kernel, but the workspace is a fixed array that is part of the
 * library image: every GPU that loads the library holds it until the process
 * exits (OOB_SPLITK_STATIC_BYTES, about 16 MiB).
 *
 * Contract
 *   C[M, N] = A[M, K] * B[N, K]^T, 16-bit inputs (dtype OOB_F16 or OOB_BF16),
 *   fp32 accumulation, `splits` >= 1 slices of K per 128x256 output tile
 *   (a value that would leave a slice empty is lowered).  The caller passes
 *   inputs and output; nothing else is needed.
 *   - No cudaMalloc, cudaFree or other allocating routine is called, on any
 *     call.  The first call on a device looks up the device address of the
 *     array and raises the kernel's shared-memory limit; make that first call
 *     before any stream capture.
 *   - A problem whose partial tiles do not fit the array
 *     (ceil(M/128) * ceil(N/256) * splits * 128 KiB > capacity) is rejected
 *     with OOB_ERR_NOMEM and a message from oob_last_error(); nothing runs.
 *   - All calls on a device share the one array.  Each call first clears the
 *     arrival counters it uses and overwrites the partial tiles it needs, so
 *     calls issued one after the other on a stream are independent; calls that
 *     overlap on the GPU (different streams, no ordering between them) race on
 *     the array and give wrong results.
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#pragma GCC visibility push(default)

/* Capacity of the built-in array for fp32 partial tiles, in bytes. */
#define OOB_SPLITK_STATIC_BYTES (16ull << 20)

int oob_gemm_splitk_static(int dtype, int M, int N, int K, const void* A, int lda, const void* B, int ldb, void* C,
                           int ldc, int splits, int max_ctas, void* stream);

/* Partial-tile bytes a problem needs (compare with OOB_SPLITK_STATIC_BYTES). */
uint64_t oob_gemm_splitk_static_need(int M, int N, int K, int splits);

#pragma GCC visibility pop
#ifdef __cplusplus
}
#endif
