// ug_gemm_noalloc: a GEMM entry point that never allocates.
//
// This entry point has no counterpart in the reference; it exists for callers of this
// library that are not allowed to obtain device memory while they enqueue work:
//   * plug-in / custom-op callbacks of an inference runtime, which are handed every
//     buffer they may touch and must not call the allocator from inside the callback;
//   * processes in which another memory manager has already reserved the whole GPU, so a
//     cudaMalloc would fail (or only succeed after that manager gives memory back);
//   * latency-critical loops that cannot afford the implicit device-wide synchronisation
//     cudaMalloc / cudaFree may perform.
//
// It computes   C = A @ B   or   C += A @ B   (A: [m, k] bf16, B: [k, n] bf16, row-major
// with arbitrary row pitches, C: [m, n] fp32 or bf16) with the same persistent tcgen05 kernel
// as ug_fused_gemm.  Everything that kernel needs besides the caller's A, B and C - the TMA
// descriptors, the task / segment / piece tables, the chunk counters and the staging area for
// operands whose address or pitch does not meet the TMA alignment rules - lives in ONE
// file-scope `static __device__` array of UG_NOALLOC_SCRATCH_BYTES bytes.  Every GPU that
// loads the library holds that array until the process exits.
//
// Rules for the caller:
//   * Sizes: the staged copies of misaligned operands (A: m x roundup(k, 64) bf16,
//     B: k x roundup(n, 64) bf16, each rounded up to 1 KiB) must fit in
//     UG_NOALLOC_STAGING_BYTES, there may be at most UG_NOALLOC_MAX_FLAGS row / column
//     chunks and UG_NOALLOC_MAX_PIECES copy pieces.  Larger problems are rejected with
//     UG_NOALLOC_ERR_TOO_LARGE and a message on stderr; nothing is launched.
//   * The first call on a device looks up the device address of the array
//     (cudaGetSymbolAddress) and raises the kernel's shared-memory limit.  Make that first
//     call before any stream capture begins on that device.
//   * All calls share the one array, and it keeps the contents of the previous call; the entry
//     point rewrites the tables and clears the counters on `stream` before each launch.  Two
//     calls whose GPU work overlaps (different streams, or different host threads on the same
//     device) therefore race on the array: serialise them on one stream.
//   * The table upload uses cudaMemcpyAsync from ordinary host memory, which may wait for
//     earlier work of `stream`; no cudaMalloc, cudaFree or other allocating routine is called.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define UG_NOALLOC_SCRATCH_BYTES (8u << 20)                 // the whole static array
#define UG_NOALLOC_STAGING_OFFSET (256u << 10)              // tables live below, staging above
#define UG_NOALLOC_STAGING_BYTES (UG_NOALLOC_SCRATCH_BYTES - UG_NOALLOC_STAGING_OFFSET)
#define UG_NOALLOC_MAX_FLAGS 1024
#define UG_NOALLOC_MAX_PIECES 4096

#define UG_NOALLOC_ERR_INVALID (-1)     // bad pointer, pitch, extent, dtype or mode
#define UG_NOALLOC_ERR_TOO_LARGE (-2)   // the problem needs more scratch than the static array has
#define UG_NOALLOC_ERR_SETUP (-3)       // per-device set-up failed (symbol lookup, TMA descriptor)

// c_dtype: 0 fp32, 1 bf16.  c_mode: 0  C += A @ B,  2  C = A @ B.
// status_ptr: optional device address of a uint32 that receives a non-zero UG_ERR_* code if a wait
// inside the kernel times out (0: use a word inside the static array).
// Returns 0, one of the UG_NOALLOC_ERR_* codes above, or a positive cudaError_t of a failed call.
int ug_gemm_noalloc(uint64_t a, int64_t lda, uint64_t b, int64_t ldb, uint64_t c, int64_t ldc, int32_t m,
                    int32_t n, int32_t k, int32_t c_dtype, int32_t c_mode, uint64_t status_ptr, void* stream);

#ifdef __cplusplus
}
#endif
