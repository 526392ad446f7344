// Allocation-free entry point (C ABI).  It has no counterpart in the reference, whose GEMMs go
// through torch.mm and allocate freely.
//
// Who needs it: code that hosts this library but may not allocate device memory while it runs.
// Examples are a serving process whose whole device-memory budget is fixed at start-up, a plugin
// called from inside another framework's memory-planned step (its allocator must not be re-entered
// and cudaMalloc would synchronise the device), and signal-safe / real-time control loops.  Such
// callers cannot use the regular weight-gradient GEMM because its split reduction needs a scratch
// buffer that the caller would have to allocate per shape.
//
// plexus_gemm_tn_noalloc computes   out[Mw, Nw] (fp32) = A[R, Mw]^T . B[R, Nw]   (A, B bf16,
// row-major, leading dimensions lda / ldb in elements) with the same tcgen05 kernel and the same
// deterministic two-stage reduction as the regular path, but keeps the per-CTA partial sums in a
// fixed array that lives in the library image: PLEXUS_NOALLOC_SCRATCH_FLOATS floats (16 MiB) on
// every GPU that loads the library, held until the process exits.  The caller passes only inputs
// and the output.  The call performs no cudaMalloc / cudaFree and calls no allocating library
// routine.
//
// Limits and rules
//   * plexus_gemm_tn_noalloc_parts(R) * Mw * Nw must not exceed PLEXUS_NOALLOC_SCRATCH_FLOATS;
//     larger problems are rejected with PLEXUS_NOALLOC_TOO_LARGE and a message, nothing is launched.
//   * Mw, Nw, lda, ldb are multiples of 8; A, B, out are 16-byte aligned device pointers.
//   * The first call on each device looks up the device address of the scratch array (a host-side
//     symbol is not a device pointer) and caches it.  Make that first call outside any stream
//     capture, with the device that will run the kernels current.
//   * All calls share the one array, which keeps the previous call's partial sums.  Nothing has to
//     start at zero (every partial that is read is written first by the same call), but two calls
//     whose kernels overlap on the GPU (different streams) race on the array: serialise them.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PLEXUS_NOALLOC_SCRATCH_FLOATS (4u * 1024u * 1024u)

enum {
  PLEXUS_NOALLOC_OK = 0,
  PLEXUS_NOALLOC_BAD_ARGUMENT = 1,
  PLEXUS_NOALLOC_TOO_LARGE = 2,
  PLEXUS_NOALLOC_CUDA_ERROR = 3,
};

// Number of partial results the split reduction produces for R reduction rows.
int plexus_gemm_tn_noalloc_parts(int64_t R);

// stream: a cudaStream_t (may be null for the default stream).
// err / err_len: optional caller-provided buffer that receives a message on failure.
// Returns PLEXUS_NOALLOC_OK or one of the codes above.
int plexus_gemm_tn_noalloc(const void* A, int64_t lda, const void* B, int64_t ldb, float* out,
                           int64_t R, int64_t Mw, int64_t Nw, void* stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
