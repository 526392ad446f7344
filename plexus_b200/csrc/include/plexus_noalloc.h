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
//   * Mw, Nw, lda, ldb are multiples of 8, lda >= Mw, ldb >= Nw, R fits in 31 bits; A, B, out are
//     16-byte aligned device pointers.  Violations return PLEXUS_NOALLOC_BAD_ARGUMENT.
//   * The first call on each device looks up the device addresses of the scratch array and of the
//     status words (a host-side symbol is not a device pointer) and caches them.  Make that first
//     call outside any stream capture, with the device that will run the kernels current.  Two host
//     threads that make their first call on the same device at the same time both perform the
//     look-up and store the same two addresses; that is harmless, no lock is taken.
//   * The kernel's internal waits are bounded.  If one ever gives up, the kernel stops without
//     writing its partial sums, `out` is then meaningless, and a record is left in eight status
//     words that also live in the library image.  The launch is asynchronous, so the entry point
//     itself cannot report this: after synchronising the stream, call plexus_noalloc_take_status,
//     which copies the words out and clears them (again without allocating).
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

// Copies the eight status words of the current device to `words` and clears them on the device.
// words[0] == 0: every call since the last take finished its waits.  Otherwise words[0..4] =
// (code, kernel, where, a, b) of the first wait that gave up (code 1 = timeout).  Synchronise the
// streams that ran plexus_gemm_tn_noalloc first.  Returns PLEXUS_NOALLOC_OK, or
// PLEXUS_NOALLOC_CUDA_ERROR if the copy failed.  Allocates nothing.
int plexus_noalloc_take_status(int words[8]);

#ifdef __cplusplus
}
#endif
