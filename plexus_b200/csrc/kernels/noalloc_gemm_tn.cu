// plexus_gemm_tn_noalloc: the weight-gradient GEMM with its split-reduction scratch in a static
// device array instead of caller-allocated memory.  See include/plexus_noalloc.h for who needs
// this and the rules of use.

#include <cuda_runtime.h>

#include <climits>
#include <cstdio>
#include <cstring>

#include "../include/plexus_kernels.h"
#include "../include/plexus_noalloc.h"

namespace {

// Partial sums of the split reduction.  Lives in the library image on every device.
static __device__ __align__(256) float g_noalloc_scratch[PLEXUS_NOALLOC_SCRATCH_FLOATS];

// Status words of the kernels launched through this entry point (see plexus_noalloc_take_status).
static __device__ int g_noalloc_status[8];

constexpr int kMaxDevices = 64;
// Device address of g_noalloc_scratch per device.  The array's name is only a host-side handle;
// kernels must be given the address cudaGetSymbolAddress reports for the current device.
// Concurrent first calls on one device store the same values; no lock is needed.
float* g_scratch_ptr[kMaxDevices] = {nullptr};
int* g_status_ptr[kMaxDevices] = {nullptr};

int fail(int code, const char* msg, char* err, int err_len) {
  if (err != nullptr && err_len > 0) {
    std::strncpy(err, msg, static_cast<size_t>(err_len) - 1);
    err[err_len - 1] = '\0';
  }
  return code;
}

}  // namespace

extern "C" int plexus_gemm_tn_noalloc_parts(int64_t R) { return plx::gemm_tn_parts(R); }

extern "C" int plexus_gemm_tn_noalloc(const void* A, int64_t lda, const void* B, int64_t ldb,
                                      float* out, int64_t R, int64_t Mw, int64_t Nw, void* stream,
                                      char* err, int err_len) {
  if (A == nullptr || B == nullptr || out == nullptr || R < 0 || Mw <= 0 || Nw <= 0)
    return fail(PLEXUS_NOALLOC_BAD_ARGUMENT, "null pointer or non-positive size", err, err_len);
  if (R > INT_MAX || Mw > INT_MAX || Nw > INT_MAX)
    return fail(PLEXUS_NOALLOC_BAD_ARGUMENT, "R, Mw and Nw must fit in 31 bits", err, err_len);
  if (lda < Mw || ldb < Nw)
    return fail(PLEXUS_NOALLOC_BAD_ARGUMENT, "leading dimensions must be at least the row widths (lda >= Mw, ldb >= Nw)",
                err, err_len);
  const int64_t need = static_cast<int64_t>(plx::gemm_tn_parts(R)) * Mw * Nw;
  if (need > static_cast<int64_t>(PLEXUS_NOALLOC_SCRATCH_FLOATS)) {
    char msg[200];
    std::snprintf(msg, sizeof(msg),
                  "problem needs %lld scratch floats (parts * Mw * Nw) but the built-in scratch "
                  "holds %u; use the allocating entry point",
                  static_cast<long long>(need), PLEXUS_NOALLOC_SCRATCH_FLOATS);
    return fail(PLEXUS_NOALLOC_TOO_LARGE, msg, err, err_len);
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(PLEXUS_NOALLOC_CUDA_ERROR, "cannot identify the current device", err, err_len);
  if (g_scratch_ptr[dev] == nullptr || g_status_ptr[dev] == nullptr) {
    // one-time set-up for this device (do it outside stream capture)
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(PLEXUS_NOALLOC_CUDA_ERROR, cudaGetErrorString(e), err, err_len);
    int* st = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&st), g_noalloc_status);
    if (e != cudaSuccess || st == nullptr)
      return fail(PLEXUS_NOALLOC_CUDA_ERROR, cudaGetErrorString(e), err, err_len);
    g_status_ptr[dev] = st;
    g_scratch_ptr[dev] = p;
  }
  const char* msg = plx::launch_gemm_tn(A, lda, B, ldb, out, g_scratch_ptr[dev],
                                        static_cast<int64_t>(PLEXUS_NOALLOC_SCRATCH_FLOATS), R, Mw, Nw,
                                        g_status_ptr[dev], static_cast<cudaStream_t>(stream));
  if (msg != nullptr) return fail(PLEXUS_NOALLOC_BAD_ARGUMENT, msg, err, err_len);
  return PLEXUS_NOALLOC_OK;
}

extern "C" int plexus_noalloc_take_status(int words[8]) {
  if (words == nullptr) return PLEXUS_NOALLOC_BAD_ARGUMENT;
  static const int zeros[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(words, g_noalloc_status, sizeof(int) * 8) != cudaSuccess)
    return PLEXUS_NOALLOC_CUDA_ERROR;
  if (words[0] != 0 && cudaMemcpyToSymbol(g_noalloc_status, zeros, sizeof(int) * 8) != cudaSuccess)
    return PLEXUS_NOALLOC_CUDA_ERROR;
  return PLEXUS_NOALLOC_OK;
}
