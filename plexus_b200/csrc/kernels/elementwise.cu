// Small elementwise kernels: ReLU derivative, weight preparation (fp32 -> bf16 and its
// transpose in one pass), dtype casts, and the bounded flag wait used by the fault tests.
//
// Reference sites: the ReLU between layers and its autograd derivative (examples/train.py:78) and
// the operand re-layout copies of the GEMM tuner (plexus/utils/matmul_tuning.py:30-51), which
// prep_weight replaces by one cast + transpose of the small operand.

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "../include/plexus_kernels.h"
#include "../include/ptx_sm100.cuh"

namespace plx {

__device__ __forceinline__ float as_float(float v) { return v; }
__device__ __forceinline__ float as_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T zero_of();
template <>
__device__ __forceinline__ float zero_of<float>() { return 0.f; }
template <>
__device__ __forceinline__ __nv_bfloat16 zero_of<__nv_bfloat16>() { return __float2bfloat16_rn(0.f); }

// grad_in = grad * (out > 0), 8 bf16 (or 4 fp32) per thread.
template <typename T>
__global__ void relu_bwd_kernel(const T* __restrict__ g, const T* __restrict__ y, T* __restrict__ o,
                                int64_t n) {
  constexpr int VN = 16 / sizeof(T);
  const int64_t nv = n / VN;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    uint4 gv = reinterpret_cast<const uint4*>(g)[i];
    const uint4 yv = reinterpret_cast<const uint4*>(y)[i];
    T* gp = reinterpret_cast<T*>(&gv);
    const T* yp = reinterpret_cast<const T*>(&yv);
#pragma unroll
    for (int k = 0; k < VN; ++k)
      if (!(as_float(yp[k]) > 0.f)) gp[k] = zero_of<T>();
    reinterpret_cast<uint4*>(o)[i] = gv;
  }
  const int64_t tail = nv * VN + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (tail < n) o[tail] = as_float(y[tail]) > 0.f ? g[tail] : zero_of<T>();
}

const char* launch_relu_bwd(int dtype, const void* grad, const void* out, void* res, int64_t n,
                            cudaStream_t stream) {
  if (n == 0) return nullptr;
  const int blocks = static_cast<int>(std::min<int64_t>(148 * 16, (n / 8 + 255) / 256 + 1));
  if (dtype == DT_BF16)
    relu_bwd_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(grad),
                                                reinterpret_cast<const __nv_bfloat16*>(out),
                                                reinterpret_cast<__nv_bfloat16*>(res), n);
  else
    relu_bwd_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(grad),
                                                reinterpret_cast<const float*>(out),
                                                reinterpret_cast<float*>(res), n);
  return last_launch_error();
}

// W fp32/bf16 [K, N]  ->  Wb bf16 [K, N] and WbT bf16 [N, K]
template <typename T>
__global__ void prep_weight_kernel(const T* __restrict__ W, __nv_bfloat16* __restrict__ Wb,
                                   __nv_bfloat16* __restrict__ WbT, int K, int N) {
  __shared__ float tile[32][33];
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int k = k0 + r, n = n0 + threadIdx.x;
    float v = 0.f;
    if (k < K && n < N) {
      v = as_float(W[static_cast<int64_t>(k) * N + n]);
      if (Wb != nullptr) Wb[static_cast<int64_t>(k) * N + n] = __float2bfloat16_rn(v);
    }
    tile[r][threadIdx.x] = v;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < K) WbT[static_cast<int64_t>(n) * K + k] = __float2bfloat16_rn(tile[threadIdx.x][r]);
  }
}

const char* launch_prep_weight(int dtype, const void* W, void* Wb, void* WbT, int K, int N,
                               cudaStream_t stream) {
  if (K == 0 || N == 0) return nullptr;
  dim3 grid((N + 31) / 32, (K + 31) / 32), block(32, 8);
  if (dtype == DT_F32)
    prep_weight_kernel<<<grid, block, 0, stream>>>(reinterpret_cast<const float*>(W),
                                                   reinterpret_cast<__nv_bfloat16*>(Wb),
                                                   reinterpret_cast<__nv_bfloat16*>(WbT), K, N);
  else
    prep_weight_kernel<<<grid, block, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(W),
                                                   reinterpret_cast<__nv_bfloat16*>(Wb),
                                                   reinterpret_cast<__nv_bfloat16*>(WbT), K, N);
  return last_launch_error();
}

// Poll a flag until it reaches `expected`, at most `max_polls` times; on expiry record a
// TIMEOUT status and return normally.  Used to check that a wait on a peer that never
// signals ends in a status word instead of a hang.
__global__ void wait_flag_kernel(const volatile int* flag, int expected, unsigned max_polls,
                                 int* status) {
  unsigned i = 0;
  int seen = *flag;
  while (seen < expected && i < max_polls) {
    __nanosleep(200);
    seen = *flag;
    ++i;
  }
  if (seen < expected) report_status(status, ST_TIMEOUT, 7, 0, expected, seen);
}

const char* launch_wait_flag(const int* flag, int expected, unsigned max_polls, int* status,
                             cudaStream_t stream) {
  wait_flag_kernel<<<1, 1, 0, stream>>>(flag, expected, max_polls, status);
  return last_launch_error();
}

}  // namespace plx
