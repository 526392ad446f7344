// Class-sharded softmax cross-entropy on logits [R, C] (bf16 or fp32), fp32 math.
//
//   xent_stats : per row (max, sum exp(l - max)) over this rank's valid classes
//   xent_loss  : sum over valid rows of -(l[target] - gmax - log gsum) for targets that fall in
//                this rank's class range, accumulated into one fp32 scalar
//   xent_grad  : (exp(l - gmax)/gsum - onehot) * scale on valid rows, 0 elsewhere
//
// A row is handled by a group of LPR lanes reading 16-byte vectors, several rows per warp, so
// narrow class shards (C = 8..64) keep the loads coalesced.  Neither a softmax nor a one-hot
// matrix is stored; logits and targets are never modified.
//
// Reference: plexus/cross_entropy.py:35-101 (about 15 ATen kernels, int64 one-hot) and :108-114.

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "../include/plexus_kernels.h"

namespace plx {

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

constexpr int XENT_THREADS = 256;

__device__ __forceinline__ int lanes_per_row(int C) {
  int l = 1;
  while (l < 32 && l * 8 < C) l <<= 1;
  return l;
}

template <typename T>
__global__ void xent_stats_kernel(const T* __restrict__ logits, int64_t ld, int R, int C,
                                  int class_offset, int num_classes, float* __restrict__ rmax,
                                  float* __restrict__ rsum) {
  const int lpr = lanes_per_row(C);
  const int rows_per_block = XENT_THREADS / lpr;
  const int li = threadIdx.x % lpr;
  for (int row = blockIdx.x * rows_per_block + threadIdx.x / lpr; row - threadIdx.x / lpr < R;
       row += gridDim.x * rows_per_block) {
    const bool live = row < R;
    float m = -INFINITY;
    if (live)
      for (int c = li; c < C; c += lpr)
        if (c + class_offset < num_classes) m = fmaxf(m, to_f(logits[row * ld + c]));
    for (int off = 1; off < lpr; off <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    const float ms = isinf(m) ? 0.f : m;
    float s = 0.f;
    if (live)
      for (int c = li; c < C; c += lpr)
        if (c + class_offset < num_classes) s += __expf(to_f(logits[row * ld + c]) - ms);
    for (int off = 1; off < lpr; off <<= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (live && li == 0) {
      rmax[row] = m;
      rsum[row] = s;
    }
  }
}

template <typename T>
__global__ void xent_loss_kernel(const T* __restrict__ logits, int64_t ld, const int64_t* __restrict__ target,
                                 const float* __restrict__ gmax, const float* __restrict__ gsum,
                                 const float* __restrict__ weight, int R, int C, int64_t row_offset,
                                 int class_offset, int64_t num_nodes, float* __restrict__ loss) {
  float acc = 0.f;
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < R; row += gridDim.x * blockDim.x) {
    const int64_t t = target[row];
    const int64_t local = t - class_offset;
    if (row + row_offset < num_nodes && t >= 0 && local >= 0 && local < C) {
      float v = -(to_f(logits[row * ld + local]) - gmax[row] - __logf(gsum[row]));
      if (weight != nullptr) v *= weight[row];
      acc += v;
    }
  }
  __shared__ float red[32];
  for (int off = 16; off; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if (threadIdx.x == 0) atomicAdd(loss, v);
  }
}

template <typename T>
__global__ void xent_grad_kernel(const T* __restrict__ logits, int64_t ld, const int64_t* __restrict__ target,
                                 const float* __restrict__ gmax, const float* __restrict__ gsum,
                                 const float* __restrict__ scale_ptr, int R, int C, int64_t row_offset,
                                 int class_offset, int64_t num_nodes, int num_classes,
                                 T* __restrict__ grad, int64_t ldg) {
  const float scale = *scale_ptr;
  const int64_t total = static_cast<int64_t>(R) * C;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(i / C), c = static_cast<int>(i % C);
    const int64_t t = target[row];
    float g = 0.f;
    if (row + row_offset < num_nodes && t >= 0) {
      const int cls = c + class_offset;
      const float p = cls < num_classes ? __expf(to_f(logits[row * ld + c]) - gmax[row]) / gsum[row] : 0.f;
      g = (p - (cls == t ? 1.f : 0.f)) * scale;
    }
    grad[row * ldg + c] = from_f<T>(g);
  }
}

static int grid_for(int64_t work_items, int threads, int cap = 148 * 16) {
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(cap, (work_items + threads - 1) / threads)));
}

const char* launch_xent_stats(int dtype, const void* logits, int64_t ld, int R, int C,
                              int class_offset, int num_classes, float* rmax, float* rsum,
                              cudaStream_t stream) {
  if (R == 0) return nullptr;
  const int blocks = grid_for(static_cast<int64_t>(R) * 8, XENT_THREADS);
  if (dtype == DT_BF16)
    xent_stats_kernel<<<blocks, XENT_THREADS, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(logits), ld, R, C, class_offset, num_classes, rmax, rsum);
  else
    xent_stats_kernel<<<blocks, XENT_THREADS, 0, stream>>>(reinterpret_cast<const float*>(logits), ld, R,
                                                           C, class_offset, num_classes, rmax, rsum);
  return last_launch_error();
}

const char* launch_xent_loss(int dtype, const void* logits, int64_t ld, const int64_t* target,
                             const float* gmax, const float* gsum, const float* weight, int R, int C,
                             int64_t row_offset, int class_offset, int64_t num_nodes, float* loss,
                             cudaStream_t stream) {
  if (R == 0) return nullptr;
  const int blocks = grid_for(R, 256, 148 * 4);
  if (dtype == DT_BF16)
    xent_loss_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld,
                                                 target, gmax, gsum, weight, R, C, row_offset,
                                                 class_offset, num_nodes, loss);
  else
    xent_loss_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(logits), ld, target,
                                                 gmax, gsum, weight, R, C, row_offset, class_offset,
                                                 num_nodes, loss);
  return last_launch_error();
}

const char* launch_xent_grad(int dtype, const void* logits, int64_t ld, const int64_t* target,
                             const float* gmax, const float* gsum, const float* scale, int R, int C,
                             int64_t row_offset, int class_offset, int64_t num_nodes, int num_classes,
                             void* grad, int64_t ldg, cudaStream_t stream) {
  if (R == 0 || C == 0) return nullptr;
  const int blocks = grid_for(static_cast<int64_t>(R) * C, 256);
  if (dtype == DT_BF16)
    xent_grad_kernel<<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(logits), ld, target, gmax, gsum, scale, R, C, row_offset,
        class_offset, num_nodes, num_classes, reinterpret_cast<__nv_bfloat16*>(grad), ldg);
  else
    xent_grad_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(logits), ld, target,
                                                 gmax, gsum, scale, R, C, row_offset, class_offset,
                                                 num_nodes, num_classes, reinterpret_cast<float*>(grad),
                                                 ldg);
  return last_launch_error();
}

}  // namespace plx
