// Class-sharded softmax cross-entropy on logits [R, C] (bf16 or fp32), fp32 math.
//
//   xent_stats   : per row (max, sum exp(l - max)) over this rank's valid classes, one pass with a
//                  running maximum; when the classes are not sharded the same kernel also adds up
//                  the loss, so the forward is this one launch
//   xent_combine : after the exchange over the class axis - per row, combine the P shards'
//                  (max, sum exp) pairs in rank order and add up the loss terms of the targets that
//                  fall in this rank's class range (one launch instead of a chain of tensor ops)
//   xent_grad    : (exp(l - gmax)/gsum - onehot) * scale on valid rows, 0 elsewhere
//
// Exchange inside the kernels (opt-in, parallel/fused.py:xent_exchange_combine): xent_stats also
// stores each row's pair into this rank's receive slot on every peer of the class axis, and
// xent_combine starts with the flag barrier of that op and reads the peers' pairs straight from its
// receive slots - two launches for the whole sharded forward, no copy kernels in between.
//
// A row is handled by a group of LPR lanes (a power of two, several rows per warp) that reads and
// writes 16-byte vectors, so narrow class shards (C = 8..64) keep the accesses coalesced; rows
// whose address is not 16-byte aligned are read element by element.  Neither a softmax nor a
// one-hot matrix is stored; logits and targets are never modified.
//
// Reference: plexus/cross_entropy.py:35-101 (about 15 ATen kernels, int64 one-hot) and :108-114.

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "../include/peer_sync.cuh"
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

template <typename T>
struct XVec;
template <>
struct XVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& r, float (&f)[4]) {
    f[0] = __uint_as_float(r.x), f[1] = __uint_as_float(r.y), f[2] = __uint_as_float(r.z), f[3] = __uint_as_float(r.w);
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};
template <>
struct XVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& r, float (&f)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      f[2 * k] = __uint_as_float(w[k] << 16);
      f[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    uint4 o;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) p[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
    return o;
  }
};

// Elements [c, c + N) of a row as floats; positions at or beyond `n_valid` read as `fill`.
template <typename T>
__device__ __forceinline__ void load_vec(const T* __restrict__ row, int c, int n_valid, bool aligned, float fill,
                                         float (&f)[XVec<T>::N]) {
  constexpr int N = XVec<T>::N;
  if (aligned && c + N <= n_valid) {
    XVec<T>::unpack(__ldg(reinterpret_cast<const uint4*>(row + c)), f);
  } else {
#pragma unroll
    for (int k = 0; k < N; ++k) f[k] = c + k < n_valid ? to_f(row[c + k]) : fill;
  }
}

static int lanes_per_row_host(int C, int vn) {
  int l = 1;
  while (l < 32 && l * vn < C) l <<= 1;
  return l;
}

// Block sum of `v`, added to *dst by one thread.
__device__ __forceinline__ void block_add(float v, float* dst) {
  __shared__ float red[32];
  for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float w = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    for (int off = 16; off; off >>= 1) w += __shfl_xor_sync(0xffffffffu, w, off);
    if (threadIdx.x == 0 && w != 0.f) atomicAdd(dst, w);
  }
}

// stats[0][row] = max, stats[1][row] = sum exp(l - max) over the valid classes of this shard
// ((-inf, 0) if it holds none).  loss != nullptr (classes not sharded): also the loss terms.
template <typename T>
__global__ void __launch_bounds__(XENT_THREADS)
xent_stats_kernel(const T* __restrict__ logits, int64_t ld, int R, int C, int class_offset, int num_classes,
                  int lpr, float* __restrict__ stats, const int64_t* __restrict__ target,
                  const float* __restrict__ weight, int64_t row_offset, int64_t num_nodes, float* __restrict__ loss,
                  const SlotList push) {
  constexpr int N = XVec<T>::N;
  const int rows_per_block = XENT_THREADS / lpr;
  const int li = threadIdx.x & (lpr - 1), gi = threadIdx.x / lpr;
  const int n_valid = min(C, num_classes - class_offset);  // may be <= 0
  const bool aligned = (reinterpret_cast<uintptr_t>(logits) % 16 == 0) && (ld * sizeof(T) % 16 == 0);
  float acc = 0.f;
  for (int base = blockIdx.x * rows_per_block; base < R; base += gridDim.x * rows_per_block) {
    const int row = base + gi;
    const bool live = row < R;
    const T* lrow = logits + static_cast<int64_t>(live ? row : 0) * ld;
    float m = -INFINITY, s = 0.f;
    if (live) {
      for (int c = li * N; c < n_valid; c += lpr * N) {
        float f[N];
        load_vec<T>(lrow, c, n_valid, aligned, -INFINITY, f);
        float vm = f[0];
#pragma unroll
        for (int k = 1; k < N; ++k) vm = fmaxf(vm, f[k]);
        const float nm = fmaxf(m, vm);
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < N; ++k) t += __expf(f[k] - nm);
        s = s * __expf(m - nm) + t;  // m = -inf on the first vector: s is 0 there, exp(-inf) = 0
        m = nm;
      }
    }
    for (int off = 1; off < lpr; off <<= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, off);
      const float os = __shfl_xor_sync(0xffffffffu, s, off);
      const float nm = fmaxf(m, om);
      if (nm != -INFINITY) s = s * __expf(m - nm) + os * __expf(om - nm);
      m = nm;
    }
    if (live && li == 0) {
      stats[row] = m;
      stats[R + row] = s;
#pragma unroll
      for (int q = 0; q < MAX_PEERS; ++q) {  // the same pair into this rank's slot on every peer
        if (q < push.n) {
          float* dst = static_cast<float*>(push.ptr[q]);
          dst[row] = m;
          dst[R + row] = s;
        }
      }
      if (loss != nullptr) {
        const int64_t t = target[row];
        const int64_t local = t - class_offset;
        if (row + row_offset < num_nodes && t >= 0 && local >= 0 && local < C) {
          float v = -(to_f(lrow[local]) - m - __logf(s));
          if (weight != nullptr) v *= weight[row];
          acc += v;
        }
      }
    }
  }
  if (loss != nullptr) block_add(acc, loss);
}

// pairs.ptr[q] = class shard q's statistics [2][R] (rank order; the local buffer, a gathered tensor
// or this rank's receive slots) -> stats[2][R] and the loss terms.  sync.n > 0: first the flag
// barrier of the op that pushed the pairs.
template <typename T>
__global__ void __launch_bounds__(256)
xent_combine_kernel(const T* __restrict__ logits, int64_t ld, const int64_t* __restrict__ target,
                    const SlotList pairs, const float* __restrict__ weight, int R, int C,
                    int64_t row_offset, int class_offset, int64_t num_nodes, float* __restrict__ stats,
                    float* __restrict__ loss, const PeerSync sync) {
  if (sync.n > 0 && !signal_and_wait(sync)) return;
  const int P = pairs.n;
  float acc = 0.f;
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < R; row += gridDim.x * blockDim.x) {
    // static indices keep the pointer list in registers (a run-time index would copy it to local memory)
    float mq[MAX_PEERS + 1], sq[MAX_PEERS + 1];
    float m = -INFINITY;
#pragma unroll
    for (int q = 0; q <= MAX_PEERS; ++q) {
      mq[q] = -INFINITY;
      sq[q] = 0.f;
      if (q < P) {
        const float* pq = static_cast<const float*>(pairs.ptr[q]);
        mq[q] = pq[row];
        sq[q] = pq[R + row];
      }
      m = fmaxf(m, mq[q]);
    }
    float s = 0.f;
#pragma unroll
    for (int q = 0; q <= MAX_PEERS; ++q)  // rank order
      if (q < P && mq[q] != -INFINITY) s += sq[q] * __expf(mq[q] - m);
    stats[row] = m;
    stats[R + row] = s;
    const int64_t t = target[row];
    const int64_t local = t - class_offset;
    if (row + row_offset < num_nodes && t >= 0 && local >= 0 && local < C) {
      float v = -(to_f(logits[static_cast<int64_t>(row) * ld + local]) - m - __logf(s));
      if (weight != nullptr) v *= weight[row];
      acc += v;
    }
  }
  block_add(acc, loss);
}

template <typename T>
__global__ void __launch_bounds__(XENT_THREADS)
xent_grad_kernel(const T* __restrict__ logits, int64_t ld, const int64_t* __restrict__ target,
                 const float* __restrict__ gmax, const float* __restrict__ gsum,
                 const float* __restrict__ scale_ptr, int R, int C, int64_t row_offset, int class_offset,
                 int64_t num_nodes, int num_classes, int lpr, T* __restrict__ grad, int64_t ldg) {
  constexpr int N = XVec<T>::N;
  const float scale = *scale_ptr;
  const int rows_per_block = XENT_THREADS / lpr;
  const int li = threadIdx.x & (lpr - 1), gi = threadIdx.x / lpr;
  const int n_valid = min(C, num_classes - class_offset);
  const bool aligned = (reinterpret_cast<uintptr_t>(logits) % 16 == 0) && (ld * sizeof(T) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(grad) % 16 == 0) && (ldg * sizeof(T) % 16 == 0);
  for (int row = blockIdx.x * rows_per_block + gi; row < R; row += gridDim.x * rows_per_block) {
    const int64_t t = target[row];
    const bool valid = row + row_offset < num_nodes && t >= 0;
    const float m = gmax[row];
    const float inv = valid ? scale / gsum[row] : 0.f;
    const int hot = valid ? static_cast<int>(t - class_offset) : -1;  // column of the one-hot term, if local
    const T* lrow = logits + static_cast<int64_t>(row) * ld;
    T* grow = grad + static_cast<int64_t>(row) * ldg;
    for (int c = li * N; c < C; c += lpr * N) {
      float f[N];
      load_vec<T>(lrow, c, n_valid, aligned, -INFINITY, f);
#pragma unroll
      for (int k = 0; k < N; ++k) {
        float g = valid ? __expf(f[k] - m) * inv : 0.f;  // exp(-inf) = 0 on padded classes
        if (c + k == hot) g -= scale;
        f[k] = g;
      }
      if (aligned && c + N <= C) {
        *reinterpret_cast<uint4*>(grow + c) = XVec<T>::pack(f);
      } else {
#pragma unroll
        for (int k = 0; k < N; ++k)
          if (c + k < C) grow[c + k] = from_f<T>(f[k]);
      }
    }
  }
}

static int grid_for(int64_t work_items, int threads, int cap = 148 * 16) {
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(cap, (work_items + threads - 1) / threads)));
}

const char* launch_xent_stats(int dtype, const void* logits, int64_t ld, int R, int C, int class_offset,
                              int num_classes, float* stats, const int64_t* target, const float* weight,
                              int64_t row_offset, int64_t num_nodes, float* loss, cudaStream_t stream,
                              const SlotList* push_in) {
  if (R == 0) return nullptr;
  if (loss != nullptr && target == nullptr) return "xent_stats: the loss needs the targets";
  SlotList push = {};
  if (push_in != nullptr) push = *push_in;
  if (push.n < 0 || push.n > MAX_PEERS) return "xent_stats: too many push targets";
  const int lpr = lanes_per_row_host(C, dtype == DT_BF16 ? 8 : 4);
  const int blocks = grid_for(static_cast<int64_t>(R) * lpr, XENT_THREADS);
  if (dtype == DT_BF16)
    xent_stats_kernel<<<blocks, XENT_THREADS, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld, R, C,
                                                           class_offset, num_classes, lpr, stats, target, weight,
                                                           row_offset, num_nodes, loss, push);
  else
    xent_stats_kernel<<<blocks, XENT_THREADS, 0, stream>>>(reinterpret_cast<const float*>(logits), ld, R, C,
                                                           class_offset, num_classes, lpr, stats, target, weight,
                                                           row_offset, num_nodes, loss, push);
  return last_launch_error();
}

const char* launch_xent_combine(int dtype, const void* logits, int64_t ld, const int64_t* target,
                                const SlotList& pairs, const float* weight, int R, int C, int64_t row_offset,
                                int class_offset, int64_t num_nodes, float* stats, float* loss,
                                cudaStream_t stream, const PeerSync* sync_in) {
  if (R == 0 && sync_in == nullptr) return nullptr;
  if (pairs.n < 1 || pairs.n > MAX_PEERS + 1) return "xent_combine: 1 to 8 sets of statistics";
  for (int q = 0; q < pairs.n; ++q)
    if (pairs.ptr[q] == nullptr) return "xent_combine: missing statistics";
  PeerSync sync = {};
  if (sync_in != nullptr) sync = *sync_in;
  if (sync.n < 0 || sync.n > MAX_PEERS) return "xent_combine: bad flag lists";
  const int blocks = grid_for(std::max(R, 1), 256, 148 * 8);
  if (dtype == DT_BF16)
    xent_combine_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld, target, pairs,
                                                    weight, R, C, row_offset, class_offset, num_nodes, stats, loss,
                                                    sync);
  else
    xent_combine_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(logits), ld, target, pairs, weight,
                                                    R, C, row_offset, class_offset, num_nodes, stats, loss, sync);
  return last_launch_error();
}

const char* launch_xent_grad(int dtype, const void* logits, int64_t ld, const int64_t* target,
                             const float* gmax, const float* gsum, const float* scale, int R, int C,
                             int64_t row_offset, int class_offset, int64_t num_nodes, int num_classes,
                             void* grad, int64_t ldg, cudaStream_t stream) {
  if (R == 0 || C == 0) return nullptr;
  const int lpr = lanes_per_row_host(C, dtype == DT_BF16 ? 8 : 4);
  const int blocks = grid_for(static_cast<int64_t>(R) * lpr, XENT_THREADS);
  if (dtype == DT_BF16)
    xent_grad_kernel<<<blocks, XENT_THREADS, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(logits), ld, target, gmax, gsum, scale, R, C, row_offset,
        class_offset, num_nodes, num_classes, lpr, reinterpret_cast<__nv_bfloat16*>(grad), ldg);
  else
    xent_grad_kernel<<<blocks, XENT_THREADS, 0, stream>>>(reinterpret_cast<const float*>(logits), ld, target, gmax,
                                                          gsum, scale, R, C, row_offset, class_offset, num_nodes,
                                                          num_classes, lpr, reinterpret_cast<float*>(grad), ldg);
  return last_launch_error();
}

}  // namespace plx
