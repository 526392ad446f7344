// Peer-memory collectives over NVLink: the receive side of the fused "compute + push" kernels,
// small stand-alone collectives, and the CUDA-IPC symmetric workspace they run on.
//
// Protocol (one axis of the process grid, p ranks, every rank runs the same sequence of ops):
//   * every rank owns a workspace [flags | buffer 0 | buffer 1]; buffer b has one receive slot
//     per source rank.  Op number e (the "epoch", counted per axis) uses buffer e % 2.
//   * producer: a compute kernel (SpMM / GEMM epilogue, or push_copy) stores its rows into slot
//     `me` of every peer's buffer with plain 16-byte stores.
//   * consumer (the next launch on the same stream): block 0 publishes flag[e%2][me] = e on every
//     peer (release, system scope); every block waits until its own flag[e%2][q] >= e for all
//     peers q (acquire), then reduces / copies the slots.
//   * a buffer is rewritten only two ops later; by then every peer has passed the wait of the op
//     in between, which its owner publishes only after it finished reading: no extra barrier.
// Every wait is bounded by a wall-clock limit (globaltimer); on expiry the kernel records
// TIMEOUT(kernel, peer, expected, seen) in the status words and returns without touching data.
//
// Reference: the collectives issued through AxoNN/NCCL at plexus/gcn_conv.py:177-278 and
// plexus/cross_entropy.py:46-98.

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>

#include "../include/peer_sync.cuh"
#include "../include/plexus_kernels.h"
#include "../include/ptx_sm100.cuh"

namespace plx {

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(p[k]);
    acc[2 * k] += f.x;
    acc[2 * k + 1] += f.y;
  }
}

// out[r, c] = act( out[r, c] + sum_q slot_q[r, c] ) with fp32 accumulation, bf16 storage.
// act = optional ReLU, then optional multiplication by (mask > 0).
__global__ void __launch_bounds__(256)
reduce_slots_bf16_kernel(__nv_bfloat16* __restrict__ out, int64_t ldo, const SlotList slots,
                         int64_t lds, int64_t rows, int cols, int relu,
                         const __nv_bfloat16* __restrict__ mask, int64_t ldm, const PeerSync sync) {
  if (!signal_and_wait(sync)) return;
  const int my_pos = slots.me;
  const int vec_per_row = cols / 8;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    // all loads first (they are independent), then one summation order for the whole group: the
    // peers before this rank, the local partial, the peers after it
    const uint4 own = *reinterpret_cast<const uint4*>(out + r * ldo + c);
    uint4 pv[MAX_PEERS];
#pragma unroll
    for (int q = 0; q < MAX_PEERS; ++q)
      if (q < slots.n)
        pv[q] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(slots.ptr[q]) + r * lds + c);
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    if (my_pos <= 0) add_bf16x8(acc, own);
#pragma unroll
    for (int q = 0; q < MAX_PEERS; ++q) {
      if (q < slots.n) {
        add_bf16x8(acc, pv[q]);
        if (q + 1 == my_pos) add_bf16x8(acc, own);
      }
    }
    if (relu) {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = fmaxf(acc[k], 0.f);
    }
    if (mask != nullptr) {
      const uint4 mv = *reinterpret_cast<const uint4*>(mask + r * ldm + c);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&mv);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(p[k]);
        if (!(f.x > 0.f)) acc[2 * k] = 0.f;
        if (!(f.y > 0.f)) acc[2 * k + 1] = 0.f;
      }
    }
    uint4 o;
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) po[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
    *reinterpret_cast<uint4*>(out + r * ldo + c) = o;
  }
}

// Flag-free receive side of the one-shot all-reduce.  The peers' partials arrive in sentinel-kept
// slots (every byte 0xFF where nothing has arrived; see TileReduce in plexus_kernels.h): a vector is
// used once none of its eight bf16 elements is the sentinel, so the producers need neither flags
// nor fences and this kernel may start while the peers are still sending.  The local partial is
// already complete (the compute kernel that wrote it precedes this launch in stream order).
//   out[r, c] = act( sum over the group, in group-rank order ), then the slots get the sentinel back.
__device__ __forceinline__ bool has_sentinel(const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  bool s = false;
#pragma unroll
  for (int i = 0; i < 4; ++i) s = s || (w[i] & 0xffffu) == 0xffffu || (w[i] >> 16) == 0xffffu;
  return s;
}
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__global__ void __launch_bounds__(256)
reduce_sentinel_bf16_kernel(__nv_bfloat16* __restrict__ out, int64_t ldo, const SlotList slots, int64_t lds,
                            int64_t rows, int cols, int relu, const __nv_bfloat16* __restrict__ mask, int64_t ldm,
                            unsigned long long timeout_ns, int kernel_id, int* status) {
  const int my_pos = slots.me;
  const int vec_per_row = cols / 8;
  const int64_t total = rows * vec_per_row;
  const uint4 fill = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    const uint4 own = *reinterpret_cast<const uint4*>(out + r * ldo + c);
    uint4 pv[MAX_PEERS];
    unsigned long long t0 = 0;
    while (true) {
      bool ready = true;
#pragma unroll
      for (int q = 0; q < MAX_PEERS; ++q)
        if (q < slots.n) {
          pv[q] = ld_cg_u4(static_cast<const __nv_bfloat16*>(slots.ptr[q]) + r * lds + c);
          ready = ready && !has_sentinel(pv[q]);
        }
      if (ready) break;
      if (t0 == 0) t0 = global_ns();
      if (global_ns() - t0 > timeout_ns) {
        report_status(status, ST_TIMEOUT, kernel_id, 40, static_cast<int>(r), c);
        return;
      }
      __nanosleep(256);
    }
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    if (my_pos <= 0) add_bf16x8(acc, own);
#pragma unroll
    for (int q = 0; q < MAX_PEERS; ++q) {
      if (q < slots.n) {
        add_bf16x8(acc, pv[q]);
        if (q + 1 == my_pos) add_bf16x8(acc, own);
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(slots.ptr[q]) + r * lds + c) = fill;
      }
    }
    if (relu) {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = fmaxf(acc[k], 0.f);
    }
    if (mask != nullptr) {
      const uint4 mv = *reinterpret_cast<const uint4*>(mask + r * ldm + c);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&mv);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(p[k]);
        if (!(f.x > 0.f)) acc[2 * k] = 0.f;
        if (!(f.y > 0.f)) acc[2 * k + 1] = 0.f;
      }
    }
    uint4 o;
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) po[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
    *reinterpret_cast<uint4*>(out + r * ldo + c) = o;
  }
}

// Two-shot all-reduce, middle step: reduce this rank's row segment and broadcast the result.
//   out rows [row0, row0 + rows) += sum_q slot_q[0 .. rows)  (fp32), then ReLU / mask, then the
//   reduced rows are written to `out` and to slot row (r - row0) of every destination in `bcast`.
__global__ void __launch_bounds__(256)
reduce_segment_bf16_kernel(__nv_bfloat16* __restrict__ out, int64_t ldo, int64_t row0, const SlotList slots,
                           int64_t lds, int64_t rows, int cols, int relu,
                           const __nv_bfloat16* __restrict__ mask, int64_t ldm, const SlotList bcast,
                           const PeerSync sync) {
  if (!signal_and_wait(sync)) return;
  const int my_pos = slots.me;
  const int vec_per_row = cols / 8;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    // all loads first (they are independent), then one summation order for the whole group: the
    // peers before this rank, the local partial, the peers after it
    const uint4 own = *reinterpret_cast<const uint4*>(out + (row0 + r) * ldo + c);
    uint4 pv[MAX_PEERS];
#pragma unroll
    for (int q = 0; q < MAX_PEERS; ++q)
      if (q < slots.n)
        pv[q] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(slots.ptr[q]) + r * lds + c);
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    if (my_pos <= 0) add_bf16x8(acc, own);
#pragma unroll
    for (int q = 0; q < MAX_PEERS; ++q) {
      if (q < slots.n) {
        add_bf16x8(acc, pv[q]);
        if (q + 1 == my_pos) add_bf16x8(acc, own);
      }
    }
    if (relu) {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = fmaxf(acc[k], 0.f);
    }
    if (mask != nullptr) {
      const uint4 mv = *reinterpret_cast<const uint4*>(mask + (row0 + r) * ldm + c);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&mv);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(p[k]);
        if (!(f.x > 0.f)) acc[2 * k] = 0.f;
        if (!(f.y > 0.f)) acc[2 * k + 1] = 0.f;
      }
    }
    uint4 o;
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) po[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
    *reinterpret_cast<uint4*>(out + (row0 + r) * ldo + c) = o;
#pragma unroll
    for (int q = 0; q < MAX_PEERS; ++q) {
      if (q >= bcast.n) break;
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(bcast.ptr[q]) + r * lds + c) = o;
    }
  }
}

// After the wait: copy n.n[q] 16-byte words of slot q to dst_q (row segments of unequal length).
__global__ void __launch_bounds__(256)
gather_segments_kernel(const SlotList src, const SlotList dst, const SlotBytes n, const PeerSync sync) {
  if (!signal_and_wait(sync)) return;
#pragma unroll
  for (int q = 0; q < MAX_PEERS; ++q) {
    if (q >= src.n) break;
    const uint4* s = static_cast<const uint4*>(src.ptr[q]);
    uint4* d = static_cast<uint4*>(dst.ptr[q]);
    const int64_t words = n.n[q];
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < words;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
      d[i] = s[i];
  }
}

// out[i] = out[i] (op) slot_q[i] for fp32 vectors; op 0 = sum, 1 = max.
__global__ void __launch_bounds__(256)
reduce_slots_f32_kernel(float* __restrict__ out, const SlotList slots, int64_t n, int op,
                        const PeerSync sync) {
  if (!signal_and_wait(sync)) return;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    // group-rank order on every rank (see SlotList::me)
    const float own = out[i];
    float a = op == 0 ? 0.f : own;
    if (op == 0 && slots.me <= 0) a += own;
    for (int q = 0; q < slots.n; ++q) {
      const float b = static_cast<const float*>(slots.ptr[q])[i];
      a = op == 0 ? a + b : fmaxf(a, b);
      if (op == 0 && q + 1 == slots.me) a += own;
    }
    out[i] = a;
  }
}

// Copy n words from src to every destination (peers' slots and local copies).
template <typename W>
__global__ void __launch_bounds__(256)
push_copy_kernel(const W* __restrict__ src, const SlotList dst, int64_t n) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const W v = src[i];
    for (int q = 0; q < dst.n; ++q) static_cast<W*>(dst.ptr[q])[i] = v;
  }
}

// After the wait: copy slot q (n words) to dst_q for every peer (all-gather landing).
template <typename W>
__global__ void __launch_bounds__(256)
gather_slots_kernel(const SlotList src, const SlotList dst, int64_t n, const PeerSync sync) {
  if (!signal_and_wait(sync)) return;
  for (int q = 0; q < src.n; ++q) {
    const W* s = static_cast<const W*>(src.ptr[q]);
    W* d = static_cast<W*>(dst.ptr[q]);
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
      d[i] = s[i];
  }
}

static int copy_grid(int64_t items) {
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(sms * 8, (items + 255) / 256)));
}

const char* launch_reduce_slots_bf16(void* out, int64_t ldo, const SlotList& slots, int64_t lds,
                                     int64_t rows, int cols, bool relu, const void* mask, int64_t ldm,
                                     const PeerSync& sync, cudaStream_t stream) {
  if (cols % 8 || ldo % 8 || lds % 8 || (mask && ldm % 8)) return "reduce_slots: widths must be multiples of 8";
  if (slots.n < 0 || slots.n > MAX_PEERS || sync.n < 0 || sync.n > MAX_PEERS) return "reduce_slots: too many peers";
  reduce_slots_bf16_kernel<<<copy_grid(rows * (cols / 8)), 256, 0, stream>>>(
      static_cast<__nv_bfloat16*>(out), ldo, slots, lds, rows, cols, relu ? 1 : 0,
      static_cast<const __nv_bfloat16*>(mask), ldm, sync);
  return last_launch_error();
}

const char* launch_reduce_sentinel_bf16(void* out, int64_t ldo, const SlotList& slots, int64_t lds, int64_t rows,
                                        int cols, bool relu, const void* mask, int64_t ldm, double timeout_ms,
                                        int kernel_id, int* status, int max_blocks, cudaStream_t stream) {
  if (cols % 8 || ldo % 8 || lds % 8 || (mask && ldm % 8)) return "reduce_sentinel: widths must be multiples of 8";
  if (slots.n < 1 || slots.n > MAX_PEERS) return "reduce_sentinel: bad number of peers";
  if (rows <= 0) return nullptr;
  int grid = copy_grid(rows * (cols / 8));
  if (max_blocks > 0) grid = std::min(grid, max_blocks);
  reduce_sentinel_bf16_kernel<<<grid, 256, 0, stream>>>(
      static_cast<__nv_bfloat16*>(out), ldo, slots, lds, rows, cols, relu ? 1 : 0,
      static_cast<const __nv_bfloat16*>(mask), ldm, static_cast<unsigned long long>(timeout_ms * 1e6), kernel_id,
      status);
  return last_launch_error();
}

const char* launch_reduce_segment_bf16(void* out, int64_t ldo, int64_t row0, const SlotList& slots,
                                       int64_t lds, int64_t rows, int cols, bool relu, const void* mask,
                                       int64_t ldm, const SlotList& bcast, const PeerSync& sync,
                                       cudaStream_t stream) {
  if (cols % 8 || ldo % 8 || lds % 8 || (mask && ldm % 8)) return "reduce_segment: widths must be multiples of 8";
  if (slots.n < 0 || slots.n > MAX_PEERS || bcast.n < 0 || bcast.n > MAX_PEERS || sync.n < 0 ||
      sync.n > MAX_PEERS)
    return "reduce_segment: too many peers";
  if (rows < 0 || row0 < 0) return "reduce_segment: bad row range";
  // an empty segment still takes part in the flag exchange
  reduce_segment_bf16_kernel<<<copy_grid(std::max<int64_t>(1, rows * (cols / 8))), 256, 0, stream>>>(
      static_cast<__nv_bfloat16*>(out), ldo, row0, slots, lds, rows, cols, relu ? 1 : 0,
      static_cast<const __nv_bfloat16*>(mask), ldm, bcast, sync);
  return last_launch_error();
}

const char* launch_gather_segments(const SlotList& src, const SlotList& dst, const SlotBytes& bytes,
                                   const PeerSync& sync, cudaStream_t stream) {
  if (src.n != dst.n || src.n < 0 || src.n > MAX_PEERS) return "gather_segments: bad arguments";
  SlotBytes words = {};
  int64_t most = 1;
  for (int q = 0; q < src.n; ++q) {
    if (bytes.n[q] < 0 || bytes.n[q] % 16) return "gather_segments: sizes must be multiples of 16 bytes";
    if (reinterpret_cast<uintptr_t>(src.ptr[q]) % 16 || reinterpret_cast<uintptr_t>(dst.ptr[q]) % 16)
      return "gather_segments: pointers must be 16-byte aligned";
    words.n[q] = bytes.n[q] / 16;
    most = std::max(most, words.n[q]);
  }
  gather_segments_kernel<<<copy_grid(most), 256, 0, stream>>>(src, dst, words, sync);
  return last_launch_error();
}

const char* launch_reduce_slots_f32(float* out, const SlotList& slots, int64_t n, int op,
                                    const PeerSync& sync, cudaStream_t stream) {
  if (slots.n < 0 || slots.n > MAX_PEERS || sync.n < 0 || sync.n > MAX_PEERS) return "reduce_slots: too many peers";
  reduce_slots_f32_kernel<<<copy_grid(n), 256, 0, stream>>>(out, slots, n, op, sync);
  return last_launch_error();
}

static bool all_aligned16(const void* a, const SlotList& l) {
  if (reinterpret_cast<uintptr_t>(a) % 16) return false;
  for (int q = 0; q < l.n; ++q)
    if (reinterpret_cast<uintptr_t>(l.ptr[q]) % 16) return false;
  return true;
}

const char* launch_push_copy(const void* src, const SlotList& dst, int64_t bytes, cudaStream_t stream) {
  if (bytes % 4) return "push_copy: size must be a multiple of 4 bytes";
  if (bytes == 0 || dst.n == 0) return nullptr;
  if (bytes % 16 == 0 && all_aligned16(src, dst))
    push_copy_kernel<uint4><<<copy_grid(bytes / 16), 256, 0, stream>>>(static_cast<const uint4*>(src), dst,
                                                                       bytes / 16);
  else
    push_copy_kernel<uint32_t><<<copy_grid(bytes / 4), 256, 0, stream>>>(static_cast<const uint32_t*>(src),
                                                                         dst, bytes / 4);
  return last_launch_error();
}

const char* launch_gather_slots(const SlotList& src, const SlotList& dst, int64_t bytes,
                                const PeerSync& sync, cudaStream_t stream) {
  if (bytes % 4 || src.n != dst.n) return "gather_slots: bad arguments";
  if (bytes % 16 == 0 && all_aligned16(nullptr, src) && all_aligned16(nullptr, dst))
    gather_slots_kernel<uint4><<<copy_grid(std::max<int64_t>(1, bytes / 16)), 256, 0, stream>>>(src, dst,
                                                                                              bytes / 16, sync);
  else
    gather_slots_kernel<uint32_t><<<copy_grid(std::max<int64_t>(1, bytes / 4)), 256, 0, stream>>>(src, dst,
                                                                                                bytes / 4, sync);
  return last_launch_error();
}

// ------------------------------------------------------------------ CUDA-IPC workspace
const char* symm_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return cudaGetErrorString(e);
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) return cudaGetErrorString(e);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cudaGetErrorString(e);
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  *ptr = p;
  return nullptr;
}

const char* symm_open(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cudaGetErrorString(e);
  *ptr = p;
  return nullptr;
}

const char* symm_close(void* ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* symm_fill(void* ptr, int byte, size_t bytes) {
  cudaError_t e = cudaMemset(ptr, byte, bytes);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* symm_free(void* ptr) {
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace plx
