// All-reduce of a matrix whose partials lie in a symmetric buffer (the same offset on every rank of
// an axis), reduced inside the NVSwitch where the buffer is bound to a multicast object.
//
//   * the compute kernel (SpMM / tcgen05 GEMM) writes its partial rows straight into the local
//     symmetric buffer S - nothing is pushed, nothing is copied;
//   * segment_reduce kernel (this file; op e): after the flag barrier of op e, rank r reduces row
//     segment r.  With a multicast address one `multimem.ld_reduce` fetches the fp32-accumulated
//     sum of the p partials of a 16-byte vector from the switch; ReLU / the ReLU-derivative mask
//     are applied and one `multimem.st` writes the result to the same place in every rank's S.
//     Per rank M/p bytes leave each GPU and M bytes arrive, whatever p is (the one-shot push
//     sends (p-1) M).  Without a multicast address (multicast refused for the group, or switched
//     off) the same kernel loads the p partials with plain peer loads, adds them in group-rank
//     order and stores the result to every rank with plain peer stores.
//   * the flagged copy of op e+1 (gather_segments in comm_fused.cu) moves S to the output tensor
//     once every rank's segment has landed.
// One rank reduces a segment and broadcasts the bits, so the replicas are bitwise equal.
// Numerics: the plain form adds the partials in fp32 and rounds once to nearest, like the other
// forms of this package.  The switch rounds the bf16 sum in its own way: measured on a 2-rank axis
// the results differ deterministically from the fp32 sum rounded to nearest (a 3-layer GCN's weight
// gradients then sit 0.07-0.11 from the fp64 oracle in max-norm instead of 0.065-0.11); a library
// all-reduce that uses the switch adds the same way.  PLEXUS_NVLS=0 selects the plain form.
// S needs no double buffering: a rank writes the partials of the next op only after the barrier
// of op e+1, which every rank passes only after it has finished reading the others' S.
//
// Reference: the all-reduces issued through AxoNN/NCCL at plexus/gcn_conv.py:191,215,261,278 on
// axes of more than two ranks.

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "../include/peer_sync.cuh"
#include "../include/plexus_kernels.h"

namespace plx {

__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_16(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ uint4 finish_bf16x8(uint4 v, int relu, const __nv_bfloat16* mask_vec) {
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
  if (relu) {
    const __nv_bfloat162 zero = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 4; ++k) p[k] = __hmax2(p[k], zero);
  }
  if (mask_vec != nullptr) {
    const uint4 mv = *reinterpret_cast<const uint4*>(mask_vec);
    const __nv_bfloat162* m = reinterpret_cast<const __nv_bfloat162*>(&mv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(m[k]);
      float2 x = __bfloat1622float2(p[k]);
      if (!(f.x > 0.f)) x.x = 0.f;
      if (!(f.y > 0.f)) x.y = 0.f;
      p[k] = __floats2bfloat162_rn(x.x, x.y);
    }
  }
  return v;
}

__device__ __forceinline__ void add8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(p[k]);
    acc[2 * k] += f.x;
    acc[2 * k + 1] += f.y;
  }
}

// Vectors [0, nvec) of this rank's segment start `elem_off` elements into S; row = vector / (cols/8).
// `mask` points at the segment's first row.
template <bool MC, int UN>
__global__ void __launch_bounds__(512)
segment_reduce_bf16_kernel(__nv_bfloat16* __restrict__ mc, const SlotList all, int64_t elem_off, int64_t nvec,
                           int cols, int relu, const __nv_bfloat16* __restrict__ mask, int64_t ldm,
                           const PeerSync sync) {
  if (!signal_and_wait(sync)) return;
  const int vpr = cols >> 3;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i0 = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i0 < nvec; i0 += stride * UN) {
    uint4 v[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int64_t i = i0 + u * stride;
      if (i >= nvec) continue;
      if constexpr (MC) {
        v[u] = multimem_ld_reduce_bf16x8(mc + elem_off + i * 8);
      } else {
        // group-rank order, fp32
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.f;
        uint4 pv[MAX_PEERS + 1];
#pragma unroll
        for (int q = 0; q <= MAX_PEERS; ++q)
          if (q < all.n)
            pv[q] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(all.ptr[q]) + elem_off + i * 8);
#pragma unroll
        for (int q = 0; q <= MAX_PEERS; ++q)
          if (q < all.n) add8(acc, pv[q]);
        __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&v[u]);
#pragma unroll
        for (int k = 0; k < 4; ++k) po[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
      }
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int64_t i = i0 + u * stride;
      if (i >= nvec) continue;
      const __nv_bfloat16* mv = nullptr;
      if (mask != nullptr) mv = mask + (i / vpr) * ldm + (i % vpr) * 8;
      const uint4 o = finish_bf16x8(v[u], relu, mv);
      if constexpr (MC) {
        multimem_st_16(mc + elem_off + i * 8, o);
      } else {
#pragma unroll
        for (int q = 0; q <= MAX_PEERS; ++q)
          if (q < all.n) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(all.ptr[q]) + elem_off + i * 8) = o;
      }
    }
  }
  // every thread orders its own stores to the other ranks before the kernel ends: the flag of the
  // next op is published by another thread of another launch, which must not overtake them
  __threadfence_system();
}

const char* launch_segment_reduce_bf16(void* mc, const SlotList& all, int64_t elem_off, int64_t rows, int cols,
                                       bool relu, const void* mask, int64_t ldm, const PeerSync& sync,
                                       int max_blocks, cudaStream_t stream) {
  if (cols <= 0 || cols % 8 || rows < 0 || elem_off < 0 || elem_off % 8)
    return "segment_reduce: columns and offset must be multiples of 8";
  if (all.n < 1 || all.n > MAX_PEERS + 1 || sync.n < 0 || sync.n > MAX_PEERS) return "segment_reduce: bad group";
  if (reinterpret_cast<uintptr_t>(mc) % 16 || reinterpret_cast<uintptr_t>(mask) % 16 || (mask && ldm % 8))
    return "segment_reduce: pointers must be 16-byte aligned";
  for (int q = 0; q < all.n; ++q)
    if (all.ptr[q] == nullptr || reinterpret_cast<uintptr_t>(all.ptr[q]) % 16)
      return "segment_reduce: buffer pointers must be 16-byte aligned";
  const int64_t nvec = rows * (cols / 8);
  constexpr int UN = 4;
  int64_t blocks = (nvec + 512 * UN - 1) / (512 * UN);
  blocks = std::max<int64_t>(1, std::min<int64_t>(blocks, max_blocks > 0 ? max_blocks : 148 * 2));
  __nv_bfloat16* m = static_cast<__nv_bfloat16*>(mc);
  const __nv_bfloat16* mk = static_cast<const __nv_bfloat16*>(mask);
  if (mc != nullptr)
    segment_reduce_bf16_kernel<true, UN><<<static_cast<int>(blocks), 512, 0, stream>>>(m, all, elem_off, nvec, cols,
                                                                                      relu ? 1 : 0, mk, ldm, sync);
  else
    segment_reduce_bf16_kernel<false, UN><<<static_cast<int>(blocks), 512, 0, stream>>>(m, all, elem_off, nvec, cols,
                                                                                       relu ? 1 : 0, mk, ldm, sync);
  return last_launch_error();
}

}  // namespace plx
