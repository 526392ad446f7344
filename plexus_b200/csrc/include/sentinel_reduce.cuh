// Device side of the all-reduce that the compute kernels finish themselves (see TileReduce in
// plexus_kernels.h).  A warp calls reduce_rows() for rows that IT has stored (locally and into the
// peers' slots) some time ago; validity of what the peers sent is carried by the data itself.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "plexus_kernels.h"
#include "ptx_sm100.cuh"

namespace plx {
namespace sentinel {

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// 16-byte load served by the L2 (the point of coherence for this GPU's memory, also for what the
// peers write into it over NVLink): never a stale line of this SM's L1
__device__ __forceinline__ uint4 ld_sys16(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ bool word_has_sentinel(uint32_t w) {
  return (w & 0xffffu) == 0xffffu || (w >> 16) == 0xffffu;
}
// true once all eight bf16 elements of the vector have arrived
__device__ __forceinline__ bool arrived(const uint4& v) {
  return !(word_has_sentinel(v.x) || word_has_sentinel(v.y) || word_has_sentinel(v.z) || word_has_sentinel(v.w));
}
__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(p[k]);
    acc[2 * k] += f.x;
    acc[2 * k + 1] += f.y;
  }
}

// One warp finishes `nrows` rows of `ncols` columns (a multiple of 8).  C and mask point at the
// first of those rows / columns; the peers' partials sit at element offset slot_off of every slot
// (leading dimension slot_ld).  C = act(sum over the group), partials added in group-rank order.
// `wait`: poll (bounded by red.timeout_ns) for vectors that have not arrived; without it the call
// returns at the first batch that is not complete.  Returns the number of vectors finished (pass it
// back as first_vec to resume), or -1 after a timeout.
// Requires: this warp stored the local partial rows itself (or is ordered after those stores).
template <int UN>
static __device__ __noinline__ int reduce_rows(__nv_bfloat16* __restrict__ C, int64_t ldc, int64_t slot_off, int64_t slot_ld,
                                        int nrows, int ncols, int first_vec, const TileReduce& red, int relu,
                                        const __nv_bfloat16* __restrict__ mask, int64_t ldm, int lane, bool wait,
                                        int kernel_id) {
  const int vpr = ncols >> 3;
  const int total = nrows * vpr;
  const uint4 fill = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);
  unsigned long long t0 = 0;
  int v0 = first_vec;
  while (v0 < total) {
    int64_t off_c[UN], off_s[UN], off_m[UN];
    bool live[UN];
    bool ready = true;
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int v = v0 + u * 32 + lane;
      live[u] = v < total;
      const int r = live[u] ? v / vpr : 0, c = live[u] ? (v - r * vpr) * 8 : 0;
      off_c[u] = static_cast<int64_t>(r) * ldc + c;
      off_s[u] = slot_off + static_cast<int64_t>(r) * slot_ld + c;
      off_m[u] = static_cast<int64_t>(r) * ldm + c;
    }
    // every load of the batch is issued before the first one is used
    uint4 own[UN], pv0[UN];
    const __nv_bfloat16* sp0 = static_cast<const __nv_bfloat16*>(red.slot[0]);
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      own[u] = live[u] ? ld_sys16(C + off_c[u]) : fill;
      pv0[u] = live[u] ? ld_sys16(sp0 + off_s[u]) : fill;
    }
    float acc[UN][8];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[u][k] = 0.f;
      if (red.me <= 0) add_bf16x8(acc[u], own[u]);
      if (live[u]) {
        ready = ready && arrived(pv0[u]);
        add_bf16x8(acc[u], pv0[u]);
        if (red.me == 1) add_bf16x8(acc[u], own[u]);
      }
    }
    for (int q = 1; q < red.n; ++q) {
      const __nv_bfloat16* sp = static_cast<const __nv_bfloat16*>(red.slot[q]);
      uint4 pv[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u)
        if (live[u]) pv[u] = ld_sys16(sp + off_s[u]);
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        if (live[u]) {
          ready = ready && arrived(pv[u]);
          add_bf16x8(acc[u], pv[u]);
          if (q + 1 == red.me) add_bf16x8(acc[u], own[u]);
        }
      }
    }
    if (!__all_sync(0xffffffffu, ready)) {
      // nothing of this batch has been changed: try again (or let the caller come back later)
      if (!wait) return v0;
      if (t0 == 0) t0 = global_ns();
      if (global_ns() - t0 > red.timeout_ns) {
        if (lane == 0) report_status(red.status, ST_TIMEOUT, kernel_id, 30, v0, total);
        return -1;
      }
      __nanosleep(64);
      continue;
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      if (!live[u]) continue;
      // the slots are clean again for the next op that receives into this buffer
      for (int q = 0; q < red.n; ++q)
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(red.slot[q]) + off_s[u]) = fill;
      if (relu) {
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[u][k] = fmaxf(acc[u][k], 0.f);
      }
      if (mask != nullptr) {
        const uint4 m = ld_sys16(mask + off_m[u]);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&m);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(p[k]);
          if (!(f.x > 0.f)) acc[u][2 * k] = 0.f;
          if (!(f.y > 0.f)) acc[u][2 * k + 1] = 0.f;
        }
      }
      uint4 o;
      __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int k = 0; k < 4; ++k) po[k] = __floats2bfloat162_rn(acc[u][2 * k], acc[u][2 * k + 1]);
      *reinterpret_cast<uint4*>(C + off_c[u]) = o;
    }
    v0 += 32 * UN;
    t0 = 0;
  }
  return total;
}

}  // namespace sentinel
}  // namespace plx
