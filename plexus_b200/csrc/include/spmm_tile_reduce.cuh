// Device side of the all-reduce that the SpMM kernels finish themselves (see TileReduce in
// plexus_kernels.h): bf16 output rows are exchanged in fixed "tiles" of consecutive rows.  A warp
// that has written rows [a, b) locally and into the peers' receive slots calls publish(a, b): the
// row counts go to the peers' counters (release, system scope) and to a device-local counter; the
// warp whose rows complete a tile on this rank becomes responsible for reducing it.  It never waits
// for the peers while it still has rows of its own to compute - the tile goes on a small pending
// list that poll(false) checks between work items and poll(true) drains at the end of the kernel.
// Both ranks' warps therefore finish their own rows unconditionally and the final waits cannot
// deadlock.  Every wait is bounded; a timeout is recorded in the status words.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "plexus_kernels.h"
#include "ptx_sm100.cuh"

namespace plx {
namespace tile_reduce {

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint4 ld_cg16(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
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
__device__ __forceinline__ uint4 pack8(const float (&a)[8]) {
  uint4 o;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
  return o;
}
__device__ __forceinline__ void mask8(float (&a)[8], const uint4& m) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&m);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(p[i]);
    if (!(f.x > 0.f)) a[2 * i] = 0.f;
    if (!(f.y > 0.f)) a[2 * i + 1] = 0.f;
  }
}

// Have all peers pushed every row of exchange tile `tile` (nrows rows)?
static __device__ __forceinline__ bool tile_arrived(const TileReduce& red, int tile, int nrows, int* seen_out) {
  for (int q = 0; q < red.n; ++q) {
    int seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(red.local_sig[q] + tile) : "memory");
    if (seen < nrows) {
      *seen_out = seen;
      return false;
    }
  }
  return true;
}

// One exchange tile (output rows [r0, r0 + nrows)) whose partials have all arrived, done by one
// warp: out = mask(sum over the group), partials added in group-rank order; finally the tile's
// counters are cleared for the next op that uses this buffer.  Not inlined: it runs once per tile
// and must not add to the register budget of the callers' inner loops.
static __device__ __noinline__ void reduce_rows_tile(__nv_bfloat16* __restrict__ out, int64_t ldo, int r0, int nrows,
                                                 int D, const __nv_bfloat16* __restrict__ mask, int64_t ldm,
                                                 const TileReduce& red, int64_t slot_ld, int tile, int lane) {
  __threadfence();
  __syncwarp();
  const int vec = D >> 3;
  const int total = nrows * vec;
  constexpr int UN = 4;
  for (int v0 = lane; v0 < total; v0 += 32 * UN) {
    int64_t off_o[UN], off_s[UN], off_m[UN];
    bool live[UN];
    uint4 own[UN];
    float acc[UN][8];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int v = v0 + u * 32;
      live[u] = v < total;
      const int r = live[u] ? v / vec : 0, c = live[u] ? (v - r * vec) * 8 : 0;
      off_o[u] = static_cast<int64_t>(r0 + r) * ldo + c;
      off_s[u] = static_cast<int64_t>(r0 + r) * slot_ld + c;
      off_m[u] = static_cast<int64_t>(r0 + r) * ldm + c;
      own[u] = ld_cg16(out + off_o[u]);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[u][k] = 0.f;
      if (red.me <= 0) add_bf16x8(acc[u], own[u]);
    }
    for (int q = 0; q < red.n; ++q) {
      const __nv_bfloat16* sp = static_cast<const __nv_bfloat16*>(red.slot[q]);
      uint4 pv[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u) pv[u] = ld_cg16(sp + off_s[u]);
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        add_bf16x8(acc[u], pv[u]);
        if (q + 1 == red.me) add_bf16x8(acc[u], own[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      if (!live[u]) continue;
      if (mask != nullptr) mask8(acc[u], ld_cg16(mask + off_m[u]));
      *reinterpret_cast<uint4*>(out + off_o[u]) = pack8(acc[u]);
    }
  }
  __syncwarp();
  if (lane == 0) {
    for (int q = 0; q < red.n; ++q) red.local_sig[q][tile] = 0;
    red.local_done[tile] = 0;
  }
}

// Per-warp state and operations; every method is called by all 32 lanes of the warp.
struct Reducer {
  const TileReduce& red;
  __nv_bfloat16* out;
  int64_t ldo;
  const __nv_bfloat16* mask;
  int64_t ldm;
  int64_t slot_ld;
  int D, out_rows, lane, kernel_id;
  int pend_tile = 0;  // lane j keeps pending tile j
  int npend = 0;
  bool ok = true;

  __device__ Reducer(const TileReduce& r, __nv_bfloat16* o, int64_t ldo_, const __nv_bfloat16* m, int64_t ldm_,
                     int64_t slot_ld_, int D_, int out_rows_, int lane_, int kid)
      : red(r), out(o), ldo(ldo_), mask(m), ldm(ldm_), slot_ld(slot_ld_), D(D_), out_rows(out_rows_),
        lane(lane_), kernel_id(kid) {}

  __device__ __forceinline__ void poll(bool blocking) {
    const unsigned long long t0 = blocking ? global_ns() : 0ull;
    while (npend > 0 && ok) {
      bool ready = false;
      int seen = 0, t_rows = 0;
      if (lane < npend) {
        t_rows = min(red.tile_rows, out_rows - pend_tile * red.tile_rows);
        ready = tile_arrived(red, pend_tile, t_rows, &seen);
      }
      const unsigned ready_mask = __ballot_sync(0xffffffffu, ready);
      if (ready_mask == 0u) {
        if (!blocking) return;
        if (global_ns() - t0 > red.timeout_ns) {
          if (lane == 0) report_status(red.status, ST_TIMEOUT, kernel_id, 20, t_rows, seen);
          ok = false;
          return;
        }
        __nanosleep(128);
        continue;
      }
      const int j = __ffs(ready_mask) - 1;
      const int T = __shfl_sync(0xffffffffu, pend_tile, j);
      const int last = __shfl_sync(0xffffffffu, pend_tile, npend - 1);
      if (lane == j) pend_tile = last;
      --npend;
      const int r0 = T * red.tile_rows;
      reduce_rows_tile(out, ldo, r0, min(red.tile_rows, out_rows - r0), D, mask, ldm, red, slot_ld, T, lane);
    }
  }

  // Finished row ranges not yet published (lane j keeps range j).  Publishing costs a system-scope
  // fence, which under load waits tens of microseconds for this warp's NVLink stores to drain, so
  // ranges are published in batches.
  int q_beg = 0, q_end = 0, nq = 0;
  static constexpr int BATCH = 4;

  // Output rows [orb, ore) are written, locally and in the peers' slots.
  __device__ __forceinline__ void publish(int orb, int ore) {
    if (lane == nq) {
      q_beg = orb;
      q_end = ore;
    }
    if (++nq == BATCH) flush();
  }

  // Publish the recorded ranges: one fence, then per exchange tile the row counts go to the peers'
  // counters and to the local one; tiles completed on this rank by this warp go on the pending list.
  __device__ __forceinline__ void flush() {
    if (nq == 0) return;
    __syncwarp();
    if (lane == 0) __threadfence_system();  // the rows (local and in the peers' slots) before the counters
    __syncwarp();
    for (int i = 0; i < nq && ok; ++i) {
      const int orb = __shfl_sync(0xffffffffu, q_beg, i), ore = __shfl_sync(0xffffffffu, q_end, i);
      for (int T = orb / red.tile_rows; T * red.tile_rows < ore && ok; ++T) {
        const int t0 = T * red.tile_rows;
        const int t_rows = min(red.tile_rows, out_rows - t0);
        const int n_rows = min(ore, t0 + red.tile_rows) - max(orb, t0);
        int mine = 0;
        if (lane == 0) {
          for (int q = 0; q < red.n; ++q)
            asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(red.remote_sig[q] + T), "r"(n_rows)
                         : "memory");
          mine = atomicAdd(red.local_done + T, n_rows) + n_rows == t_rows;
        }
        mine = __shfl_sync(0xffffffffu, mine, 0);
        if (mine) {
          if (npend == 32) poll(true);  // list full: cannot happen with sane tile sizes
          if (lane == npend) pend_tile = T;
          ++npend;
        }
      }
    }
    nq = 0;
  }

  // End of the kernel: publish what is left, then wait (bounded) for the peers and reduce.
  __device__ __forceinline__ void finish() {
    flush();
    if (ok) poll(true);
  }
};

}  // namespace tile_reduce
}  // namespace plx
