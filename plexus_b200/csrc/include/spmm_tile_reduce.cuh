// Per-warp bookkeeping of the all-reduce that the SpMM kernels finish themselves (TileReduce in
// plexus_kernels.h, device code in sentinel_reduce.cuh).  A warp that has stored output rows
// [a, b) locally and into the peers' receive slots calls publish(a, b); the range goes on a small
// queue (lane j of the warp keeps entry j).  poll() finishes the oldest ranges once a few newer
// ones are queued behind them - by then the peers' partials of those rows have normally arrived -
// but never waits: if something is missing it comes back later, so a warp always gets on with its
// own rows and the two ranks cannot wait for each other in a cycle.  finish() drains the queue at
// the end of the kernel with bounded waits (a timeout is recorded in the status words).
#pragma once

#include "sentinel_reduce.cuh"

namespace plx {
namespace tile_reduce {

struct Reducer {
  const TileReduce& red;
  __nv_bfloat16* out;
  int64_t ldo;
  const __nv_bfloat16* mask;
  int64_t ldm;
  int64_t slot_ld;
  int D, lane, kernel_id;
  int q_beg = 0, q_end = 0;  // lane j: queue entry j (a ring over the 32 lanes)
  int head = 0, count = 0;   // uniform over the warp
  int head_pos = 0;          // vectors of the head entry already finished
  bool ok = true;
  static constexpr int LAG = 2;

  __device__ Reducer(const TileReduce& r, __nv_bfloat16* o, int64_t ldo_, const __nv_bfloat16* m, int64_t ldm_,
                     int64_t slot_ld_, int D_, int /*out_rows*/, int lane_, int kid)
      : red(r), out(o), ldo(ldo_), mask(m), ldm(ldm_), slot_ld(slot_ld_), D(D_), lane(lane_), kernel_id(kid) {}

  // Work on the head entry; true if it is finished (and removed).
  __device__ __forceinline__ bool reduce_head(bool wait) {
    const int rb = __shfl_sync(0xffffffffu, q_beg, head), re = __shfl_sync(0xffffffffu, q_end, head);
    __syncwarp();
    const int total = (re - rb) * (D >> 3);
    const int done = sentinel::reduce_rows<4>(out + static_cast<int64_t>(rb) * ldo, ldo,
                                           static_cast<int64_t>(rb) * slot_ld, slot_ld, re - rb, D, head_pos,
                                           red, 0, mask ? mask + static_cast<int64_t>(rb) * ldm : nullptr, ldm,
                                           lane, wait, kernel_id);
    if (done < 0) {
      ok = false;
      return false;
    }
    if (done < total) {
      head_pos = done;
      return false;
    }
    head = (head + 1) & 31;
    --count;
    head_pos = 0;
    return true;
  }

  // Output rows [orb, ore) are written by this warp, locally and in the peers' slots.
  __device__ __forceinline__ void publish(int orb, int ore) {
    if (ore <= orb) return;
    while (count == 32 && ok) reduce_head(true);  // queue full: cannot happen with LAG << 32
    if (lane == ((head + count) & 31)) {
      q_beg = orb;
      q_end = ore;
    }
    ++count;
  }

  __device__ __forceinline__ void poll(bool /*blocking*/) {
    while (count > LAG && ok) {
      if (!reduce_head(false)) break;
    }
  }

  __device__ __forceinline__ void finish() {
    while (count > 0 && ok) reduce_head(true);
  }
};

}  // namespace tile_reduce
}  // namespace plx
