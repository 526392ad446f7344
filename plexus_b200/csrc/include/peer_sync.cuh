// Flag barrier of the peer-memory collectives (see kernels/comm_fused.cu for the protocol): block 0
// publishes this rank's flag of the op on every peer, every block waits - bounded by a wall-clock
// limit - for the peers' flags.
#pragma once

#include <cuda_runtime.h>

#include "plexus_kernels.h"
#include "ptx_sm100.cuh"

namespace plx {

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Publish this rank's flag on every peer, then wait for every peer's flag.  Returns false on
// timeout (uniform over the block).
__device__ __forceinline__ bool signal_and_wait(const PeerSync& s) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  if (blockIdx.x == 0 && threadIdx.x < s.n) {
    __threadfence_system();
    st_release_sys(s.remote_flag[threadIdx.x], s.epoch);
  }
  if (threadIdx.x == 0) {
    const unsigned long long t0 = global_ns();
    for (int q = 0; q < s.n; ++q) {
      int seen = ld_acquire_sys(s.local_flag[q]);
      while (seen < s.epoch) {
        if (global_ns() - t0 > s.timeout_ns) {
          report_status(s.status, ST_TIMEOUT, s.kernel_id, q, s.epoch, seen);
          ok_flag = 0;
          break;
        }
        __nanosleep(64);
        seen = ld_acquire_sys(s.local_flag[q]);
      }
      if (!ok_flag) break;
    }
  }
  __syncthreads();
  return ok_flag != 0;
}

}  // namespace plx
