// Tall-skinny bf16 GEMMs of a GCN layer on the 5th-generation tensor cores.
//
//   gemm_nt :  C[M,N]  = A[M,K] . B[N,K]^T      (OUT = AGG.W with B = W^T; gradAGG = gradOUT.W^T
//                                                with B = W).  Both operands K-major.
//   gemm_tn :  C[Mw,Nw] = A[R,Mw]^T . B[R,Nw]   (gradW = AGG^T.gradOUT).  Both operands MN-major,
//                                                split over R across CTAs, fp32 partials.
//
// M (or R) is millions of rows while K and N are at most a few hundred, so the kernels are
// bandwidth bound: the design keeps the small operand resident in shared memory, streams the
// tall operand once through a TMA ring, accumulates in TMEM and overlaps the epilogue of one
// row tile with the MMAs of the next (two TMEM accumulators).
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (each owns one 32-lane TMEM quadrant).
// No TMA load uses cluster multicast.  Every mbarrier wait is bounded.
//
// Fused collective: gemm_nt's epilogue can store each finished row, besides (or instead of) the
// local output, into receive slots in other GPUs' memory with plain 16-byte stores over NVLink -
// to every peer (one-shot all-reduce) or only to the rank that owns the row (the reduce-scatter
// half of a two-shot all-reduce); see PushTargets and comm_fused.cu for the receive side.  In a
// debug run every such store is checked against the slot size first (push_in_bounds).
//
// gemm_nt_kernel<OutT, FUSED = true> (320 threads) is a separate instantiation that also finishes
// the one-shot all-reduce itself: warps 6..9 are reducer warps, one per 32-row quadrant of a tile.
// An epilogue warp pushes the raw partial (ReLU / mask deferred) and signals its reducer warp
// through shared memory; the reducer warp waits - bounded - until the peers' partials of those
// rows have arrived in the sentinel-kept receive slots, adds them in group-rank order, applies
// ReLU / the mask and stores the final rows (TileReduce, sentinel_reduce.cuh).  Measured slower
// than the flagged reduce launch (the reduce wants a full grid of threads), so it is opt-in.
//
// Reference call sites replaced: plexus/gcn_conv.py:211 (OUT), :237 (gradW), :256 (gradAGG),
// which go to cuBLAS SGEMM through torch.mm.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "../include/plexus_kernels.h"
#include "../include/ptx_sm100.cuh"
#include "../include/sentinel_reduce.cuh"

namespace plx {

constexpr int GEMM_THREADS = 192;
constexpr int BM = 128;
constexpr int BK = 64;                    // one 128-byte swizzle atom of bf16
constexpr int A_STAGE_BYTES = BM * 128;   // 16 KB
constexpr int SMEM_LIMIT = 232448;        // 227 KB opt-in maximum per CTA
constexpr int TMEM_COLS = 512;
constexpr int KERNEL_ID_GEMM = 6;

struct alignas(8) GemmBarriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t bfull;
  uint64_t tfull[2];
  uint64_t tempty[2];
  uint32_t tmem_base;
  int abort_flag;
  int stored[4];  // in-kernel all-reduce: tiles each epilogue warp has stored (read by its reducer warp)
  int pad[2];
};

// Epilogue staging: every epilogue warp owns 32 rows; a segment of SEG_BYTES per row goes
// TMEM -> registers -> shared memory, then leaves with 16-byte stores in which consecutive lanes
// cover consecutive bytes of one row (256-byte bursts), locally and into the peers' slots.
constexpr int SEG_BYTES = 256;
constexpr int STAGE_PITCH = SEG_BYTES + 16;  // padding spreads the rows over the banks
constexpr int STAGING_BYTES = 4 * 32 * STAGE_PITCH;

// Convert 16 accumulator columns (fp32 bits) and store them at `dst` in shared memory.
template <typename OutT>
__device__ __forceinline__ void stage16(uint8_t* dst, const uint32_t* r, bool relu);

template <>
__device__ __forceinline__ void stage16<__nv_bfloat16>(uint8_t* dst, const uint32_t* r, bool relu) {
  uint32_t packed[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float a = __uint_as_float(r[2 * i]), b = __uint_as_float(r[2 * i + 1]);
    if (relu) {
      a = fmaxf(a, 0.f);
      b = fmaxf(b, 0.f);
    }
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    packed[i] = *reinterpret_cast<uint32_t*>(&v);
  }
  uint4* d = reinterpret_cast<uint4*>(dst);
  d[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  d[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
}

template <>
__device__ __forceinline__ void stage16<float>(uint8_t* dst, const uint32_t* r, bool relu) {
  uint4* d = reinterpret_cast<uint4*>(dst);
  uint32_t v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i)
    v[i] = relu ? __float_as_uint(fmaxf(__uint_as_float(r[i]), 0.f)) : r[i];
  d[0] = make_uint4(v[0], v[1], v[2], v[3]);
  d[1] = make_uint4(v[4], v[5], v[6], v[7]);
  d[2] = make_uint4(v[8], v[9], v[10], v[11]);
  d[3] = make_uint4(v[12], v[13], v[14], v[15]);
}

// v = v where mask > 0 else 0, on a 16-byte vector of OutT
template <typename OutT>
__device__ __forceinline__ void apply_relu_mask(uint4& v, const uint4& m);
template <>
__device__ __forceinline__ void apply_relu_mask<__nv_bfloat16>(uint4& v, const uint4& m) {
  uint32_t* vw = reinterpret_cast<uint32_t*>(&v);
  const uint32_t* mw = reinterpret_cast<const uint32_t*>(&m);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t lo = mw[i] & 0xffffu, hi = mw[i] >> 16;
    // positive bf16: sign bit clear and not zero
    const uint32_t keep_lo = ((lo & 0x8000u) == 0 && (lo & 0x7fffu) != 0) ? 0x0000ffffu : 0u;
    const uint32_t keep_hi = ((hi & 0x8000u) == 0 && (hi & 0x7fffu) != 0) ? 0xffff0000u : 0u;
    vw[i] &= keep_lo | keep_hi;
  }
}
template <>
__device__ __forceinline__ void apply_relu_mask<float>(uint4& v, const uint4& m) {
  uint32_t* vw = reinterpret_cast<uint32_t*>(&v);
  const float* mf = reinterpret_cast<const float*>(&m);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (!(mf[i] > 0.f)) vw[i] = 0u;
}

// ---------------------------------------------------------------------------------------
// C[M,N] = A[M,K] . B[N,K]^T   (persistent over 128-row tiles; blockIdx.y = block of bn_box columns)
// ---------------------------------------------------------------------------------------
// FUSED: with the in-kernel all-reduce (bf16 result, four more warps); a separate instantiation so
// that the plain kernel keeps its register budget.
template <typename OutT, bool FUSED>
__global__ void __launch_bounds__(FUSED ? GEMM_THREADS + 128 : GEMM_THREADS, 1)
gemm_nt_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               OutT* __restrict__ C, int ldc, int M, int N, int K, int bn_box, int stages,
               int b_resident, int relu, int* status, const PushTargets push,
               const OutT* __restrict__ mask_in, int ldm, const TileReduce red) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);

  const int relu_in = relu;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = (K + BK - 1) / BK;
  const int n0 = blockIdx.y * bn_box;
  const int n_valid = min(bn_box, N - n0);
  const int bn = (n_valid + 15) & ~15;  // UMMA N
  const int b_blk_bytes = bn_box * 128;
  const int num_tiles = (M + BM - 1) / BM;

  uint8_t* b_res = smem;                                        // KB blocks when resident
  uint8_t* ring = smem + (b_resident ? KB * b_blk_bytes : 0);   // stages
  const int stage_bytes = A_STAGE_BYTES + (b_resident ? 0 : b_blk_bytes);
  GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(ring + stages * stage_bytes);
  uint8_t* staging = reinterpret_cast<uint8_t*>(bars) + ((sizeof(GemmBarriers) + 15) & ~15);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->bfull, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->tfull[b], 1);
      mbar_init(&bars->tempty[b], 4);
    }
    bars->abort_flag = 0;
    bars->stored[0] = bars->stored[1] = bars->stored[2] = bars->stored[3] = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  volatile int* abort_flag = &bars->abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      if (b_resident) {
        mbar_expect_tx(&bars->bfull, KB * b_blk_bytes);
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d(b_res + kb * b_blk_bytes, &tmB, &bars->bfull, kb * BK, n0);
      }
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1;
          if (*abort_flag || !mbar_wait(&bars->empty[s], ph ^ 1)) {
            report_status(status, ST_TIMEOUT, KERNEL_ID_GEMM, 0, s, it);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* st = ring + s * stage_bytes;
          mbar_expect_tx(&bars->full[s], stage_bytes);
          tma_load_2d(st, &tmA, &bars->full[s], kb * BK, tile * BM);
          if (!b_resident) tma_load_2d(st + A_STAGE_BYTES, &tmB, &bars->full[s], kb * BK, n0);
        }
      }
      if (!ok) {
        // giving up: let the copies already issued land before the CTA exits
        for (uint32_t j = it > (uint32_t)stages ? it - stages : 0; j < it; ++j)
          mbar_wait(&bars->full[j % stages], (j / stages) & 1);
        if (b_resident) mbar_wait(&bars->bfull, 0);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, bn, false, false);
      bool ok = true;
      if (b_resident && !mbar_wait(&bars->bfull, 0)) {
        report_status(status, ST_TIMEOUT, KERNEL_ID_GEMM, 1, 0, 0);
        *abort_flag = 1;
        ok = false;
      }
      uint32_t it = 0, t = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
        const int buf = t & 1;
        if (*abort_flag || !mbar_wait(&bars->tempty[buf], ((t >> 1) & 1) ^ 1)) {
          report_status(status, ST_TIMEOUT, KERNEL_ID_GEMM, 2, buf, t);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * 256;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1;
          if (*abort_flag || !mbar_wait(&bars->full[s], ph)) {
            report_status(status, ST_TIMEOUT, KERNEL_ID_GEMM, 3, s, it);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(ring + s * stage_bytes);
          const uint32_t b_addr = b_resident ? smem_u32(b_res + kb * b_blk_bytes)
                                             : a_addr + A_STAGE_BYTES;
          const int ksteps = min(4, (K - kb * BK + 15) / 16);
          for (int k = 0; k < ksteps; ++k) {
            const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t bd = make_smem_desc(b_addr + k * 32, 16, 1024);
            umma_bf16(d_tmem, ad, bd, idesc, (kb | k) != 0);
          }
          umma_commit(&bars->empty[s]);  // stage reusable once these MMAs retire
        }
        if (ok) umma_commit(&bars->tfull[buf]);
      }
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quadrant owned by this warp
    // with the in-kernel all-reduce the activation and the mask are applied after the sum
    constexpr bool fuse_reduce = FUSED;
    const OutT* mask = fuse_reduce ? nullptr : mask_in;
    if (fuse_reduce) relu = 0;
    uint32_t t = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t) {
      const int buf = t & 1;
      bool ok = !*abort_flag && mbar_wait(&bars->tfull[buf], (t >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report_status(status, ST_TIMEOUT, KERNEL_ID_GEMM, 4, buf, t);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      constexpr int ESZ = sizeof(OutT);
      constexpr int SEG_COLS = SEG_BYTES / ESZ;  // columns per staged segment
      constexpr int LANES_PER_ROW = SEG_BYTES / 16;
      constexpr int ROWS_PER_ITER = 32 / LANES_PER_ROW;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * 256;
      uint8_t* my_stage = staging + (warp - 2) * 32 * STAGE_PITCH;
      const int row0 = tile * BM + q * 32;
      for (int seg0 = 0; seg0 < bn; seg0 += SEG_COLS) {
        const int seg_cols = min(SEG_COLS, bn - seg0);
        if (seg_cols == 128) {
          // full bf16 segment: two 64-column loads in flight, one wait
          uint32_t r[128];
          tmem_ld64(taddr + seg0, *reinterpret_cast<uint32_t(*)[64]>(&r[0]));
          tmem_ld64(taddr + seg0 + 64, *reinterpret_cast<uint32_t(*)[64]>(&r[64]));
          tmem_ld_wait();
#pragma unroll
          for (int c0 = 0; c0 < 128; c0 += 16)
            stage16<OutT>(my_stage + lane * STAGE_PITCH + c0 * ESZ, &r[c0], relu != 0);
        } else if (seg_cols == 64) {
          uint32_t r[64];
          tmem_ld64(taddr + seg0, r);
          tmem_ld_wait();
#pragma unroll
          for (int c0 = 0; c0 < 64; c0 += 16)
            stage16<OutT>(my_stage + lane * STAGE_PITCH + c0 * ESZ, &r[c0], relu != 0);
        } else {
          for (int c0 = 0; c0 < seg_cols; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(taddr + seg0 + c0, r);
            tmem_ld_wait();
            stage16<OutT>(my_stage + lane * STAGE_PITCH + c0 * ESZ, r, relu != 0);
          }
        }
        if (seg0 + SEG_COLS >= bn) {
          // all TMEM reads of this tile are done: hand the accumulator back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->tempty[buf]);
        } else {
          __syncwarp();
        }
        const int sub = lane / LANES_PER_ROW, l = lane % LANES_PER_ROW;
        const int col = seg0 + l * (16 / ESZ);  // first column of this lane's 16 bytes
        if (col + 16 / ESZ <= n_valid) {
          // read the whole staged segment into registers first, then stream the stores back to back
          constexpr int NIT = 32 / ROWS_PER_ITER;
          uint4 v[NIT];
#pragma unroll
          for (int i = 0; i < NIT; ++i)
            v[i] = *reinterpret_cast<const uint4*>(my_stage + (i * ROWS_PER_ITER + sub) * STAGE_PITCH + l * 16);
          if (mask != nullptr) {
            // ReLU derivative of the layer input: zero the gradient where the saved activation is <= 0
            uint4 mk[NIT];
            const OutT* mbase = mask + static_cast<size_t>(row0 + sub) * ldm + n0 + col;
#pragma unroll
            for (int i = 0; i < NIT; ++i) {
              mk[i] = make_uint4(0, 0, 0, 0);
              if (row0 + i * ROWS_PER_ITER + sub < M)
                mk[i] = __ldg(reinterpret_cast<const uint4*>(mbase + static_cast<size_t>(i * ROWS_PER_ITER) * ldm));
            }
#pragma unroll
            for (int i = 0; i < NIT; ++i) apply_relu_mask<OutT>(v[i], mk[i]);
          }
          OutT* cbase = C + static_cast<size_t>(row0 + sub) * ldc + n0 + col;
          if (push.seg_rows > 0) {
            // reduce-scatter push: a row owned by a peer goes only into that peer's receive slot,
            // at its position inside the owner's row segment
#pragma unroll
            for (int i = 0; i < NIT; ++i) {
              const int row = row0 + i * ROWS_PER_ITER + sub;
              if (row < M) {
                const int owner = row / push.seg_rows;
                OutT* dst = cbase + static_cast<size_t>(i * ROWS_PER_ITER) * ldc;
                if (owner != push.me) {
                  const int idx = owner - (owner > push.me ? 1 : 0);
                  void* sel = push.base[0];
#pragma unroll
                  for (int p = 1; p < MAX_PEERS; ++p)  // static indices keep the pointers in registers
                    if (idx == p) sel = push.base[p];
                  const int64_t off = static_cast<int64_t>(row - owner * push.seg_rows) * push.ld + n0 + col;
                  if (!push_in_bounds(push.limit_elems, push.status, KERNEL_ID_GEMM, off, 8, row, n0 + col)) continue;
                  dst = static_cast<OutT*>(sel) + off;
                }
                *reinterpret_cast<uint4*>(dst) = v[i];
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < NIT; ++i) {
              const int row = row0 + i * ROWS_PER_ITER + sub;
              if (row < M) *reinterpret_cast<uint4*>(cbase + static_cast<size_t>(i * ROWS_PER_ITER) * ldc) = v[i];
            }
            // one-shot push: the same bytes go straight into every peer's receive slot
#pragma unroll
            for (int p = 0; p < MAX_PEERS; ++p) {  // static indices keep the pointers in registers
              if (p < push.n) {
                OutT* pbase = static_cast<OutT*>(push.base[p]) + static_cast<size_t>(row0 + sub) * push.ld + n0 + col;
#pragma unroll
                for (int i = 0; i < NIT; ++i) {
                  const int row = row0 + i * ROWS_PER_ITER + sub;
                  if (row < M &&
                      push_in_bounds(push.limit_elems, push.status, KERNEL_ID_GEMM,
                                     static_cast<int64_t>(row) * push.ld + n0 + col, 8, row, n0 + col))
                    *reinterpret_cast<uint4*>(pbase + static_cast<size_t>(i * ROWS_PER_ITER) * push.ld) = v[i];
                }
              }
            }
          }
        }
        __syncwarp();
      }
      if constexpr (FUSED) {
        {
          // this warp's 32 rows of the tile are stored, locally and in the peers' slots: tell the
          // reducer warp of this row quadrant
          __syncwarp();
          if (lane == 0)
            asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(smem_u32(&bars->stored[q])),
                         "r"(static_cast<int>(t) + 1)
                         : "memory");
        }
      }
    }
  } else {
    // ------------------------------------------------ reducer warps (in-kernel all-reduce only)
    // Warp 6 + q finishes the rows of quadrant q: as soon as epilogue warp q has stored a tile it
    // re-reads those rows together with the peers' partials of the same rows (valid once they no
    // longer hold the sentinel), sums in group-rank order, applies ReLU / the mask and writes the
    // final rows.  Waiting for the peers happens here, off the path of the MMAs and the pushes.
    if constexpr (FUSED) {
      const int q = warp - 6;
      const int my_tiles = (num_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                           static_cast<int>(gridDim.x);
      const int relu_after = relu;
      for (int k = 0; k < my_tiles && red.n > 0; ++k) {
        const unsigned long long t0 = sentinel::global_ns();
        bool have = false;
        while (!have && !*abort_flag) {
          int v;
          asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(v) : "r"(smem_u32(&bars->stored[q])) : "memory");
          have = v > k;
          if (!have) {
            if (sentinel::global_ns() - t0 > 4 * red.timeout_ns) break;  // the producers report their own timeouts
            __nanosleep(64);
          }
        }
        have = __all_sync(0xffffffffu, have);
        if (!have) break;
        const int r0 = (static_cast<int>(blockIdx.x) + k * static_cast<int>(gridDim.x)) * BM + q * 32;
        const int nrows = min(32, M - r0);
        if (nrows <= 0) continue;
        const int done = sentinel::reduce_rows<8>(
            reinterpret_cast<__nv_bfloat16*>(C) + static_cast<int64_t>(r0) * ldc + n0, ldc,
            static_cast<int64_t>(r0) * push.ld + n0, push.ld, nrows, n_valid, 0, red, relu_after,
            mask_in ? reinterpret_cast<const __nv_bfloat16*>(mask_in) + static_cast<int64_t>(r0) * ldm + n0 : nullptr,
            ldm, lane, true, KERNEL_ID_GEMM);
        if (done < 0) {
          *abort_flag = 1;
          break;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------
// partial[x][Mw,Nw] = A[rows_x, Mw]^T . B[rows_x, Nw]   (rows split over blockIdx.x)
// blockIdx.y = 256-wide block of Mw, blockIdx.z = 256-wide block of Nw.
// ---------------------------------------------------------------------------------------
constexpr int KT = 64;                  // reduction rows per stage
constexpr int ATOM_BYTES = KT * 128;    // 64 rows x 64 bf16 = 8 KB

struct alignas(8) WgradBarriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t done;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               float* __restrict__ partial, int R, int Mw, int Nw, int tiles_per_cta, int stages,
               int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * 256, n0 = blockIdx.z * 256;
  const int m_valid = min(256, Mw - m0), n_valid = min(256, Nw - n0);
  const int a_loaded = (m_valid + 63) / 64;       // atoms TMA fills
  const int a_atoms = (a_loaded + 1) & ~1;        // atoms the MMAs read (pairs of 64 = M 128)
  const int b_atoms = (n_valid + 63) / 64;
  const int MB = a_atoms / 2;
  const int bn = (n_valid + 15) & ~15;
  const int stage_bytes = (a_atoms + b_atoms) * ATOM_BYTES;
  const int total_tiles = (R + KT - 1) / KT;
  const int tile_begin = blockIdx.x * tiles_per_cta;
  const int tile_end = min(total_tiles, tile_begin + tiles_per_cta);
  const int ntiles = max(0, tile_end - tile_begin);

  WgradBarriers* bars = reinterpret_cast<WgradBarriers*>(smem + stages * stage_bytes);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->done, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  // The odd padding atom is never written by TMA: clear it so the MMAs read zeros.
  if (a_atoms != a_loaded) {
    for (int s = 0; s < stages; ++s) {
      uint4* z = reinterpret_cast<uint4*>(smem + s * stage_bytes + a_loaded * ATOM_BYTES);
      for (int i = threadIdx.x; i < ATOM_BYTES / 16; i += GEMM_THREADS) z[i] = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  volatile int* abort_flag = &bars->abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      for (int it = 0; it < ntiles; ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1;
        if (*abort_flag || !mbar_wait(&bars->empty[s], ph ^ 1)) {
          report_status(status, ST_TIMEOUT, KERNEL_ID_GEMM, 10, s, it);
          *abort_flag = 1;
          // giving up: let the copies already issued land before the CTA exits
          for (int j = it > stages ? it - stages : 0; j < it; ++j)
            mbar_wait(&bars->full[j % stages], (j / stages) & 1);
          break;
        }
        uint8_t* st = smem + s * stage_bytes;
        const int r0 = (tile_begin + it) * KT;
        mbar_expect_tx(&bars->full[s], (a_loaded + b_atoms) * ATOM_BYTES);
        for (int a = 0; a < a_loaded; ++a)
          tma_load_2d(st + a * ATOM_BYTES, &tmA, &bars->full[s], m0 + a * 64, r0);
        for (int b = 0; b < b_atoms; ++b)
          tma_load_2d(st + (a_atoms + b) * ATOM_BYTES, &tmB, &bars->full[s], n0 + b * 64, r0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, bn, true, true);
      bool ok = true;
      for (int it = 0; it < ntiles; ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1;
        if (*abort_flag || !mbar_wait(&bars->full[s], ph)) {
          report_status(status, ST_TIMEOUT, KERNEL_ID_GEMM, 11, s, it);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * stage_bytes);
        const uint32_t b_addr = a_addr + a_atoms * ATOM_BYTES;
        for (int kk = 0; kk < KT / 16; ++kk) {
          const uint64_t bd = make_smem_desc(b_addr + kk * 2048, ATOM_BYTES, 1024);
          for (int mb = 0; mb < MB; ++mb) {
            const uint64_t ad =
                make_smem_desc(a_addr + mb * 2 * ATOM_BYTES + kk * 2048, ATOM_BYTES, 1024);
            umma_bf16(tmem_base + mb * 256, ad, bd, idesc, (it | kk) != 0);
          }
        }
        umma_commit(&bars->empty[s]);
      }
      if (ok) umma_commit(&bars->done);
    }
  } else {
    const int q = warp & 3;
    float* out = partial + static_cast<size_t>(blockIdx.x) * Mw * Nw;
    if (ntiles > 0) {
      bool ok = !*abort_flag && mbar_wait(&bars->done, 0);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report_status(status, ST_TIMEOUT, KERNEL_ID_GEMM, 12, 0, 0);
        *abort_flag = 1;
      } else {
        tc_fence_after();
        for (int mb = 0; mb < MB; ++mb) {
          const int m = m0 + mb * 128 + q * 32 + lane;
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + mb * 256;
          for (int c0 = 0; c0 < bn; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(taddr + c0, r);
            tmem_ld_wait();
            if (m < Mw && mb * 128 + q * 32 + lane < m_valid) {
              float* dst = out + static_cast<size_t>(m) * Nw + n0 + c0;
#pragma unroll
              for (int j = 0; j < 16; j += 4) {
                if (c0 + j + 4 <= n_valid)
                  *reinterpret_cast<float4*>(dst + j) =
                      make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                  __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
              }
            }
          }
        }
      }
    } else {
      // no rows for this CTA: its partial is zero
      for (int i = (warp - 2) * 32 + lane; i < m_valid * n_valid; i += 128) {
        const int m = i / n_valid, n = i % n_valid;
        out[static_cast<size_t>(m0 + m) * Nw + n0 + n] = 0.f;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// Deterministic second stage of the split reduction: out[i] = sum_x partial[x][i].
__global__ void reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                       int parts, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int p = 0; p < parts; ++p) acc += partial[static_cast<size_t>(p) * n + i];
    out[i] = acc;
  }
}

// ----------------------------------------------------------------------------- host side
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

static EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeFn>(p);
  }
  return fn;
}

// Row-major bf16 matrix [rows, cols] with leading dimension ld (elements); box = box_rows x 64.
static const char* make_tmap_bf16(CUtensorMap* tm, const void* ptr, int64_t rows, int64_t cols,
                                  int64_t ld, int box_rows) {
  if (reinterpret_cast<uintptr_t>(ptr) % 16) return "gemm: TMA base must be 16-byte aligned";
  if ((ld * 2) % 16) return "gemm: TMA row stride must be a multiple of 16 bytes";
  EncodeFn enc = get_encode_fn();
  if (enc == nullptr) return "gemm: cuTensorMapEncodeTiled is not available from the driver";
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? nullptr : "gemm: cuTensorMapEncodeTiled failed";
}

static int num_sms() {
  int dev = 0, n = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

// max_stages / ctas_limit / nb_override (column-block width) select the launch variant (0 = default).
const char* launch_gemm_nt(const void* A, int64_t lda, const void* B, int64_t ldb, void* C,
                           int64_t ldc, int c_dtype, int64_t M, int64_t N, int64_t K, bool relu,
                           int* status, int max_stages, int ctas_limit, int nb_override,
                           const PushTargets* push_in, const void* mask, int64_t ldm, cudaStream_t stream,
                           const TileReduce* reduce_in) {
  TileReduce red = {};
  if (reduce_in != nullptr && reduce_in->n > 0) {
    red = *reduce_in;
    if (c_dtype != DT_BF16) return "gemm_nt: the in-kernel all-reduce needs a bf16 result";
    if (push_in == nullptr || push_in->n != red.n || push_in->seg_rows != 0)
      return "gemm_nt: the in-kernel all-reduce goes with the broadcast push to the same peers";
    if (red.n > MAX_PEERS) return "gemm_nt: too many peers";
    for (int q = 0; q < red.n; ++q)
      if (red.slot[q] == nullptr || reinterpret_cast<uintptr_t>(red.slot[q]) % 16)
        return "gemm_nt: bad in-kernel all-reduce description";
    red.status = status;
  }
  if (mask != nullptr && (ldm % 8 || reinterpret_cast<uintptr_t>(mask) % 16))
    return "gemm_nt: mask must be 16-byte aligned with a leading dimension multiple of 8";
  PushTargets push = {};
  if (push_in != nullptr) {
    push = *push_in;
    if (push.n < 0 || push.n > MAX_PEERS || push.ld % 8) return "gemm_nt: bad push targets";
    if (push.seg_rows < 0 || (push.seg_rows > 0 && (push.me < 0 || push.me > push.n ||
                                                    static_cast<int64_t>(push.seg_rows) * (push.n + 1) < M)))
      return "gemm_nt: bad reduce-scatter push description";
    for (int q = 0; q < push.n; ++q)
      if (reinterpret_cast<uintptr_t>(push.base[q]) % 16) return "gemm_nt: push targets must be 16-byte aligned";
  }
  if (K % 8 || N % 8 || lda % 8 || ldb % 8 || ldc % 8 || K <= 0)
    return "gemm_nt: K, N and leading dimensions must be positive multiples of 8";
  if (reinterpret_cast<uintptr_t>(C) % 16) return "gemm_nt: C must be 16-byte aligned";
  if (M == 0 || N == 0) return nullptr;
  const int KB = static_cast<int>((K + BK - 1) / BK);
  const int bar_bytes = sizeof(GemmBarriers) + 16 + STAGING_BYTES + 1024;  // + staging + alignment slack
  // Column block: as wide as possible, so that A is streamed exactly once (measured: a 256-wide
  // block with a 3-stage ring reaches 0.87 of copy bandwidth, two 128-wide blocks sharing the A
  // tiles through L2 only 0.52).  nb_override narrows it for tuning.
  int bn_box = static_cast<int>(std::min<int64_t>(256, (N + 15) / 16 * 16));
  if (nb_override > 0) bn_box = std::min(bn_box, std::max(16, (nb_override + 15) / 16 * 16));
  int b_resident = 1, stages = 0;
  const int b_blk = bn_box * 128;
  {
    int64_t left = SMEM_LIMIT - bar_bytes - static_cast<int64_t>(KB) * b_blk;
    stages = left > 0 ? static_cast<int>(left / A_STAGE_BYTES) : 0;
  }
  if (stages < 3) {
    b_resident = 0;
    stages = (SMEM_LIMIT - bar_bytes) / (A_STAGE_BYTES + b_blk);
  }
  stages = std::min(stages, 8);
  if (max_stages > 0) stages = std::min(stages, std::max(2, max_stages));
  if (stages < 2) return "gemm_nt: tile does not fit in shared memory";
  const int stage_bytes = A_STAGE_BYTES + (b_resident ? 0 : b_blk);
  const size_t smem = (b_resident ? static_cast<size_t>(KB) * b_blk : 0) +
                      static_cast<size_t>(stages) * stage_bytes + bar_bytes;

  CUtensorMap tmA, tmB;
  if (const char* e = make_tmap_bf16(&tmA, A, M, K, lda, BM)) return e;
  if (const char* e = make_tmap_bf16(&tmB, B, N, K, ldb, bn_box)) return e;
  const int tiles = static_cast<int>((M + BM - 1) / BM);
  const int n_blocks = static_cast<int>((N + bn_box - 1) / bn_box);
  const int ctas = std::min(tiles, ctas_limit > 0 ? ctas_limit : std::max(1, num_sms() / n_blocks));
  dim3 grid(ctas, static_cast<unsigned>(n_blocks));
  if (c_dtype == DT_BF16) {
    if (red.n > 0) {
      auto kern = gemm_nt_kernel<__nv_bfloat16, true>;
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      kern<<<grid, GEMM_THREADS + 128, smem, stream>>>(tmA, tmB, reinterpret_cast<__nv_bfloat16*>(C),
                                                       static_cast<int>(ldc), static_cast<int>(M),
                                                       static_cast<int>(N), static_cast<int>(K), bn_box, stages,
                                                       b_resident, relu ? 1 : 0, status, push,
                                                       reinterpret_cast<const __nv_bfloat16*>(mask),
                                                       static_cast<int>(ldm), red);
    } else {
      auto kern = gemm_nt_kernel<__nv_bfloat16, false>;
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      kern<<<grid, GEMM_THREADS, smem, stream>>>(tmA, tmB, reinterpret_cast<__nv_bfloat16*>(C),
                                                 static_cast<int>(ldc), static_cast<int>(M),
                                                 static_cast<int>(N), static_cast<int>(K), bn_box, stages,
                                                 b_resident, relu ? 1 : 0, status, push,
                                                 reinterpret_cast<const __nv_bfloat16*>(mask),
                                                 static_cast<int>(ldm), red);
    }
  } else if (c_dtype == DT_F32) {
    auto kern = gemm_nt_kernel<float, false>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<grid, GEMM_THREADS, smem, stream>>>(tmA, tmB, reinterpret_cast<float*>(C),
                                               static_cast<int>(ldc), static_cast<int>(M),
                                               static_cast<int>(N), static_cast<int>(K), bn_box, stages,
                                               b_resident, relu ? 1 : 0, status, push,
                                               reinterpret_cast<const float*>(mask), static_cast<int>(ldm), red);
  } else {
    return "gemm_nt: C must be bf16 or fp32";
  }
  return last_launch_error();
}

// Number of row-split CTAs gemm_tn uses for R reduction rows (scratch = parts * Mw * Nw floats).
int gemm_tn_parts(int64_t R) {
  const int total_tiles = static_cast<int>((R + KT - 1) / KT);
  const int want = std::max(1, std::min(num_sms(), total_tiles / 4));
  const int tpc = (total_tiles + want - 1) / want;
  return std::max(1, (total_tiles + tpc - 1) / std::max(1, tpc));
}

const char* launch_gemm_tn(const void* A, int64_t lda, const void* B, int64_t ldb, float* out,
                           float* scratch, int64_t scratch_elems, int64_t R, int64_t Mw, int64_t Nw,
                           int* status, cudaStream_t stream) {
  if (Mw % 8 || Nw % 8 || lda % 8 || ldb % 8)
    return "gemm_tn: widths and leading dimensions must be multiples of 8";
  if (Mw == 0 || Nw == 0) return nullptr;
  if (R == 0) {
    cudaMemsetAsync(out, 0, sizeof(float) * Mw * Nw, stream);
    return last_launch_error();
  }
  const int total_tiles = static_cast<int>((R + KT - 1) / KT);
  const int parts = gemm_tn_parts(R);
  const int tpc = (total_tiles + parts - 1) / parts;
  if (scratch_elems < static_cast<int64_t>(parts) * Mw * Nw) return "gemm_tn: scratch too small";

  const int a_atoms = ((static_cast<int>(std::min<int64_t>(256, Mw)) + 63) / 64 + 1) & ~1;
  const int b_atoms = (static_cast<int>(std::min<int64_t>(256, Nw)) + 63) / 64;
  const int stage_bytes = (a_atoms + b_atoms) * ATOM_BYTES;
  const int bar_bytes = sizeof(WgradBarriers) + 1024;
  const int stages = std::min(8, (SMEM_LIMIT - bar_bytes) / stage_bytes);
  if (stages < 2) return "gemm_tn: tile does not fit in shared memory";
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + bar_bytes;

  CUtensorMap tmA, tmB;
  if (const char* e = make_tmap_bf16(&tmA, A, R, Mw, lda, KT)) return e;
  if (const char* e = make_tmap_bf16(&tmB, B, R, Nw, ldb, KT)) return e;
  dim3 grid(parts, static_cast<unsigned>((Mw + 255) / 256), static_cast<unsigned>((Nw + 255) / 256));
  cudaFuncSetAttribute(gemm_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       static_cast<int>(smem));
  gemm_tn_kernel<<<grid, GEMM_THREADS, smem, stream>>>(tmA, tmB, scratch, static_cast<int>(R),
                                                       static_cast<int>(Mw), static_cast<int>(Nw), tpc,
                                                       stages, status);
  if (const char* e = last_launch_error()) return e;
  const int n = static_cast<int>(Mw * Nw);
  reduce_partials_kernel<<<std::min(1024, (n + 255) / 256), 256, 0, stream>>>(scratch, out, parts, n);
  return last_launch_error();
}

}  // namespace plx
