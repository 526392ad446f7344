// CSR SpMM  OUT[r0:r1, :] = A[r0:r1, :] . H   with bf16 (or fp32) features, fp32 accumulation.
//
// The op is bound by the gather of feature rows (each nonzero pulls one 2*D-byte row of H), so
// the kernel is organised around memory-level parallelism:
//   * one warp per row; the warp is split in G = 32/LPR groups of LPR lanes, a group reads one
//     feature row with 16-byte loads (LPR*VPL vectors cover the D columns), different groups
//     take different nonzeros of the row, and each group keeps several nonzeros in flight;
//   * column indices / values are read coalesced, 32 at a time, and broadcast by shuffles;
//   * load balance on power-law graphs comes from a per-matrix schedule built once on the
//     device: consecutive rows are grouped in blocks of about equal cost (nonzeros + a per-row
//     constant) and warps walk the blocks round-robin; rows longer than PIECE nonzeros are cut
//     in pieces of PIECE nonzeros, one warp per piece writes an fp32 partial row to scratch
//     memory and a fix-up launch sums the pieces of each long row in a fixed order;
//   * the epilogue optionally multiplies by (mask > 0): that is the ReLU derivative of the
//     layer input, applied where the input gradient is produced.
//
// Reference call sites replaced: plexus/gcn_conv.py:98,188,265 (torch.sparse.mm -> cuSPARSE, fp32).

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <type_traits>

#include "../include/plexus_kernels.h"

namespace plx {

constexpr int SPMM_WARPS = 8;
constexpr int PIECE = 256;  // rows longer than this are cut in pieces of this many nonzeros

// Packed fp32x2 arithmetic (sm_100): one instruction updates two accumulators, which halves
// the issue slots the multiply-adds take.  The SpMM inner loop is issue bound, not DRAM bound.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ unsigned long long pack2u(uint32_t lo, uint32_t hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void ffma2(unsigned long long& acc, unsigned long long x, unsigned long long a) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(x), "l"(a));
}

template <typename T>
struct Vec16;  // 16-byte vector of T
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  // acc2[i] holds columns (2i, 2i+1); a bf16 pair widens to fp32x2 with one shift and one mask
  __device__ static void fma2(unsigned long long (&acc2)[4], const uint4& v, unsigned long long a2) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) ffma2(acc2[i], pack2u(w[i] << 16, w[i] & 0xffff0000u), a2);
  }
  __device__ static uint4 pack(const float (&acc)[8]) {
    uint4 o;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    return o;
  }
  __device__ static void mask(float (&acc)[8], const uint4& m) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&m);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(p[i]);
      if (!(f.x > 0.f)) acc[2 * i] = 0.f;
      if (!(f.y > 0.f)) acc[2 * i + 1] = 0.f;
    }
  }
};
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static void fma2(unsigned long long (&acc2)[2], const uint4& v, unsigned long long a2) {
    ffma2(acc2[0], pack2u(v.x, v.y), a2);
    ffma2(acc2[1], pack2u(v.z, v.w), a2);
  }
  __device__ static uint4 pack(const float (&acc)[4]) {
    uint4 o;
    float* p = reinterpret_cast<float*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = acc[i];
    return o;
  }
  __device__ static void mask(float (&acc)[4], const uint4& m) {
    const float* p = reinterpret_cast<const float*>(&m);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (!(p[i] > 0.f)) acc[i] = 0.f;
  }
};

__device__ __forceinline__ uint4 ldg16(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

// Accumulate nonzeros [beg, end) of one row.  Group g of the warp takes nonzeros g, g+G, ...
// and keeps U of them in flight.
template <typename T, int LPR, int VPL>
__device__ __forceinline__ void row_accumulate(const int* __restrict__ col,
                                               const float* __restrict__ val,
                                               const T* __restrict__ H, int64_t ldh, int D,
                                               int64_t beg, int64_t end, int lane,
                                               float (&acc)[VPL][Vec16<T>::N]) {
  constexpr int VN = Vec16<T>::N;
  constexpr int G = 32 / LPR;
#ifndef PLX_SPMM_U
#define PLX_SPMM_U 4
#endif
  constexpr int U = VPL == 1 ? PLX_SPMM_U : 2;  // nonzeros in flight per group
  const int g = lane / LPR, li = lane % LPR;
  const uint32_t ldh32 = static_cast<uint32_t>(ldh);  // 32 x 32 -> 64-bit multiply-add per row address
  bool active[VPL];
  const T* hbase[VPL];  // this lane's column offset folded into the base pointer
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    active[v] = (v * LPR + li) * VN < D;
    hbase[v] = H + (v * LPR + li) * VN;
  }
  unsigned long long acc2[VPL][VN / 2];
#pragma unroll
  for (int v = 0; v < VPL; ++v)
#pragma unroll
    for (int i = 0; i < VN / 2; ++i) acc2[v][i] = 0ull;

  for (int64_t base = beg; base < end; base += 32) {
    const int cnt = (end - base) < 32 ? static_cast<int>(end - base) : 32;
    int c = 0;
    float a = 0.f;
    if (lane < cnt) {
      c = __ldg(col + base + lane);
      a = __ldg(val + base + lane);
    }
    // lanes beyond cnt repeat the batch's last column with weight 0: their products vanish
    // (and cannot introduce a NaN the row would not have anyway), so the loop below needs no
    // per-nonzero predicate
    {
      const int c_last = __shfl_sync(0xffffffffu, c, cnt - 1);
      if (lane >= cnt) c = c_last;
    }
    for (int jj = 0; jj < cnt; jj += U * G) {  // trip count is uniform across the warp
      int cj[U];
      unsigned long long aj[U];
      uint4 vj[U][VPL];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int j = (jj + u * G + g) & 31;
        cj[u] = __shfl_sync(0xffffffffu, c, j);
        const float av = __shfl_sync(0xffffffffu, a, j);
        aj[u] = pack2(av, av);
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int v = 0; v < VPL; ++v)
          if (active[v])
            vj[u][v] = ldg16(hbase[v] + static_cast<uint64_t>(static_cast<uint32_t>(cj[u])) * ldh32);
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int v = 0; v < VPL; ++v)
          if (active[v]) Vec16<T>::fma2(acc2[v], vj[u][v], aj[u]);
    }
  }
#pragma unroll
  for (int v = 0; v < VPL; ++v)
#pragma unroll
    for (int i = 0; i < VN / 2; ++i) unpack2(acc2[v][i], acc[v][2 * i], acc[v][2 * i + 1]);
  // combine the G groups
#pragma unroll
  for (int off = LPR; off < 32; off <<= 1) {
#pragma unroll
    for (int v = 0; v < VPL; ++v)
#pragma unroll
      for (int i = 0; i < VN; ++i) acc[v][i] += __shfl_xor_sync(0xffffffffu, acc[v][i], off);
  }
}

// ---------------------------------------------------------------------------------------
// Tensor-core variant of row_accumulate for bf16 features with D <= 256.
//
// The FMA loop above spends ~28 warp instructions per nonzero and is issue bound.  Here the
// gathered rows of a batch of 16 nonzeros are copied to shared memory with cp.async (no
// registers, no widening), and the weighted sum over the batch is a [D x 16] . [16 x 8] product
// done by warp-level MMAs (m16n8k16, fp32 accumulate): the 16 features of an MMA come from
// ldmatrix.trans of the staged rows, column 0 / 1 of the 8-wide operand hold the high / low
// bf16 halves of the fp32 edge weights (hi + lo keeps 16 mantissa bits), the other columns are
// zero.  About 2 instructions per 16 features and 16 nonzeros instead of 12 per 8 and 1.
// (tcgen05 is not used here: its smallest tile has M = 128 rows in TMEM per CTA and a
// single-thread issue model, which does not fit one independent accumulator per output row.)
// ---------------------------------------------------------------------------------------
constexpr int MMA_WARPS = 4;      // warps per CTA of the MMA kernels (3 CTAs per SM fit)
constexpr int MMA_BATCH = 16;     // nonzeros per staged batch (= K of the MMA)

// shared memory of one warp: two batches of staged rows + a 1 KB exchange area for the result
__host__ __device__ constexpr int mma_pitch(int LPR) { return LPR * 16 + 16; }  // bytes per staged row
__host__ __device__ constexpr int mma_warp_bytes(int LPR) { return 2 * MMA_BATCH * mma_pitch(LPR) + 1024; }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// LPR lanes cover a row with 16 bytes each, i.e. LPR / 2 blocks of 16 features.
template <int LPR>
__device__ __forceinline__ void row_accumulate_mma(const int* __restrict__ col,
                                                   const float* __restrict__ val,
                                                   const __nv_bfloat16* __restrict__ H, int64_t ldh,
                                                   int D, int64_t beg, int64_t end, int lane,
                                                   uint8_t* stage, float (&acc)[1][8]) {
  constexpr int G = 32 / LPR;
  constexpr int MB = LPR / 2;
  constexpr int pitch = mma_pitch(LPR);
  const int g = lane / LPR, li = lane % LPR;
  const uint32_t stage_addr = static_cast<uint32_t>(__cvta_generic_to_shared(stage));
  const bool col_active = li * 8 < D;
  const uint32_t ldh32 = static_cast<uint32_t>(ldh);
  const __nv_bfloat16* hbase = H + li * 8;
  const int gid = lane >> 2, tig = lane & 3;
  // ldmatrix.x4: lanes 0-7 / 8-15 / 16-23 / 24-31 give the row addresses of the four 8x8 blocks
  // (k 0-7, m 0-7), (k 0-7, m 8-15), (k 8-15, m 0-7), (k 8-15, m 8-15) of a 16-feature block.
  const uint32_t ldm_off = ((lane & 7) + ((lane & 16) ? 8 : 0)) * pitch + ((lane & 8) ? 16 : 0);

  float c[MB][4];
#pragma unroll
  for (int m = 0; m < MB; ++m)
#pragma unroll
    for (int i = 0; i < 4; ++i) c[m][i] = 0.f;

  int pending = 0;          // 1 if a batch is in flight / staged but not yet multiplied
  uint32_t pb0 = 0, pb1 = 0;  // its weight fragments
  int cur = 0;              // buffer the next batch is gathered into

  auto consume = [&](int buf, uint32_t b0, uint32_t b1) {
    const uint32_t base = stage_addr + buf * (MMA_BATCH * pitch) + ldm_off;
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      uint32_t a[4];
      ldmatrix_x4_trans(base + m * 32, a);
      mma_bf16_16816(c[m], a, b0, b1);
    }
  };

  for (int64_t base = beg; base < end; base += 32) {
    const int cnt = (end - base) < 32 ? static_cast<int>(end - base) : 32;
    int cc = 0;
    float a = 0.f;
    if (lane < cnt) {
      cc = __ldg(col + base + lane);
      a = __ldg(val + base + lane);
    }
    // split the fp32 weight in two bf16 terms: hi in the low half-word, lo in the high one
    uint32_t hl;
    {
      const __nv_bfloat16 hi = __float2bfloat16_rn(a);
      const __nv_bfloat16 lo = __float2bfloat16_rn(a - __bfloat162float(hi));
      hl = static_cast<uint32_t>(__bfloat16_as_ushort(hi)) |
           (static_cast<uint32_t>(__bfloat16_as_ushort(lo)) << 16);
    }
    for (int half = 0; half * MMA_BATCH < cnt; ++half) {
      const int k0 = half * MMA_BATCH;
      // ---- gather up to 16 rows of H into buffer `cur`
      const uint32_t dst0 = stage_addr + cur * (MMA_BATCH * pitch) + li * 16;
#pragma unroll
      for (int s = 0; s < MMA_BATCH / G; ++s) {
        const int kk = s * G + g;  // slot inside the batch
        const int ck = __shfl_sync(0xffffffffu, cc, (k0 + kk) & 31);
        if (k0 + kk < cnt && col_active)
          cp_async16(dst0 + kk * pitch, hbase + static_cast<uint64_t>(static_cast<uint32_t>(ck)) * ldh32);
      }
      cp_async_commit();
      // ---- weight fragments of this batch: B[k][n], n = 0 -> hi, n = 1 -> lo, else 0
      uint32_t x0 = __shfl_sync(0xffffffffu, hl, (k0 + 2 * tig) & 31);
      uint32_t x1 = __shfl_sync(0xffffffffu, hl, (k0 + 2 * tig + 1) & 31);
      uint32_t x2 = __shfl_sync(0xffffffffu, hl, (k0 + 2 * tig + 8) & 31);
      uint32_t x3 = __shfl_sync(0xffffffffu, hl, (k0 + 2 * tig + 9) & 31);
      uint32_t b0 = 0, b1 = 0;
      if (gid == 0) {
        b0 = (x0 & 0xffffu) | (x1 << 16);
        b1 = (x2 & 0xffffu) | (x3 << 16);
      } else if (gid == 1) {
        b0 = (x0 >> 16) | (x1 & 0xffff0000u);
        b1 = (x2 >> 16) | (x3 & 0xffff0000u);
      }
      // ---- multiply the previous batch while this one is in flight
      if (pending) {
        cp_async_wait<1>();
        __syncwarp();
        consume(cur ^ 1, pb0, pb1);
        __syncwarp();
      }
      pending = 1;
      pb0 = b0;
      pb1 = b1;
      cur ^= 1;
    }
  }
  if (pending) {
    cp_async_wait<0>();
    __syncwarp();
    consume(cur ^ 1, pb0, pb1);
    __syncwarp();
  }
  // lanes with tig == 0 hold feature (16 m + gid) in c[m][0] + c[m][1] and feature
  // (16 m + gid + 8) in c[m][2] + c[m][3]; hand every lane its 8 consecutive features
  float* xch = reinterpret_cast<float*>(stage + 2 * MMA_BATCH * pitch);  // separate from the staged rows
  if (tig == 0) {
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      xch[m * 16 + gid] = c[m][0] + c[m][1];
      xch[m * 16 + gid + 8] = c[m][2] + c[m][3];
    }
  }
  __syncwarp();
  if (g == 0 && col_active) {
    const float4 lo4 = *reinterpret_cast<const float4*>(xch + li * 8);
    const float4 hi4 = *reinterpret_cast<const float4*>(xch + li * 8 + 4);
    acc[0][0] = lo4.x; acc[0][1] = lo4.y; acc[0][2] = lo4.z; acc[0][3] = lo4.w;
    acc[0][4] = hi4.x; acc[0][5] = hi4.y; acc[0][6] = hi4.z; acc[0][7] = hi4.w;
  }
  __syncwarp();
}

// Peer slot that owns output row `orow` in the reduce-scatter mode (nullptr: this rank owns it).
// Static indices keep the pointer table in registers.
template <typename T>
__device__ __forceinline__ T* scatter_target(const PushTargets& push, int64_t orow, int64_t& slot_row) {
  const int owner = static_cast<int>(orow / push.seg_rows);
  if (owner == push.me) return nullptr;
  const int idx = owner - (owner > push.me ? 1 : 0);
  void* sel = push.base[0];
#pragma unroll
  for (int q = 1; q < MAX_PEERS; ++q)
    if (idx == q) sel = push.base[q];
  slot_row = orow - static_cast<int64_t>(owner) * push.seg_rows;
  return static_cast<T*>(sel);
}

template <typename T, int LPR, int VPL>
__device__ __forceinline__ void row_store(T* __restrict__ out_row, const T* __restrict__ mask_row,
                                          int D, int lane, float (&acc)[VPL][Vec16<T>::N],
                                          const PushTargets& push, int64_t orow) {
  constexpr int VN = Vec16<T>::N;
  if (lane >= LPR) return;
  if (push.seg_rows > 0) {
    // reduce-scatter: a row owned by a peer goes only into that peer's receive slot
    int64_t slot_row = 0;
    T* peer = scatter_target<T>(push, orow, slot_row);
    if (peer != nullptr) out_row = peer + slot_row * push.ld;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const int c = (v * LPR + lane) * VN;
      if (c < D) {
        if (mask_row != nullptr) Vec16<T>::mask(acc[v], ldg16(mask_row + c));
        *reinterpret_cast<uint4*>(out_row + c) = Vec16<T>::pack(acc[v]);
      }
    }
    return;
  }
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    const int c = (v * LPR + lane) * VN;
    if (c < D) {
      if (mask_row != nullptr) Vec16<T>::mask(acc[v], ldg16(mask_row + c));
      const uint4 packed = Vec16<T>::pack(acc[v]);
      *reinterpret_cast<uint4*>(out_row + c) = packed;
      // fused collective: the same row goes straight into the peers' receive slots
#pragma unroll
      for (int q = 0; q < MAX_PEERS; ++q)  // static indices keep the pointers in registers
        if (q < push.n)
          *reinterpret_cast<uint4*>(static_cast<T*>(push.base[q]) + orow * push.ld + c) = packed;
    }
  }
}

template <int VPL, int VN>
__device__ __forceinline__ void zero_acc(float (&acc)[VPL][VN]) {
#pragma unroll
  for (int v = 0; v < VPL; ++v)
#pragma unroll
    for (int i = 0; i < VN; ++i) acc[v][i] = 0.f;
}

// Rows of at most PIECE nonzeros.  block_start[b] .. block_start[b+1] are consecutive rows of
// about equal total cost; warps take blocks round-robin.
// Dispatch to the tensor-core or the FMA accumulation.
template <typename T, int LPR, int VPL, bool MMA>
__device__ __forceinline__ void accumulate_row(const int* col, const float* val, const T* H, int64_t ldh,
                                               int D, int64_t beg, int64_t end, int lane, uint8_t* stage,
                                               float (&acc)[VPL][Vec16<T>::N]) {
  if constexpr (MMA) {
    row_accumulate_mma<LPR>(col, val, H, ldh, D, beg, end, lane, stage, acc);
  } else {
    row_accumulate<T, LPR, VPL>(col, val, H, ldh, D, beg, end, lane, acc);
  }
}

// Per-warp staging area of the MMA kernels (dynamic shared memory), zeroed once so that slots a
// short batch leaves unfilled hold finite values (they are multiplied by a zero weight).
template <int LPR, bool MMA>
__device__ __forceinline__ uint8_t* warp_stage(int lane) {
  if constexpr (MMA) {
    extern __shared__ uint4 spmm_smem[];
    uint8_t* st = reinterpret_cast<uint8_t*>(spmm_smem) + (threadIdx.x >> 5) * mma_warp_bytes(LPR);
    uint4* z = reinterpret_cast<uint4*>(st);
    for (int i = lane; i < mma_warp_bytes(LPR) / 16; i += 32) z[i] = make_uint4(0, 0, 0, 0);
    __syncwarp();
    return st;
  } else {
    return nullptr;
  }
}

template <typename T, int LPR, int VPL, bool MMA>
#ifndef PLX_SPMM_MINB
#define PLX_SPMM_MINB 4
#endif
__global__ void __launch_bounds__(MMA ? MMA_WARPS * 32 : SPMM_WARPS * 32, MMA ? 3 : (VPL == 1 ? PLX_SPMM_MINB : 2))
spmm_rows_kernel(const int* __restrict__ rowptr, const int* __restrict__ col,
                 const float* __restrict__ val, const T* __restrict__ H, int64_t ldh,
                 T* __restrict__ out, int64_t ldo, const T* __restrict__ mask, int64_t ldm, int D,
                 int row_begin, const int* __restrict__ block_start, int num_blocks,
                 const PushTargets push) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int warp_global = blockIdx.x * wpb + (threadIdx.x >> 5);
  const int warps_total = gridDim.x * wpb;
  uint8_t* stage = warp_stage<LPR, MMA>(lane);
  for (int b = warp_global; b < num_blocks; b += warps_total) {
    const int rb = __ldg(block_start + b), re = __ldg(block_start + b + 1);
    for (int row = rb; row < re; ++row) {
      const int64_t beg = __ldg(rowptr + row), end = __ldg(rowptr + row + 1);
      if (end - beg > PIECE) continue;  // handled by the piece kernels
      float acc[VPL][Vec16<T>::N];
      zero_acc(acc);
      accumulate_row<T, LPR, VPL, MMA>(col, val, H, ldh, D, beg, end, lane, stage, acc);
      const int64_t orow = row - row_begin;
      row_store<T, LPR, VPL>(out + orow * ldo, mask ? mask + orow * ldm : nullptr, D, lane, acc, push,
                             orow);
    }
  }
}

// One warp per piece of a long row: fp32 partial row -> scratch[piece][LPR*VPL*VN].
template <typename T, int LPR, int VPL, bool MMA>
__global__ void __launch_bounds__(MMA ? MMA_WARPS * 32 : SPMM_WARPS * 32, MMA ? 3 : (VPL == 1 ? PLX_SPMM_MINB : 2))
spmm_pieces_kernel(const int* __restrict__ piece_beg, const int* __restrict__ piece_end,
                   int num_pieces, const int* __restrict__ col, const float* __restrict__ val,
                   const T* __restrict__ H, int64_t ldh, int D, float* __restrict__ scratch) {
  constexpr int VN = Vec16<T>::N;
  constexpr int W = LPR * VPL * VN;
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int warp_global = blockIdx.x * wpb + (threadIdx.x >> 5);
  const int warps_total = gridDim.x * wpb;
  uint8_t* stage = warp_stage<LPR, MMA>(lane);
  for (int p = warp_global; p < num_pieces; p += warps_total) {
    float acc[VPL][VN];
    zero_acc(acc);
    accumulate_row<T, LPR, VPL, MMA>(col, val, H, ldh, D, __ldg(piece_beg + p), __ldg(piece_end + p),
                                     lane, stage, acc);
    if (lane < LPR) {
      float* dst = scratch + static_cast<int64_t>(p) * W;
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        float4* d4 = reinterpret_cast<float4*>(dst + (v * LPR + lane) * VN);
#pragma unroll
        for (int i = 0; i < VN; i += 4) d4[i / 4] = make_float4(acc[v][i], acc[v][i + 1], acc[v][i + 2], acc[v][i + 3]);
      }
    }
  }
}

// One warp per long row: sum its pieces in order, apply the mask, store.
template <typename T, int LPR, int VPL>
__global__ void __launch_bounds__(SPMM_WARPS * 32)
spmm_fixup_kernel(const int* __restrict__ long_rows, const int* __restrict__ long_piece_start,
                  int num_long, const float* __restrict__ scratch, T* __restrict__ out, int64_t ldo,
                  const T* __restrict__ mask, int64_t ldm, int D, int row_begin,
                  const PushTargets push) {
  constexpr int VN = Vec16<T>::N;
  constexpr int W = LPR * VPL * VN;
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int warp_global = blockIdx.x * wpb + (threadIdx.x >> 5);
  const int warps_total = gridDim.x * wpb;
  for (int i = warp_global; i < num_long; i += warps_total) {
    float acc[VPL][VN];
    zero_acc(acc);
    const int p0 = __ldg(long_piece_start + i), p1 = __ldg(long_piece_start + i + 1);
    if (lane < LPR) {
      for (int p = p0; p < p1; ++p) {
        const float* src = scratch + static_cast<int64_t>(p) * W;
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
          const float4* s4 = reinterpret_cast<const float4*>(src + (v * LPR + lane) * VN);
#pragma unroll
          for (int k = 0; k < VN; k += 4) {
            const float4 f = s4[k / 4];
            acc[v][k] += f.x;
            acc[v][k + 1] += f.y;
            acc[v][k + 2] += f.z;
            acc[v][k + 3] += f.w;
          }
        }
      }
    }
    const int64_t orow = __ldg(long_rows + i) - row_begin;
    row_store<T, LPR, VPL>(out + orow * ldo, mask ? mask + orow * ldm : nullptr, D, lane, acc, push,
                           orow);
  }
}

static int spmm_grid(int work_items, int warps_per_block, int blocks_per_sm) {
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return std::max(1, std::min(sms * blocks_per_sm, (work_items + warps_per_block - 1) / warps_per_block));
}

// use_mma: tensor-core accumulation (bf16 features, at most 256 columns)
template <typename T, int LPR, int VPL>
static void launch_spmm(const int* rowptr, const int* col, const float* val, const T* H, int64_t ldh,
                        T* out, int64_t ldo, const T* mask, int64_t ldm, int D, int row_begin,
                        const SpmmSchedule& s, float* scratch, const PushTargets& push, bool use_mma,
                        cudaStream_t stream) {
  constexpr bool CAN_MMA = std::is_same<T, __nv_bfloat16>::value && VPL == 1;
  if constexpr (CAN_MMA) {
    if (use_mma) {
      constexpr int smem = MMA_WARPS * mma_warp_bytes(LPR);
      auto rows_k = spmm_rows_kernel<T, LPR, VPL, true>;
      auto pieces_k = spmm_pieces_kernel<T, LPR, VPL, true>;
      cudaFuncSetAttribute(rows_k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      cudaFuncSetAttribute(pieces_k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (s.num_blocks > 0)
        rows_k<<<spmm_grid(s.num_blocks, MMA_WARPS, 6), MMA_WARPS * 32, smem, stream>>>(
            rowptr, col, val, H, ldh, out, ldo, mask, ldm, D, row_begin, s.block_start, s.num_blocks, push);
      if (s.num_long > 0) {
        pieces_k<<<spmm_grid(s.num_pieces, MMA_WARPS, 6), MMA_WARPS * 32, smem, stream>>>(
            s.piece_beg, s.piece_end, s.num_pieces, col, val, H, ldh, D, scratch);
        spmm_fixup_kernel<T, LPR, VPL><<<spmm_grid(s.num_long, SPMM_WARPS, 8), SPMM_WARPS * 32, 0, stream>>>(
            s.long_rows, s.long_piece_start, s.num_long, scratch, out, ldo, mask, ldm, D, row_begin, push);
      }
      return;
    }
  }
  if (s.num_blocks > 0)
    spmm_rows_kernel<T, LPR, VPL, false><<<spmm_grid(s.num_blocks, SPMM_WARPS, 8), SPMM_WARPS * 32, 0, stream>>>(
        rowptr, col, val, H, ldh, out, ldo, mask, ldm, D, row_begin, s.block_start, s.num_blocks, push);
  if (s.num_long > 0) {
    spmm_pieces_kernel<T, LPR, VPL, false><<<spmm_grid(s.num_pieces, SPMM_WARPS, 8), SPMM_WARPS * 32, 0, stream>>>(
        s.piece_beg, s.piece_end, s.num_pieces, col, val, H, ldh, D, scratch);
    spmm_fixup_kernel<T, LPR, VPL><<<spmm_grid(s.num_long, SPMM_WARPS, 8), SPMM_WARPS * 32, 0, stream>>>(
        s.long_rows, s.long_piece_start, s.num_long, scratch, out, ldo, mask, ldm, D, row_begin, push);
  }
}

// fp32 scratch elements per piece for a feature width of D elements of the given dtype.
int64_t spmm_scratch_per_piece(int dtype, int D) {
  const int vn = dtype == DT_BF16 ? 8 : 4;
  const int vecs = (D + vn - 1) / vn;
  int lpr = 4;
  while (lpr < 32 && lpr < vecs) lpr <<= 1;
  const int vpl = (vecs + 31) / 32 > 1 ? (vecs + 31) / 32 : 1;
  return static_cast<int64_t>(lpr) * vpl * vn;
}

template <typename T>
static const char* dispatch_spmm(int D, const int* rowptr, const int* col, const float* val, const T* H,
                                 int64_t ldh, T* out, int64_t ldo, const T* mask, int64_t ldm,
                                 int row_begin, const SpmmSchedule& s, float* scratch,
                                 const PushTargets& push, bool use_mma, cudaStream_t stream) {
  constexpr int VN = Vec16<T>::N;
  const int vecs = (D + VN - 1) / VN;  // 16-byte vectors per feature row
#define PLX_SPMM(LPR, VPL) \
  launch_spmm<T, LPR, VPL>(rowptr, col, val, H, ldh, out, ldo, mask, ldm, D, row_begin, s, scratch, push, \
                           use_mma, stream)
  if (vecs <= 4) PLX_SPMM(4, 1);
  else if (vecs <= 8) PLX_SPMM(8, 1);
  else if (vecs <= 16) PLX_SPMM(16, 1);
  else if (vecs <= 32) PLX_SPMM(32, 1);
  else if (vecs <= 64) PLX_SPMM(32, 2);
  else if (vecs <= 96) PLX_SPMM(32, 3);
  else if (vecs <= 128) PLX_SPMM(32, 4);
  else return "spmm: feature width too large (max 128 16-byte vectors per row)";
#undef PLX_SPMM
  return last_launch_error();
}

int spmm_piece_size() { return PIECE; }

// out[r - row_begin] = A[r, :] . H for the rows covered by the schedule (optionally masked).
const char* launch_spmm_csr(int dtype, const int* rowptr, const int* col, const float* val,
                            const void* H, int64_t ldh, void* out, int64_t ldo, const void* mask,
                            int64_t ldm, int D, int row_begin, const SpmmSchedule& sched,
                            float* scratch, int64_t scratch_elems, const PushTargets* push_in,
                            int variant, cudaStream_t stream) {
  const bool use_mma = variant == SPMM_VARIANT_TENSOR;
  const int esz = dtype == DT_BF16 ? 2 : 4;
  PushTargets push = {};
  if (push_in != nullptr) {
    push = *push_in;
    if (push.n < 0 || push.n > MAX_PEERS || (push.ld * esz) % 16) return "spmm: bad push targets";
    if (push.seg_rows < 0 || (push.seg_rows > 0 && (push.me < 0 || push.me > push.n)))
      return "spmm: bad reduce-scatter push description";
    for (int q = 0; q < push.n; ++q)
      if (reinterpret_cast<uintptr_t>(push.base[q]) % 16) return "spmm: push targets must be 16-byte aligned";
  }
  if ((ldh * esz) % 16 || (ldo * esz) % 16 || (D * esz) % 16 || (mask && (ldm * esz) % 16))
    return "spmm: feature rows must be multiples of 16 bytes";
  if (ldh < 0 || ldh > 0x7fffffffLL) return "spmm: leading dimension of H out of range";
  if (reinterpret_cast<uintptr_t>(H) % 16 || reinterpret_cast<uintptr_t>(out) % 16 ||
      reinterpret_cast<uintptr_t>(mask) % 16 || reinterpret_cast<uintptr_t>(scratch) % 16)
    return "spmm: feature pointers must be 16-byte aligned";
  if (D == 0 || (sched.num_blocks == 0 && sched.num_long == 0)) return nullptr;
  if (sched.num_pieces > 0 &&
      scratch_elems < static_cast<int64_t>(sched.num_pieces) * spmm_scratch_per_piece(dtype, D))
    return "spmm: scratch too small for the long-row pieces";
  if (dtype == DT_BF16)
    return dispatch_spmm<__nv_bfloat16>(D, rowptr, col, val, reinterpret_cast<const __nv_bfloat16*>(H),
                                        ldh, reinterpret_cast<__nv_bfloat16*>(out), ldo,
                                        reinterpret_cast<const __nv_bfloat16*>(mask), ldm, row_begin,
                                        sched, scratch, push, use_mma, stream);
  if (dtype == DT_F32)
    return dispatch_spmm<float>(D, rowptr, col, val, reinterpret_cast<const float*>(H), ldh,
                                reinterpret_cast<float*>(out), ldo, reinterpret_cast<const float*>(mask),
                                ldm, row_begin, sched, scratch, push, false, stream);
  return "spmm: features must be bf16 or fp32";
}

}  // namespace plx
