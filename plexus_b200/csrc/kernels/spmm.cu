// CSR SpMM  OUT[r0:r1, :] = A[r0:r1, :] . H   with bf16 (or fp32) features, fp32 accumulation, on
// the CUDA cores (the tensor-core variant for bf16 features is in spmm_mma.cu).
//
// The op is bound by the gather of feature rows (each nonzero pulls one 2*D-byte row of H), so
// the kernel is organised around memory-level parallelism:
//   * one warp per row; the warp is split in G = 32/LPR groups of LPR lanes, a group reads one
//     feature row with 16-byte loads (LPR*VPL vectors cover the D columns), different groups
//     take different nonzeros of the row, and each group keeps several nonzeros in flight;
//   * column indices / values are read coalesced, 32 at a time, and broadcast by shuffles;
//   * load balance on power-law graphs comes from a per-matrix list of work items built once on
//     the device: blocks of consecutive rows of about equal cost (nonzeros + a per-row constant),
//     and, first in the list, the pieces of rows longer than a threshold.  A piece is accumulated
//     by one warp into an fp32 partial row in scratch memory; the warp that delivers the last piece
//     of a row sums the pieces in index order (the same order whoever comes last) and stores the
//     row.  Everything runs in ONE launch;
//   * the epilogue optionally multiplies by (mask > 0): that is the ReLU derivative of the
//     layer input, applied where the input gradient is produced;
//   * fused collectives: every finished row can also be stored into receive slots in other GPUs'
//     memory (PushTargets), and the all-reduce can be finished inside the kernel (TileReduce, see
//     spmm_tile_reduce.cuh).
//
// Reference call sites replaced: plexus/gcn_conv.py:98,188,265 (torch.sparse.mm -> cuSPARSE, fp32).

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <type_traits>

#include "../include/plexus_kernels.h"
#include "../include/spmm_tile_reduce.cuh"

namespace plx {

constexpr int SPMM_WARPS = 8;
constexpr int KERNEL_ID_SPMM = 1;

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
        if (peer != nullptr &&
            !push_in_bounds(push.limit_elems, push.status, KERNEL_ID_SPMM, slot_row * push.ld + c, VN, orow, c))
          continue;
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
      if (push.n > 0 &&
          !push_in_bounds(push.limit_elems, push.status, KERNEL_ID_SPMM, orow * push.ld + c, VN, orow, c))
        continue;
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


#ifndef PLX_SPMM_MINB
#define PLX_SPMM_MINB 4
#endif

// acc = sum of the fp32 partial rows of pieces [p0, p1), in index order.
template <typename T, int LPR, int VPL>
__device__ __forceinline__ void sum_pieces(const float* __restrict__ scratch, int p0, int p1, int lane,
                                           float (&acc)[VPL][Vec16<T>::N]) {
  constexpr int VN = Vec16<T>::N;
  constexpr int W = LPR * VPL * VN;
  zero_acc(acc);
  if (lane < LPR) {
    for (int p = p0; p < p1; ++p) {
      const float* src = scratch + static_cast<int64_t>(p) * W;
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
#pragma unroll
        for (int k = 0; k < VN; k += 4) {
          const float4 f = __ldcg(reinterpret_cast<const float4*>(src + (v * LPR + lane) * VN + k));
          acc[v][k] += f.x;
          acc[v][k + 1] += f.y;
          acc[v][k + 2] += f.z;
          acc[v][k + 3] += f.w;
        }
      }
    }
  }
}

// Second launch of the plain (not fused) form: one warp per long row sums its pieces and stores it.
template <typename T, int LPR, int VPL>
__global__ void __launch_bounds__(SPMM_WARPS * 32)
spmm_long_rows_kernel(const int4* __restrict__ items, const int* __restrict__ long_piece_start, int num_long,
                      const float* __restrict__ scratch, T* __restrict__ out, int64_t ldo,
                      const T* __restrict__ mask, int64_t ldm, int D, int row_begin, const PushTargets push) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int warps_total = gridDim.x * wpb;
  for (int L = blockIdx.x * wpb + (threadIdx.x >> 5); L < num_long; L += warps_total) {
    const int p0 = __ldg(long_piece_start + L), p1 = __ldg(long_piece_start + L + 1);
    float acc[VPL][Vec16<T>::N];
    sum_pieces<T, LPR, VPL>(scratch, p0, p1, lane, acc);
    const int64_t orow = __ldg(items + p0).x - row_begin;  // every piece item carries its row
    row_store<T, LPR, VPL>(out + orow * ldo, mask ? mask + orow * ldm : nullptr, D, lane, acc, push, orow);
  }
}

// Work items, 4 ints each (built by ops/cuda.py): first the pieces of the long rows
// {row, -(long id + 1), first nonzero, last nonzero + 1} - the index of a piece is also the index of
// its fp32 partial row (W = LPR * VPL * VN floats) in `scratch` - then blocks of whole rows
// {first row, last row + 1, 0, 0}.  Warps take items round-robin.
// FUSED: with the in-kernel all-reduce (bf16 only); a separate instantiation so that the plain
// kernel carries none of its code or registers.
template <typename T, int LPR, int VPL, bool FUSED>
__global__ void __launch_bounds__(SPMM_WARPS * 32, VPL == 1 ? PLX_SPMM_MINB : 2)
spmm_items_kernel(const int* __restrict__ rowptr, const int* __restrict__ col, const float* __restrict__ val,
                  const T* __restrict__ H, int64_t ldh, T* __restrict__ out, int64_t ldo,
                  const T* __restrict__ mask, int64_t ldm, int D, int row_begin,
                  const int4* __restrict__ items, int num_items, const int* __restrict__ long_piece_start,
                  int num_long, int* __restrict__ long_counter, float* __restrict__ scratch,
                  const PushTargets push, const TileReduce red, int out_rows) {
  constexpr int VN = Vec16<T>::N;
  constexpr int W = LPR * VPL * VN;
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int warp_global = blockIdx.x * wpb + (threadIdx.x >> 5);
  const int warps_total = gridDim.x * wpb;
  // with the in-kernel all-reduce the mask is applied after the sum, not to the pushed partials
  constexpr bool fused_reduce = FUSED;
  const T* store_mask = fused_reduce ? nullptr : mask;
  tile_reduce::Reducer reducer(red, reinterpret_cast<__nv_bfloat16*>(out), ldo,
                               reinterpret_cast<const __nv_bfloat16*>(mask), ldm, push.ld, D, out_rows, lane,
                               KERNEL_ID_SPMM);
  // The first item of a warp is its own index; the following ones are handed out by a counter, so
  // that a warp with cheap items takes more of them (the items are sorted by falling cost: pieces,
  // then blocks).  Which warp computes an item has no influence on the result.
  int* work_next = long_counter + num_long;  // {next item - warps_total, warps that are done}
  for (int b = warp_global; b < num_items && (!FUSED || reducer.ok);) {
    const int4 item = __ldg(items + b);
    if (item.y >= 0) {
      for (int row = item.x; row < item.y; ++row) {
        const int64_t beg = __ldg(rowptr + row), end = __ldg(rowptr + row + 1);
        float acc[VPL][VN];
        zero_acc(acc);
        row_accumulate<T, LPR, VPL>(col, val, H, ldh, D, beg, end, lane, acc);
        const int64_t orow = row - row_begin;
        row_store<T, LPR, VPL>(out + orow * ldo, store_mask ? store_mask + orow * ldm : nullptr, D, lane, acc,
                               push, orow);
      }
      if constexpr (FUSED) reducer.publish(item.x - row_begin, item.y - row_begin);
    } else {
      float acc[VPL][VN];
      zero_acc(acc);
      row_accumulate<T, LPR, VPL>(col, val, H, ldh, D, item.z, item.w, lane, acc);
      if (lane < LPR) {
        float* dst = scratch + static_cast<int64_t>(b) * W;
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
          float4* d4 = reinterpret_cast<float4*>(dst + (v * LPR + lane) * VN);
#pragma unroll
          for (int i = 0; i < VN; i += 4) d4[i / 4] = make_float4(acc[v][i], acc[v][i + 1], acc[v][i + 2], acc[v][i + 3]);
        }
      }
      if constexpr (FUSED) {
        // one launch: the warp that delivers the last piece of a row sums all pieces in index order
        // (the same order whoever comes last) and stores the row
        __syncwarp();
        const int L = -item.y - 1;
        const int p0 = __ldg(long_piece_start + L), p1 = __ldg(long_piece_start + L + 1);
        int last = 0;
        if (lane == 0) {
          __threadfence();
          last = atomicAdd(long_counter + L, 1) == p1 - p0 - 1;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          __threadfence();
          sum_pieces<T, LPR, VPL>(scratch, p0, p1, lane, acc);
          const int64_t orow = item.x - row_begin;
          row_store<T, LPR, VPL>(out + orow * ldo, store_mask ? store_mask + orow * ldm : nullptr, D, lane, acc,
                                 push, orow);
          if (lane == 0) long_counter[L] = 0;  // ready for the next launch on this matrix
          reducer.publish(item.x - row_begin, item.x - row_begin + 1);
        }
      }
      // otherwise the long rows are finished by spmm_long_rows_kernel, launched right after
    }
    if constexpr (FUSED) reducer.poll(false);
    if (lane == 0) b = atomicAdd(work_next, 1) + warps_total;
    b = __shfl_sync(0xffffffffu, b, 0);
  }
  if constexpr (FUSED) reducer.finish();
  // the last warp to leave zeroes the counters for the next launch on this matrix
  if (lane == 0 && atomicAdd(work_next + 1, 1) == warps_total - 1) {
    work_next[0] = 0;
    work_next[1] = 0;
  }
}

static int spmm_grid(int work_items, int warps_per_block, int blocks_per_sm) {
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return std::max(1, std::min(sms * blocks_per_sm, (work_items + warps_per_block - 1) / warps_per_block));
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
                                 int64_t ldh, T* out, int64_t ldo, const T* mask, int64_t ldm, int row_begin,
                                 const int4* items, int num_items, const int* long_piece_start, int num_long,
                                 int* long_counter, float* scratch, const PushTargets& push,
                                 const TileReduce& red, int out_rows, cudaStream_t stream) {
  constexpr int VN = Vec16<T>::N;
  const int vecs = (D + VN - 1) / VN;  // 16-byte vectors per feature row
  constexpr bool CAN_FUSE = std::is_same<T, __nv_bfloat16>::value;
#define PLX_SPMM(LPR, VPL)                                                                                     \
  do {                                                                                                         \
    if (CAN_FUSE && red.n > 0)                                                                                 \
      spmm_items_kernel<T, LPR, VPL, CAN_FUSE><<<spmm_grid(num_items, SPMM_WARPS, 8), SPMM_WARPS * 32, 0,     \
                                                 stream>>>(rowptr, col, val, H, ldh, out, ldo, mask, ldm, D,  \
                                                           row_begin, items, num_items, long_piece_start,     \
                                                           num_long, long_counter, scratch, push, red,        \
                                                           out_rows);                                          \
    else {                                                                                                     \
      spmm_items_kernel<T, LPR, VPL, false><<<spmm_grid(num_items, SPMM_WARPS, 8), SPMM_WARPS * 32, 0,        \
                                              stream>>>(rowptr, col, val, H, ldh, out, ldo, mask, ldm, D,     \
                                                        row_begin, items, num_items, long_piece_start,        \
                                                        num_long, long_counter, scratch, push, red,           \
                                                        out_rows);                                             \
      if (num_long > 0)                                                                                        \
        spmm_long_rows_kernel<T, LPR, VPL><<<spmm_grid(num_long, SPMM_WARPS, 8), SPMM_WARPS * 32, 0,          \
                                             stream>>>(items, long_piece_start, num_long, scratch, out, ldo,  \
                                                       mask, ldm, D, row_begin, push);                        \
    }                                                                                                          \
  } while (0)
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

// out[r - row_begin] = A[r, :] . H for the rows covered by the work items (optionally masked).
const char* launch_spmm_csr(int dtype, const int* rowptr, const int* col, const float* val,
                            const void* H, int64_t ldh, void* out, int64_t ldo, const void* mask,
                            int64_t ldm, int D, int row_begin, const int* items_in, int num_items,
                            int num_pieces, const int* long_piece_start, int num_long, int* long_counter,
                            float* scratch, int64_t scratch_elems, const PushTargets* push_in,
                            cudaStream_t stream, const TileReduce* reduce_in, int out_rows) {
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
  TileReduce red = {};
  if (reduce_in != nullptr && reduce_in->n > 0) {
    red = *reduce_in;
    if (dtype != DT_BF16) return "spmm: the in-kernel all-reduce needs bf16 features";
    if (push_in == nullptr || push_in->n != red.n || push_in->seg_rows != 0)
      return "spmm: the in-kernel all-reduce goes with the broadcast push to the same peers";
    if (D % 8) return "spmm: bad in-kernel all-reduce description";
    for (int q = 0; q < red.n; ++q)
      if (red.slot[q] == nullptr || reinterpret_cast<uintptr_t>(red.slot[q]) % 16)
        return "spmm: bad in-kernel all-reduce description";
  }
  if ((ldh * esz) % 16 || (ldo * esz) % 16 || (D * esz) % 16 || (mask && (ldm * esz) % 16))
    return "spmm: feature rows must be multiples of 16 bytes";
  if (ldh < 0 || ldh > 0x7fffffffLL) return "spmm: leading dimension of H out of range";
  if (reinterpret_cast<uintptr_t>(H) % 16 || reinterpret_cast<uintptr_t>(out) % 16 ||
      reinterpret_cast<uintptr_t>(mask) % 16 || reinterpret_cast<uintptr_t>(scratch) % 16 ||
      reinterpret_cast<uintptr_t>(items_in) % 16)
    return "spmm: feature pointers and work items must be 16-byte aligned";
  if (D == 0 || num_items == 0) return nullptr;
  if (long_counter == nullptr) return "spmm: the counters (long rows + 2 zeros) are missing";
  if (num_pieces > 0 && (long_piece_start == nullptr || scratch == nullptr ||
                         scratch_elems < static_cast<int64_t>(num_pieces) * spmm_scratch_per_piece(dtype, D)))
    return "spmm: long rows need the piece index, the counters and scratch for the pieces";
  const int4* items = reinterpret_cast<const int4*>(items_in);
  if (dtype == DT_BF16)
    return dispatch_spmm<__nv_bfloat16>(D, rowptr, col, val, reinterpret_cast<const __nv_bfloat16*>(H),
                                        ldh, reinterpret_cast<__nv_bfloat16*>(out), ldo,
                                        reinterpret_cast<const __nv_bfloat16*>(mask), ldm, row_begin, items,
                                        num_items, long_piece_start, num_long, long_counter, scratch, push, red,
                                        out_rows, stream);
  if (dtype == DT_F32)
    return dispatch_spmm<float>(D, rowptr, col, val, reinterpret_cast<const float*>(H), ldh,
                                reinterpret_cast<float*>(out), ldo, reinterpret_cast<const float*>(mask),
                                ldm, row_begin, items, num_items, long_piece_start, num_long, long_counter, scratch,
                                push, red, out_rows, stream);
  return "spmm: features must be bf16 or fp32";
}

}  // namespace plx
