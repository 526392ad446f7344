// CSR SpMM on the tensor cores for bf16 features:  OUT[r, :] = sum_k val[k] * H[col[k], :].
//
// The CUDA-core kernel (spmm.cu) spends about 12 instructions per 16 gathered bytes per lane on
// widening bf16 and multiply-adding, and is bound by instruction issue.  Here the gathered rows
// never enter the register file as data: a warp streams the nonzeros of its rows through a ring
// in shared memory, 16 nonzeros per stage, filled by asynchronous 16-byte copies (cp.async, one
// commit group per stage; the warp stalls in cp.async.wait_group, it does not poll), and the
// weighted sums are formed by warp-level MMAs:
//
//     C[16 features x 8] += A[16 features x 16 nonzeros] . B[16 nonzeros x 8]
//
// A comes from the staged rows with ldmatrix.trans.  B carries the edge weights: column 2s holds
// the high bf16 half of the weights of the nonzeros that belong to "row slot" s, column 2s+1 the
// low half (hi + lo keeps 16 mantissa bits of the fp32 weight), zeros elsewhere.  The four slots
// are four consecutive output rows (slot = row & 3), so a stage may span row boundaries: the
// nonzeros of a warp's rows are one contiguous range of the CSR arrays and are consumed as a flat
// stream, whatever the row lengths.  Accumulators stay in registers until four rows are open,
// then go through a small exchange area in shared memory and leave as 16-byte stores (with the
// optional ReLU-derivative mask and the optional stores into the peers' receive slots).
//
// tcgen05 is not used: its accumulator is a 128-lane tile in tensor memory shared by a CTA, while
// this product needs an independent accumulator per output row and 16 x 8 tiles.  One bulk copy
// (cp.async.bulk) per gathered row was measured too: the copy engine takes about 20 cycles per
// copy and SM whatever the size, which is slower than the 16-byte copies for rows of 96-512 bytes.
//
// Reference call sites replaced: plexus/gcn_conv.py:98,188,265 (torch.sparse.mm -> cuSPARSE, fp32).

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <climits>

#include "../include/plexus_kernels.h"
#include "../include/ptx_sm100.cuh"
#include "../include/spmm_tile_reduce.cuh"

namespace plx {

namespace {

constexpr int KB = 16;  // nonzeros per stage = K of the MMA
constexpr int KERNEL_ID_SPMM_MMA = 7;
constexpr int MAX_STAGES = 8;

// VEC: 16-byte pieces per feature row (D = 8 * VEC); MB: 16-feature blocks the MMAs cover.
template <int VEC>
struct Cfg {
  static constexpr int MB = (VEC + 1) / 2;
  static constexpr int ROW_BYTES = MB * 32;                // staged row, features padded to 16
  static constexpr int PITCH = ROW_BYTES + 16;             // odd number of 16-byte units: no bank conflicts
  static constexpr int STAGE_BYTES = KB * PITCH;
  static constexpr int XP = MB * 16 + 8;                   // floats per slot of the exchange area
  static constexpr int XCH_BYTES = 4 * XP * 4;
  static constexpr int BT_BYTES = KB * 16;                 // weight tile: 8 bf16 per nonzero
  __host__ __device__ static constexpr int warp_bytes(int stages) {
    return stages * STAGE_BYTES + XCH_BYTES + BT_BYTES;
  }
};

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t addr, uint32_t& r0, uint32_t& r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];"
               : "=r"(r0), "=r"(r1)
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
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Wait until at most `n` of this thread's most recent commit groups are still in flight (n < 8).
__device__ __forceinline__ void cp_async_wait_pending(int n) {
  switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
  }
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&a)[8]) {
  uint4 o;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
  return o;
}
__device__ __forceinline__ void mask_bf16x8(float (&a)[8], const uint4& m) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&m);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(p[i]);
    if (!(f.x > 0.f)) a[2 * i] = 0.f;
    if (!(f.y > 0.f)) a[2 * i + 1] = 0.f;
  }
}

// Store 8 result columns of output row `orow` (+ the fused-collective stores, see PushTargets).
__device__ __forceinline__ void store_vec(__nv_bfloat16* __restrict__ out, int64_t ldo, int64_t orow, int c,
                                          const uint4& packed, const PushTargets& push) {
  if (push.seg_rows > 0) {
    const int owner = static_cast<int>(orow / push.seg_rows);
    if (owner != push.me) {
      const int idx = owner - (owner > push.me ? 1 : 0);
      void* sel = push.base[0];
#pragma unroll
      for (int q = 1; q < MAX_PEERS; ++q)
        if (idx == q) sel = push.base[q];
      const int64_t slot_row = orow - static_cast<int64_t>(owner) * push.seg_rows;
      if (push_in_bounds(push.limit_elems, push.status, KERNEL_ID_SPMM_MMA, slot_row * push.ld + c, 8, orow, c))
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(sel) + slot_row * push.ld + c) = packed;
      return;
    }
    *reinterpret_cast<uint4*>(out + orow * ldo + c) = packed;
    return;
  }
  *reinterpret_cast<uint4*>(out + orow * ldo + c) = packed;
  if (push.n > 0 && !push_in_bounds(push.limit_elems, push.status, KERNEL_ID_SPMM_MMA, orow * push.ld + c, 8, orow, c))
    return;
#pragma unroll
  for (int q = 0; q < MAX_PEERS; ++q)
    if (q < push.n)
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(push.base[q]) + orow * push.ld + c) = packed;
}

// VEC: 16-byte pieces per feature row (D = 8 * VEC), a compile-time constant so that the piece ->
// (nonzero, column) mapping of the staging copies costs no division.
template <int VEC>
__global__ void __launch_bounds__(256, 2)
spmm_mma_kernel(const int* __restrict__ rowptr, const int* __restrict__ col, const float* __restrict__ val,
                const __nv_bfloat16* __restrict__ H, int64_t ldh, __nv_bfloat16* __restrict__ out,
                int64_t ldo, const __nv_bfloat16* __restrict__ mask, int64_t ldm, int D, int row_begin,
                const int4* __restrict__ items, int num_items, const int* __restrict__ long_piece_start,
                int* __restrict__ long_counter, float* __restrict__ scratch, const PushTargets push, int stages,
                int* status, const TileReduce red, int out_rows) {
  using C = Cfg<VEC>;
  constexpr int MB = C::MB;
  // with the in-kernel all-reduce the mask is applied after the sum, not to the pushed partials
  const __nv_bfloat16* flush_mask = red.n > 0 ? nullptr : mask;
  extern __shared__ __align__(128) uint8_t spmm_mma_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int wpb = blockDim.x >> 5;
  uint8_t* ws = spmm_mma_smem + warp * C::warp_bytes(stages);
  float* xch = reinterpret_cast<float*>(ws + stages * C::STAGE_BYTES);
  uint8_t* bt = reinterpret_cast<uint8_t*>(xch) + C::XCH_BYTES;
  const uint32_t stage0 = smem_u32(ws);
  const uint32_t bt_addr = smem_u32(bt);

  // staged rows a short stage leaves unwritten, and the padding columns, must hold finite values
  for (int i = lane; i < stages * C::STAGE_BYTES / 16; i += 32) reinterpret_cast<uint4*>(ws)[i] = make_uint4(0, 0, 0, 0);
  __syncwarp();

  constexpr int vec = VEC;
  const uint32_t ldh32 = static_cast<uint32_t>(ldh);
  // flush mapping: `vec` lanes write one row, 32 / vec rows at a time
  const int rows_per_iter = 32 / vec;      // >= 1 because D <= 256
  const int f_row = lane / vec, f_v = lane - f_row * vec;
  const bool f_active = f_row < rows_per_iter;
  // ldmatrix.x4.trans row addresses: see the four 8x8 blocks (k 0-7 / 8-15) x (feature 0-7 / 8-15)
  const uint32_t ldm_off = ((lane & 7) + ((lane & 16) ? 8 : 0)) * C::PITCH + ((lane & 8) ? 16 : 0);

  int pos = 0;  // ring stage of the next stage to consume
  bool ok = true;

  // in-kernel all-reduce (red.n > 0): see spmm_tile_reduce.cuh
  tile_reduce::Reducer reducer(red, out, ldo, mask, ldm, push.ld, D, out_rows, lane, KERNEL_ID_SPMM_MMA);

  const int warp_global = blockIdx.x * wpb + warp;
  const int warps_total = gridDim.x * wpb;
  for (int b = warp_global; b < num_items && ok; b += warps_total) {
    // work item: a block of whole rows {rb, re, -, -}, or one piece of a long row
    // {row, -(long id + 1), first nonzero, last nonzero + 1}; the pieces come first in the list and
    // the index of a piece is also the index of its fp32 partial row in `scratch`
    const int4 item = __ldg(items + b);
    const bool piece = item.y < 0;
    const int rb = item.x, re = piece ? item.x + 1 : item.y;
    const int nb = piece ? item.z : __ldg(rowptr + rb), ne = piece ? item.w : __ldg(rowptr + re);
    const int nbatch = (ne - nb + KB - 1) / KB;

    float c[MB][4];
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
      for (int i = 0; i < 4; ++i) c[m][i] = 0.f;

    // ---- issue stage `bi` of the block (nonzeros [i0, i0 + 16)) into ring stage `s`: piece q of
    //      the stage is 16 bytes number q % VEC of the row gathered for nonzero q / VEC; lanes 0..15
    //      pass the column index of their nonzero.  One commit group per call, also when empty.
    auto issue = [&](int bi, int s, int my_col) {
      const uint32_t st_addr = stage0 + s * C::STAGE_BYTES;
      const int cnt = bi < nbatch ? min(KB, ne - (nb + bi * KB)) : 0;
      constexpr int ITER = (KB * VEC + 31) / 32;
#pragma unroll
      for (int t = 0; t < ITER; ++t) {
        const int q = t * 32 + lane;
        const int k = q / VEC, v = q - k * VEC;
        const int ck = __shfl_sync(0xffffffffu, my_col, k & 15);
        if (k < cnt)
          cp_async16(st_addr + k * C::PITCH + v * 16,
                     H + static_cast<uint64_t>(static_cast<uint32_t>(ck)) * ldh32 + v * 8);
      }
      cp_async_commit();
    };

    // ---- prologue: fill the ring
    const int pre = min(stages, nbatch);
    {
      int s = pos;
      for (int bi = 0; bi < stages; ++bi) {  // always `stages` groups, the ones beyond the block empty
        const int i = nb + bi * KB + lane;
        const int my_col = (lane < KB && i < ne) ? __ldg(col + i) : 0;
        issue(bi, s, my_col);
        s = s + 1 == stages ? 0 : s + 1;
      }
    }
    // column indices of the stage that will be issued next, and weights of the stage consumed next
    int col_next = 0;
    {
      const int i = nb + pre * KB + lane;
      if (pre < nbatch && lane < KB && i < ne) col_next = __ldg(col + i);
    }
    float val_cur = 0.f;
    {
      const int i = nb + lane;
      if (lane < KB && i < ne) val_cur = __ldg(val + i);
    }

    int rf = rb;                    // first row whose result has not been written yet
    int lo = nb;                    // rowptr[rf]
    int E0, E1, E2, E3;             // rowptr[rf + 1 .. rf + 4] (INT_MAX beyond the block)
    auto load_ends = [&]() {
      // a piece is a single open row: nothing of it ends inside the piece
      E0 = !piece && rf + 1 <= re ? __ldg(rowptr + rf + 1) : INT_MAX;
      E1 = !piece && rf + 2 <= re ? __ldg(rowptr + rf + 2) : INT_MAX;
      E2 = !piece && rf + 3 <= re ? __ldg(rowptr + rf + 3) : INT_MAX;
      E3 = !piece && rf + 4 <= re ? __ldg(rowptr + rf + 4) : INT_MAX;
    };
    load_ends();

    // ---- write rows rf .. rf + n - 1 (n <= 4) from the accumulators and clear them
    auto flush = [&](int n) {
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        xch[tig * C::XP + m * 16 + gid] = c[m][0] + c[m][1];
        xch[tig * C::XP + m * 16 + gid + 8] = c[m][2] + c[m][3];
        c[m][0] = c[m][1] = c[m][2] = c[m][3] = 0.f;
      }
      __syncwarp();
      for (int j0 = 0; j0 < n; j0 += rows_per_iter) {
        const int j = j0 + f_row;
        if (f_active && j < n) {
          const int r = rf + j;
          const float* src = xch + (r & 3) * C::XP + f_v * 8;
          const float4 x0 = *reinterpret_cast<const float4*>(src);
          const float4 x1 = *reinterpret_cast<const float4*>(src + 4);
          float a[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
          const int64_t orow = r - row_begin;
          if (flush_mask != nullptr)
            mask_bf16x8(a, __ldg(reinterpret_cast<const uint4*>(flush_mask + orow * ldm + f_v * 8)));
          store_vec(out, ldo, orow, f_v * 8, pack_bf16x8(a), push);
        }
      }
      __syncwarp();
    };

    for (int bi = 0; bi < nbatch; ++bi) {
      const int i0 = nb + bi * KB;
      const int i_mine = i0 + (lane & 15);
      const bool valid = lane < KB && i_mine < ne;
      // prefetch: weights of the next stage, columns of the stage after the one issued below
      float val_next = 0.f;
      if (bi + 1 < nbatch && lane < KB && i_mine + KB < ne) val_next = __ldg(val + i_mine + KB);
      int col_after = 0;
      {
        const int i = nb + (bi + stages + 1) * KB + lane;
        if (bi + stages + 1 < nbatch && lane < KB && i < ne) col_after = __ldg(col + i);
      }
      // weights split in two bf16 terms
      uint32_t hl;
      {
        const __nv_bfloat16 hi = __float2bfloat16_rn(val_cur);
        const __nv_bfloat16 lw = __float2bfloat16_rn(val_cur - __bfloat162float(hi));
        hl = static_cast<uint32_t>(__bfloat16_as_ushort(hi)) |
             (static_cast<uint32_t>(__bfloat16_as_ushort(lw)) << 16);
      }
      const int s = pos;
      // stage bi is the oldest of the `stages` groups in flight
      cp_async_wait_pending(stages - 1);
      __syncwarp();
      pos = s + 1 == stages ? 0 : s + 1;
      const uint32_t a_base = stage0 + s * C::STAGE_BYTES + ldm_off;

      // one pass covers the nonzeros of rows rf .. rf + 3; later rows of the stage need a flush first
      while (true) {
        const int cc = (i_mine >= E0) + (i_mine >= E1) + (i_mine >= E2) + (i_mine >= E3);
        const bool in_pass = valid && i_mine >= lo && cc < 4;
        const bool beyond = valid && cc == 4;
        if (lane < KB) {
          const int slot = (rf + cc) & 3;
          const uint32_t w = in_pass ? hl : 0u;
          *reinterpret_cast<uint4*>(bt + lane * 16) =
              make_uint4(slot == 0 ? w : 0u, slot == 1 ? w : 0u, slot == 2 ? w : 0u, slot == 3 ? w : 0u);
        }
        __syncwarp();
        uint32_t b0, b1;
        ldmatrix_x2_trans(bt_addr + (lane & 15) * 16, b0, b1);
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          uint32_t a[4];
          ldmatrix_x4_trans(a_base + m * 32, a);
          mma_bf16_16816(c[m], a, b0, b1);
        }
        if (!__any_sync(0xffffffffu, beyond)) break;
        // rows rf .. rf + 3 are complete (a later row has started): write them and move the window
        flush(4);
        rf += 4;
        lo = E3;
        load_ends();
      }

      // the stage is free again: refill it with stage bi + stages (an empty group past the end)
      __syncwarp();
      issue(bi + stages, s, col_next);
      col_next = col_after;
      val_cur = val_next;
    }
    if (!piece) {
      // ---- end of the block: write what is still open (and any trailing empty rows)
      while (rf < re) {
        flush(min(4, re - rf));
        rf += 4;
      }
      if (red.n > 0) reducer.publish(rb - row_begin, re - row_begin);
    } else {
      // ---- end of a piece: fp32 partial row to scratch; the warp that delivers the last piece of
      //      the row sums all pieces in index order (the same order whoever comes last) and writes it
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        xch[tig * C::XP + m * 16 + gid] = c[m][0] + c[m][1];
        xch[tig * C::XP + m * 16 + gid + 8] = c[m][2] + c[m][3];
      }
      __syncwarp();
      if (lane < vec) {
        const float* src = xch + (rb & 3) * C::XP + lane * 8;
        float* dst = scratch + static_cast<int64_t>(b) * D + lane * 8;
        *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
        *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<const float4*>(src + 4);
      }
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
        if (lane < vec) {
          float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int pp = p0; pp < p1; ++pp) {
            const float* src = scratch + static_cast<int64_t>(pp) * D + lane * 8;
            float4 x0, x1;
            asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x0.x), "=f"(x0.y), "=f"(x0.z), "=f"(x0.w) : "l"(src));
            asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x1.x), "=f"(x1.y), "=f"(x1.z), "=f"(x1.w) : "l"(src + 4));
            a[0] += x0.x; a[1] += x0.y; a[2] += x0.z; a[3] += x0.w;
            a[4] += x1.x; a[5] += x1.y; a[6] += x1.z; a[7] += x1.w;
          }
          const int64_t orow = rb - row_begin;
          if (flush_mask != nullptr)
            mask_bf16x8(a, __ldg(reinterpret_cast<const uint4*>(flush_mask + orow * ldm + lane * 8)));
          store_vec(out, ldo, orow, lane * 8, pack_bf16x8(a), push);
        }
        if (lane == 0) long_counter[L] = 0;  // ready for the next launch on this matrix
        if (red.n > 0) reducer.publish(rb - row_begin, rb - row_begin + 1);
      }
    }
    if (red.n > 0) {
      reducer.poll(false);
      ok = ok && reducer.ok;
    }
  }
  if (red.n > 0 && ok) reducer.finish();
}

template <int VEC>
const char* launch_one(const int* rowptr, const int* col, const float* val, const __nv_bfloat16* H, int64_t ldh,
                       __nv_bfloat16* out, int64_t ldo, const __nv_bfloat16* mask, int64_t ldm, int D,
                       int row_begin, const int4* items, int num_items, const int* long_piece_start,
                       int* long_counter, float* scratch, const PushTargets& push,
                       int* status, const TileReduce& red, int out_rows, int stages_override,
                       cudaStream_t stream) {
  using C = Cfg<VEC>;
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // about 8 KB of gathered rows in flight per warp
  int stages = 8192 / (KB * D * 2) + 1;
  stages = std::max(3, std::min(MAX_STAGES, stages));
  if (stages_override > 0) stages = std::max(2, std::min(MAX_STAGES, stages_override));
  const int limit = 232448;
  // warps per SM: bounded by shared memory and by registers (128 per thread -> 16 warps)
  const int wb = C::warp_bytes(stages);
  int best_w = 1, best_ctas = 1, best_total = 0;
  for (int ctas = 1; ctas <= 4; ++ctas) {
    int w = std::min(8, (limit / ctas - 1024) / wb);
    if (w < 1) continue;
    const int total = std::min(w * ctas, 16);
    if (total > best_total) {
      best_total = total;
      best_w = std::min(w, (total + ctas - 1) / ctas);
      best_ctas = ctas;
    }
  }
  const size_t smem = static_cast<size_t>(best_w) * wb;
  auto kern = spmm_mma_kernel<VEC>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  const int grid = std::max(1, std::min(sms * best_ctas, (num_items + best_w - 1) / best_w));
  kern<<<grid, best_w * 32, smem, stream>>>(rowptr, col, val, H, ldh, out, ldo, mask, ldm, D, row_begin,
                                            items, num_items, long_piece_start, long_counter, scratch, push,
                                            stages, status, red, out_rows);
  return last_launch_error();
}

const char* dispatch_vec(int vec, const int* rowptr, const int* col, const float* val, const __nv_bfloat16* H,
                         int64_t ldh, __nv_bfloat16* out, int64_t ldo, const __nv_bfloat16* mask, int64_t ldm,
                         int D, int row_begin, const int4* items, int num_items, const int* long_piece_start,
                         int* long_counter, float* scratch, const PushTargets& push,
                         int* status, const TileReduce& red, int out_rows, int stages, cudaStream_t stream) {
#define PLX_VEC(N)                                                                                           \
  case N:                                                                                                    \
    return launch_one<N>(rowptr, col, val, H, ldh, out, ldo, mask, ldm, D, row_begin, items, num_items,     \
                         long_piece_start, long_counter, scratch, push, status, red, out_rows, stages, stream)
  switch (vec) {
    PLX_VEC(1); PLX_VEC(2); PLX_VEC(3); PLX_VEC(4); PLX_VEC(5); PLX_VEC(6); PLX_VEC(7); PLX_VEC(8);
    PLX_VEC(9); PLX_VEC(10); PLX_VEC(11); PLX_VEC(12); PLX_VEC(13); PLX_VEC(14); PLX_VEC(15); PLX_VEC(16);
    PLX_VEC(17); PLX_VEC(18); PLX_VEC(19); PLX_VEC(20); PLX_VEC(21); PLX_VEC(22); PLX_VEC(23); PLX_VEC(24);
    PLX_VEC(25); PLX_VEC(26); PLX_VEC(27); PLX_VEC(28); PLX_VEC(29); PLX_VEC(30); PLX_VEC(31); PLX_VEC(32);
  }
#undef PLX_VEC
  return "spmm_mma: unsupported width";
}

}  // namespace

// Work items (see the kernel): the pieces of the long rows first, then blocks of whole rows; row
// numbers are those of the CSR arrays, output row = row - row_begin.  scratch holds one fp32 row of D
// columns per piece, long_counter one zero-initialised int per long row (the kernel leaves it zero).
// bf16 features, D a multiple of 8; wider matrices are processed in column chunks of 256.
// stages: depth of the shared-memory ring (0 = chosen from the row size).
const char* launch_spmm_mma(const int* rowptr, const int* col, const float* val, const void* H, int64_t ldh,
                            void* out, int64_t ldo, const void* mask, int64_t ldm, int D, int row_begin,
                            const int* items_in, int num_items, int num_pieces, const int* long_piece_start,
                            int* long_counter, float* scratch, int64_t scratch_elems,
                            const PushTargets* push_in, int stages,
                            int* status, cudaStream_t stream, const TileReduce* reduce_in, int out_rows) {
  const int4* items = reinterpret_cast<const int4*>(items_in);
  if (reinterpret_cast<uintptr_t>(items_in) % 16) return "spmm_mma: the work items must be 16-byte aligned";
  if (num_pieces > 0 && (long_piece_start == nullptr || long_counter == nullptr || scratch == nullptr ||
                         reinterpret_cast<uintptr_t>(scratch) % 16 ||
                         scratch_elems < static_cast<int64_t>(num_pieces) * D))
    return "spmm_mma: long rows need the piece index, the counters and num_pieces * D scratch floats";
  TileReduce red = {};
  if (reduce_in != nullptr && reduce_in->n > 0) {
    red = *reduce_in;
    red.status = status;
    if (push_in == nullptr || push_in->n != red.n || push_in->seg_rows != 0)
      return "spmm_mma: the in-kernel all-reduce goes with the broadcast push to the same peers";
    if (D > 256) return "spmm_mma: the in-kernel all-reduce handles at most 256 columns";
    for (int q = 0; q < red.n; ++q)
      if (red.slot[q] == nullptr || reinterpret_cast<uintptr_t>(red.slot[q]) % 16)
        return "spmm_mma: bad in-kernel all-reduce description";
  }
  PushTargets push = {};
  if (push_in != nullptr) {
    push = *push_in;
    if (push.n < 0 || push.n > MAX_PEERS || push.ld % 8) return "spmm_mma: bad push targets";
    if (push.seg_rows < 0 || (push.seg_rows > 0 && (push.me < 0 || push.me > push.n)))
      return "spmm_mma: bad reduce-scatter push description";
    for (int q = 0; q < push.n; ++q)
      if (reinterpret_cast<uintptr_t>(push.base[q]) % 16) return "spmm_mma: push targets must be 16-byte aligned";
  }
  if (D % 8 || ldh % 8 || ldo % 8 || (mask && ldm % 8)) return "spmm_mma: feature rows must be multiples of 16 bytes";
  if (ldh < 0 || ldh > 0x7fffffffLL) return "spmm_mma: leading dimension of H out of range";
  if (reinterpret_cast<uintptr_t>(H) % 16 || reinterpret_cast<uintptr_t>(out) % 16 ||
      reinterpret_cast<uintptr_t>(mask) % 16)
    return "spmm_mma: feature pointers must be 16-byte aligned";
  if (D == 0 || num_items == 0) return nullptr;
  if (num_pieces > 0 && D > 256) return "spmm_mma: long rows with more than 256 columns are not handled here";
  const __nv_bfloat16* Hb = static_cast<const __nv_bfloat16*>(H);
  __nv_bfloat16* ob = static_cast<__nv_bfloat16*>(out);
  const __nv_bfloat16* mb_ptr = static_cast<const __nv_bfloat16*>(mask);
  for (int c0 = 0; c0 < D; c0 += 256) {
    const int d = std::min(256, D - c0);
    PushTargets p = push;
    for (int q = 0; q < p.n; ++q) p.base[q] = static_cast<__nv_bfloat16*>(p.base[q]) + c0;
    const char* e = dispatch_vec(d / 8, rowptr, col, val, Hb + c0, ldh, ob + c0, ldo, mb_ptr ? mb_ptr + c0 : nullptr,
                                 ldm, d, row_begin, items, num_items, long_piece_start, long_counter, scratch, p,
                                 status, red, out_rows, stages, stream);
    if (e) return e;
  }
  return nullptr;
}

}  // namespace plx
