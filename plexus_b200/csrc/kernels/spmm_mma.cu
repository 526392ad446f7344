// CSR SpMM on the tensor cores for bf16 features:  OUT[r, :] = sum_k val[k] * H[col[k], :].
//
// The CUDA-core kernel (spmm.cu) spends about 12 instructions per 16 gathered bytes per lane on
// widening bf16 and multiply-adding, and is bound by instruction issue.  Here the gathered rows
// never enter the register file as data: a warp streams the nonzeros of its rows through a ring
// in shared memory, 16 nonzeros per stage, filled asynchronously either by one bulk copy per
// gathered row (cp.async.bulk, one lane issues a whole row, completion counted in bytes on an
// mbarrier) or by 16-byte cp.async copies, and the weighted sums are formed by warp-level MMAs:
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
// this product needs an independent accumulator per output row and 16 x 8 tiles.
//
// Reference call sites replaced: plexus/gcn_conv.py:98,188,265 (torch.sparse.mm -> cuSPARSE, fp32).

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <climits>

#include "../include/plexus_kernels.h"
#include "../include/ptx_sm100.cuh"

namespace plx {

namespace {

constexpr int KB = 16;  // nonzeros per stage = K of the MMA
constexpr int KERNEL_ID_SPMM_MMA = 7;
constexpr int MAX_STAGES = 8;

template <int MB>
struct Cfg {
  static constexpr int ROW_BYTES = MB * 32;                // staged row, features padded to 16
  static constexpr int PITCH = ROW_BYTES + 16;             // odd number of 16-byte units: no bank conflicts
  static constexpr int STAGE_BYTES = KB * PITCH;
  static constexpr int XP = MB * 16 + 8;                   // floats per slot of the exchange area
  static constexpr int XCH_BYTES = 4 * XP * 4;
  static constexpr int BT_BYTES = KB * 16;                 // weight tile: 8 bf16 per nonzero
  static constexpr int BAR_BYTES = MAX_STAGES * 8;
  __host__ __device__ static constexpr int warp_bytes(int stages) {
    return stages * STAGE_BYTES + XCH_BYTES + BT_BYTES + BAR_BYTES;
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
// One gathered row: global -> shared, completion in bytes on an mbarrier of this CTA (no multicast).
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// The mbarrier receives one arrival from this thread when all its earlier cp.async have landed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_addr(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait_addr(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < PLX_WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
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
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(sel) + slot_row * push.ld + c) = packed;
      return;
    }
    *reinterpret_cast<uint4*>(out + orow * ldo + c) = packed;
    return;
  }
  *reinterpret_cast<uint4*>(out + orow * ldo + c) = packed;
#pragma unroll
  for (int q = 0; q < MAX_PEERS; ++q)
    if (q < push.n)
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(push.base[q]) + orow * push.ld + c) = packed;
}

// MB: number of 16-feature blocks (D <= 16 * MB).  BULK: one bulk copy per gathered row instead of
// 16-byte cp.async copies.
template <int MB, bool BULK>
__global__ void __launch_bounds__(256)
spmm_mma_kernel(const int* __restrict__ rowptr, const int* __restrict__ col, const float* __restrict__ val,
                const __nv_bfloat16* __restrict__ H, int64_t ldh, __nv_bfloat16* __restrict__ out,
                int64_t ldo, const __nv_bfloat16* __restrict__ mask, int64_t ldm, int D, int row_begin,
                const int* __restrict__ block_start, int num_blocks, const PushTargets push, int stages,
                int* status) {
  using C = Cfg<MB>;
  extern __shared__ __align__(128) uint8_t spmm_mma_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int wpb = blockDim.x >> 5;
  uint8_t* ws = spmm_mma_smem + warp * C::warp_bytes(stages);
  float* xch = reinterpret_cast<float*>(ws + stages * C::STAGE_BYTES);
  uint8_t* bt = reinterpret_cast<uint8_t*>(xch) + C::XCH_BYTES;
  const uint32_t stage0 = smem_u32(ws);
  const uint32_t bt_addr = smem_u32(bt);
  const uint32_t bar0 = bt_addr + C::BT_BYTES;

  // staged rows a short stage leaves unwritten, and the padding columns, must hold finite values
  for (int i = lane; i < stages * C::STAGE_BYTES / 16; i += 32) reinterpret_cast<uint4*>(ws)[i] = make_uint4(0, 0, 0, 0);
  if (lane < stages)
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar0 + lane * 8), "r"(BULK ? 1 : 32));
  fence_mbar_init();
  fence_proxy_async();
  __syncwarp();

  const int vec = D >> 3;                  // 16-byte pieces per feature row
  const uint32_t row_bytes = static_cast<uint32_t>(D) * 2;
  const uint32_t ldh32 = static_cast<uint32_t>(ldh);
  // flush mapping: `vec` lanes write one row, 32 / vec rows at a time
  const int rows_per_iter = 32 / vec;      // >= 1 because D <= 256
  const int f_row = lane / vec, f_v = lane - f_row * vec;
  const bool f_active = f_row < rows_per_iter;
  // ldmatrix.x4.trans row addresses: see the four 8x8 blocks (k 0-7 / 8-15) x (feature 0-7 / 8-15)
  const uint32_t ldm_off = ((lane & 7) + ((lane & 16) ? 8 : 0)) * C::PITCH + ((lane & 8) ? 16 : 0);

  int pos = 0;              // ring stage of the next stage to consume
  uint32_t phase_bits = 0;  // bit s: parity the next wait on stage s expects
  bool ok = true;

  const int warp_global = blockIdx.x * wpb + warp;
  const int warps_total = gridDim.x * wpb;
  for (int b = warp_global; b < num_blocks && ok; b += warps_total) {
    const int rb = __ldg(block_start + b), re = __ldg(block_start + b + 1);
    const int nb = __ldg(rowptr + rb), ne = __ldg(rowptr + re);
    const int nbatch = (ne - nb + KB - 1) / KB;

    float c[MB][4];
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
      for (int i = 0; i < 4; ++i) c[m][i] = 0.f;

    // ---- issue stage `bi` of the block (nonzeros [i0, i0 + 16)) into ring stage `s`;
    //      lanes 0..15 pass the column index of their nonzero
    auto issue = [&](int bi, int s, int my_col) {
      const uint32_t st_addr = stage0 + s * C::STAGE_BYTES;
      const uint32_t bar = bar0 + s * 8;
      const int i0 = nb + bi * KB;
      const int cnt = min(KB, ne - i0);
      if constexpr (BULK) {
        if (lane == 0) mbar_expect_tx_addr(bar, static_cast<uint32_t>(cnt) * row_bytes);
        __syncwarp();
        if (lane < cnt)
          bulk_copy_g2s(st_addr + lane * C::PITCH,
                        H + static_cast<uint64_t>(static_cast<uint32_t>(my_col)) * ldh32, row_bytes, bar);
      } else {
        const int pieces = cnt * vec;
        for (int q0 = 0; q0 < pieces; q0 += 32) {  // uniform trip count: every lane takes part in the shuffle
          const int q = q0 + lane;
          const int k = q / vec, v = q - k * vec;
          const int ck = __shfl_sync(0xffffffffu, my_col, k & 15);
          if (q < pieces)
            cp_async16(st_addr + k * C::PITCH + v * 16,
                       H + static_cast<uint64_t>(static_cast<uint32_t>(ck)) * ldh32 + v * 8);
        }
        cp_async_arrive_noinc(bar);
      }
    };

    // ---- prologue: fill the ring
    const int pre = min(stages, nbatch);
    {
      int s = pos;
      for (int bi = 0; bi < pre; ++bi) {
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
      E0 = rf + 1 <= re ? __ldg(rowptr + rf + 1) : INT_MAX;
      E1 = rf + 2 <= re ? __ldg(rowptr + rf + 2) : INT_MAX;
      E2 = rf + 3 <= re ? __ldg(rowptr + rf + 3) : INT_MAX;
      E3 = rf + 4 <= re ? __ldg(rowptr + rf + 4) : INT_MAX;
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
          if (mask != nullptr)
            mask_bf16x8(a, __ldg(reinterpret_cast<const uint4*>(mask + orow * ldm + f_v * 8)));
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
      if (!mbar_wait_addr(bar0 + s * 8, (phase_bits >> s) & 1u)) {
        if (lane == 0) report_status(status, ST_TIMEOUT, KERNEL_ID_SPMM_MMA, s, bi, b);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        // giving up: let the other copies already issued land before the CTA exits (bounded)
        int t = s;
        for (int bj = bi + 1; bj < min(nbatch, bi + stages); ++bj) {
          t = t + 1 == stages ? 0 : t + 1;
          mbar_wait_addr(bar0 + t * 8, (phase_bits >> t) & 1u);
        }
        break;
      }
      phase_bits ^= 1u << s;
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

      // the stage is free again: refill it with stage bi + stages
      __syncwarp();
      if (bi + stages < nbatch) {
        fence_proxy_async();
        issue(bi + stages, s, col_next);
      }
      col_next = col_after;
      val_cur = val_next;
    }
    if (!ok) break;
    // ---- end of the block: write what is still open (and any trailing empty rows)
    while (rf < re) {
      flush(min(4, re - rf));
      rf += 4;
    }
  }
}

template <int MB, bool BULK>
const char* launch_one(const int* rowptr, const int* col, const float* val, const __nv_bfloat16* H, int64_t ldh,
                       __nv_bfloat16* out, int64_t ldo, const __nv_bfloat16* mask, int64_t ldm, int D,
                       int row_begin, const int* block_start, int num_blocks, const PushTargets& push,
                       int* status, cudaStream_t stream) {
  using C = Cfg<MB>;
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // about 6 KB of gathered rows in flight per warp
  int stages = 6144 / (KB * D * 2) + 1;
  stages = std::max(3, std::min(MAX_STAGES, stages));
  const int limit = 232448;
  // warps per SM bounded by shared memory and by registers (about 128 per thread at MB = 16)
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
  auto kern = spmm_mma_kernel<MB, BULK>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  const int grid = std::max(1, std::min(sms * best_ctas, (num_blocks + best_w - 1) / best_w));
  kern<<<grid, best_w * 32, smem, stream>>>(rowptr, col, val, H, ldh, out, ldo, mask, ldm, D, row_begin,
                                            block_start, num_blocks, push, stages, status);
  return last_launch_error();
}

template <bool BULK>
const char* dispatch_mb(int mb, const int* rowptr, const int* col, const float* val, const __nv_bfloat16* H,
                        int64_t ldh, __nv_bfloat16* out, int64_t ldo, const __nv_bfloat16* mask, int64_t ldm,
                        int D, int row_begin, const int* block_start, int num_blocks, const PushTargets& push,
                        int* status, cudaStream_t stream) {
#define PLX_MB(N)                                                                                            \
  case N:                                                                                                    \
    return launch_one<N, BULK>(rowptr, col, val, H, ldh, out, ldo, mask, ldm, D, row_begin, block_start,    \
                               num_blocks, push, status, stream)
  switch (mb) {
    PLX_MB(1); PLX_MB(2); PLX_MB(3); PLX_MB(4); PLX_MB(5); PLX_MB(6); PLX_MB(7); PLX_MB(8);
    PLX_MB(9); PLX_MB(10); PLX_MB(11); PLX_MB(12); PLX_MB(13); PLX_MB(14); PLX_MB(15); PLX_MB(16);
  }
#undef PLX_MB
  return "spmm_mma: unsupported width";
}

}  // namespace

// All rows of block_start[0] .. block_start[num_blocks] (absolute row numbers of the CSR arrays);
// output row = row - row_begin.  bf16 features, D a multiple of 8; wider matrices are processed in
// column chunks of 256.  staging: 0 = 16-byte cp.async copies, 1 = one bulk copy per gathered row.
const char* launch_spmm_mma(const int* rowptr, const int* col, const float* val, const void* H, int64_t ldh,
                            void* out, int64_t ldo, const void* mask, int64_t ldm, int D, int row_begin,
                            const int* block_start, int num_blocks, const PushTargets* push_in, int staging,
                            int* status, cudaStream_t stream) {
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
  if (D == 0 || num_blocks == 0) return nullptr;
  const __nv_bfloat16* Hb = static_cast<const __nv_bfloat16*>(H);
  __nv_bfloat16* ob = static_cast<__nv_bfloat16*>(out);
  const __nv_bfloat16* mb_ptr = static_cast<const __nv_bfloat16*>(mask);
  for (int c0 = 0; c0 < D; c0 += 256) {
    const int d = std::min(256, D - c0);
    const int mb = (d + 15) / 16;
    PushTargets p = push;
    for (int q = 0; q < p.n; ++q) p.base[q] = static_cast<__nv_bfloat16*>(p.base[q]) + c0;
    const char* e = staging == 1
        ? dispatch_mb<true>(mb, rowptr, col, val, Hb + c0, ldh, ob + c0, ldo, mb_ptr ? mb_ptr + c0 : nullptr,
                            ldm, d, row_begin, block_start, num_blocks, p, status, stream)
        : dispatch_mb<false>(mb, rowptr, col, val, Hb + c0, ldh, ob + c0, ldo, mb_ptr ? mb_ptr + c0 : nullptr,
                             ldm, d, row_begin, block_start, num_blocks, p, status, stream);
    if (e) return e;
  }
  return nullptr;
}

}  // namespace plx
