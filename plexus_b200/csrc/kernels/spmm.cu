// CSR SpMM  OUT[r0:r1, :] = A[r0:r1, :] . H   with bf16 (or fp32) features, fp32 accumulation.
//
// The op is bound by the gather of feature rows (each nonzero pulls one 2*D-byte row of H), so
// the kernel is organised around memory-level parallelism:
//   * one warp per row; the warp is split in G = 32/LPR groups of LPR lanes, a group reads one
//     feature row with 16-byte loads (LPR*VPL vectors cover the D columns), different groups
//     take different nonzeros of the row, several nonzeros are in flight per group (unroll);
//   * column indices / values are read coalesced, 32 at a time, and broadcast by shuffles;
//   * rows longer than LONG_ROW nonzeros are skipped here and processed by a second launch
//     with one CTA per long row (power-law graphs have a few rows of >10K nonzeros);
//   * the epilogue optionally multiplies by (mask > 0): that is the ReLU derivative of the
//     layer input, applied where the input gradient is produced.
//
// Reference call sites replaced: plexus/gcn_conv.py:98,188,265 (torch.sparse.mm -> cuSPARSE, fp32).

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "../include/plexus_kernels.h"

namespace plx {

constexpr int SPMM_WARPS = 8;
constexpr int LONG_ROW = 4096;

template <typename T>
struct Vec16;  // 16-byte vector of T
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void fma(float (&acc)[8], const uint4& v, float a) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(p[i]);
      acc[2 * i] = fmaf(a, f.x, acc[2 * i]);
      acc[2 * i + 1] = fmaf(a, f.y, acc[2 * i + 1]);
    }
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
  __device__ static void fma(float (&acc)[4], const uint4& v, float a) {
    const float* p = reinterpret_cast<const float*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = fmaf(a, p[i], acc[i]);
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
template <typename T, int LPR, int VPL>
__device__ __forceinline__ void row_accumulate(const int* __restrict__ col,
                                               const float* __restrict__ val,
                                               const T* __restrict__ H, int64_t ldh, int D,
                                               int64_t beg, int64_t end, int lane,
                                               float (&acc)[VPL][Vec16<T>::N]) {
  constexpr int VN = Vec16<T>::N;
  constexpr int G = 32 / LPR;
  const int g = lane / LPR, li = lane % LPR;
  bool active[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) active[v] = (v * LPR + li) * VN < D;

  for (int64_t base = beg; base < end; base += 32) {
    const int cnt = (end - base) < 32 ? static_cast<int>(end - base) : 32;
    int c = 0;
    float a = 0.f;
    if (lane < cnt) {
      c = __ldg(col + base + lane);
      a = __ldg(val + base + lane);
    }
    // every group walks the 32 staged nonzeros with stride G, two at a time
    for (int jj = 0; jj < cnt; jj += 2 * G) {  // trip count is uniform across the warp
      const int j0 = jj + g, j1 = jj + G + g;
      const int c0 = __shfl_sync(0xffffffffu, c, j0 & 31);
      const float a0 = __shfl_sync(0xffffffffu, a, j0 & 31);
      const int c1 = __shfl_sync(0xffffffffu, c, j1 & 31);
      const float a1 = __shfl_sync(0xffffffffu, a, j1 & 31);
      uint4 v0[VPL], v1[VPL];
      const bool p0 = j0 < cnt, p1 = j1 < cnt;
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        if (p0 && active[v]) v0[v] = ldg16(H + c0 * ldh + (v * LPR + li) * VN);
        if (p1 && active[v]) v1[v] = ldg16(H + c1 * ldh + (v * LPR + li) * VN);
      }
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        if (p0 && active[v]) Vec16<T>::fma(acc[v], v0[v], a0);
        if (p1 && active[v]) Vec16<T>::fma(acc[v], v1[v], a1);
      }
    }
  }
  // combine the G groups
#pragma unroll
  for (int off = LPR; off < 32; off <<= 1) {
#pragma unroll
    for (int v = 0; v < VPL; ++v)
#pragma unroll
      for (int i = 0; i < VN; ++i) acc[v][i] += __shfl_xor_sync(0xffffffffu, acc[v][i], off);
  }
}

template <typename T, int LPR, int VPL>
__device__ __forceinline__ void row_store(T* __restrict__ out_row, const T* __restrict__ mask_row,
                                          int D, int lane, float (&acc)[VPL][Vec16<T>::N]) {
  constexpr int VN = Vec16<T>::N;
  if (lane >= LPR) return;
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    const int c = (v * LPR + lane) * VN;
    if (c < D) {
      if (mask_row != nullptr) Vec16<T>::mask(acc[v], ldg16(mask_row + c));
      *reinterpret_cast<uint4*>(out_row + c) = Vec16<T>::pack(acc[v]);
    }
  }
}

template <typename T, int LPR, int VPL>
__global__ void __launch_bounds__(SPMM_WARPS * 32)
spmm_rows_kernel(const int* __restrict__ rowptr, const int* __restrict__ col,
                 const float* __restrict__ val, const T* __restrict__ H, int64_t ldh,
                 T* __restrict__ out, int64_t ldo, const T* __restrict__ mask, int64_t ldm, int D,
                 int row_begin, int row_end, int skip_long) {
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * SPMM_WARPS + (threadIdx.x >> 5);
  const int warps_total = gridDim.x * SPMM_WARPS;
  for (int row = row_begin + warp_global; row < row_end; row += warps_total) {
    const int64_t beg = __ldg(rowptr + row), end = __ldg(rowptr + row + 1);
    if (skip_long && end - beg > LONG_ROW) continue;
    float acc[VPL][Vec16<T>::N];
#pragma unroll
    for (int v = 0; v < VPL; ++v)
#pragma unroll
      for (int i = 0; i < Vec16<T>::N; ++i) acc[v][i] = 0.f;
    row_accumulate<T, LPR, VPL>(col, val, H, ldh, D, beg, end, lane, acc);
    const int64_t orow = row - row_begin;
    row_store<T, LPR, VPL>(out + orow * ldo, mask ? mask + orow * ldm : nullptr, D, lane, acc);
  }
}

// One CTA per long row: the warps split the nonzeros, partial sums meet in shared memory.
template <typename T, int LPR, int VPL>
__global__ void __launch_bounds__(SPMM_WARPS * 32)
spmm_long_rows_kernel(const int* __restrict__ long_rows, const int* __restrict__ rowptr,
                      const int* __restrict__ col, const float* __restrict__ val,
                      const T* __restrict__ H, int64_t ldh, T* __restrict__ out, int64_t ldo,
                      const T* __restrict__ mask, int64_t ldm, int D, int row_begin, int row_end) {
  constexpr int VN = Vec16<T>::N;
  __shared__ float red[SPMM_WARPS][VPL * LPR * VN];
  const int row = long_rows[blockIdx.x];
  if (row < row_begin || row >= row_end) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t beg = rowptr[row], end = rowptr[row + 1];
  const int64_t n = end - beg;
  const int64_t per = ((n + SPMM_WARPS - 1) / SPMM_WARPS + 31) / 32 * 32;
  int64_t b = beg + warp * per;
  if (b > end) b = end;
  int64_t e = b + per;
  if (e > end) e = end;
  float acc[VPL][VN];
#pragma unroll
  for (int v = 0; v < VPL; ++v)
#pragma unroll
    for (int i = 0; i < VN; ++i) acc[v][i] = 0.f;
  row_accumulate<T, LPR, VPL>(col, val, H, ldh, D, b, e, lane, acc);
  if (lane < LPR) {
#pragma unroll
    for (int v = 0; v < VPL; ++v)
#pragma unroll
      for (int i = 0; i < VN; ++i) red[warp][(v * LPR + lane) * VN + i] = acc[v][i];
  }
  __syncthreads();
  if (warp == 0) {
    if (lane < LPR) {
#pragma unroll
      for (int v = 0; v < VPL; ++v)
#pragma unroll
        for (int i = 0; i < VN; ++i) {
          float s = 0.f;
          for (int w = 0; w < SPMM_WARPS; ++w) s += red[w][(v * LPR + lane) * VN + i];
          acc[v][i] = s;
        }
    }
    const int64_t orow = row - row_begin;
    row_store<T, LPR, VPL>(out + orow * ldo, mask ? mask + orow * ldm : nullptr, D, lane, acc);
  }
}

template <typename T, int LPR, int VPL>
static void launch_spmm(const int* rowptr, const int* col, const float* val, const T* H, int64_t ldh,
                        T* out, int64_t ldo, const T* mask, int64_t ldm, int D, int row_begin,
                        int row_end, const int* long_rows, int n_long, cudaStream_t stream) {
  const int rows = row_end - row_begin;
  if (rows <= 0) return;
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int max_blocks = sms * 8;
  const int blocks = std::max(1, std::min(max_blocks, (rows + SPMM_WARPS - 1) / SPMM_WARPS));
  spmm_rows_kernel<T, LPR, VPL><<<blocks, SPMM_WARPS * 32, 0, stream>>>(
      rowptr, col, val, H, ldh, out, ldo, mask, ldm, D, row_begin, row_end, n_long > 0 ? 1 : 0);
  if (n_long > 0) {
    spmm_long_rows_kernel<T, LPR, VPL><<<n_long, SPMM_WARPS * 32, 0, stream>>>(
        long_rows, rowptr, col, val, H, ldh, out, ldo, mask, ldm, D, row_begin, row_end);
  }
}

template <typename T>
static const char* dispatch_spmm(int D, const int* rowptr, const int* col, const float* val, const T* H,
                                 int64_t ldh, T* out, int64_t ldo, const T* mask, int64_t ldm,
                                 int row_begin, int row_end, const int* long_rows, int n_long,
                                 cudaStream_t stream) {
  constexpr int VN = Vec16<T>::N;
  const int vecs = (D + VN - 1) / VN;  // 16-byte vectors per feature row
#define PLX_SPMM(LPR, VPL)                                                                        \
  launch_spmm<T, LPR, VPL>(rowptr, col, val, H, ldh, out, ldo, mask, ldm, D, row_begin, row_end, \
                           long_rows, n_long, stream)
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

int spmm_long_row_threshold() { return LONG_ROW; }

// out[row_begin:row_end] = A[row_begin:row_end] . H  (optionally masked by mask > 0).
// long_rows: int32 list of rows with more than LONG_ROW nonzeros (may be empty).
const char* launch_spmm_csr(int dtype, const int* rowptr, const int* col, const float* val,
                            const void* H, int64_t ldh, void* out, int64_t ldo, const void* mask,
                            int64_t ldm, int D, int row_begin, int row_end, const int* long_rows,
                            int n_long, cudaStream_t stream) {
  const int esz = dtype == DT_BF16 ? 2 : 4;
  if ((ldh * esz) % 16 || (ldo * esz) % 16 || (D * esz) % 16 || (mask && (ldm * esz) % 16))
    return "spmm: feature rows must be multiples of 16 bytes";
  if (reinterpret_cast<uintptr_t>(H) % 16 || reinterpret_cast<uintptr_t>(out) % 16 ||
      reinterpret_cast<uintptr_t>(mask) % 16)
    return "spmm: feature pointers must be 16-byte aligned";
  if (row_end <= row_begin || D == 0) return nullptr;
  if (dtype == DT_BF16)
    return dispatch_spmm<__nv_bfloat16>(D, rowptr, col, val, reinterpret_cast<const __nv_bfloat16*>(H),
                                        ldh, reinterpret_cast<__nv_bfloat16*>(out), ldo,
                                        reinterpret_cast<const __nv_bfloat16*>(mask), ldm, row_begin,
                                        row_end, long_rows, n_long, stream);
  if (dtype == DT_F32)
    return dispatch_spmm<float>(D, rowptr, col, val, reinterpret_cast<const float*>(H), ldh,
                                reinterpret_cast<float*>(out), ldo, reinterpret_cast<const float*>(mask),
                                ldm, row_begin, row_end, long_rows, n_long, stream);
  return "spmm: features must be bf16 or fp32";
}

}  // namespace plx
