// Plain C++ launch interface of the sm_100a kernels (no torch types): raw device pointers, a
// stream, and a `const char*` result that is nullptr on success or a static error message.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace plx {

enum DType : int { DT_BF16 = 0, DT_F32 = 1 };

// ---- spmm.cu
// Per-matrix work schedule (device arrays, built once per shard; see ops/cuda.py):
//   block_start[num_blocks+1] : consecutive-row blocks of about equal cost
//   long rows (more than spmm_piece_size() nonzeros) are cut in pieces [piece_beg, piece_end) of
//   the nonzero range; long_piece_start[num_long+1] indexes the pieces of each long row.
struct SpmmSchedule {
  const int* block_start;
  int num_blocks;
  const int* piece_beg;
  const int* piece_end;
  int num_pieces;
  const int* long_rows;
  const int* long_piece_start;
  int num_long;
};
int spmm_piece_size();
int64_t spmm_scratch_per_piece(int dtype, int D);
// scratch: fp32, num_pieces * spmm_scratch_per_piece(dtype, D) elements (unused without long rows)
const char* launch_spmm_csr(int dtype, const int* rowptr, const int* col, const float* val,
                            const void* H, int64_t ldh, void* out, int64_t ldo, const void* mask,
                            int64_t ldm, int D, int row_begin, const SpmmSchedule& sched,
                            float* scratch, int64_t scratch_elems, cudaStream_t stream);

// ---- gemm_tcgen05.cu
// C[M,N] = A[M,K] . B[N,K]^T ; A, B bf16 row-major (lda/ldb in elements); C bf16 or fp32.
const char* launch_gemm_nt(const void* A, int64_t lda, const void* B, int64_t ldb, void* C,
                           int64_t ldc, int c_dtype, int64_t M, int64_t N, int64_t K, bool relu,
                           int* status, int max_stages, int ctas_limit, cudaStream_t stream);
// out[Mw,Nw] fp32 = A[R,Mw]^T . B[R,Nw]; scratch >= gemm_tn_parts(R)*Mw*Nw floats.
int gemm_tn_parts(int64_t R);
const char* launch_gemm_tn(const void* A, int64_t lda, const void* B, int64_t ldb, float* out,
                           float* scratch, int64_t scratch_elems, int64_t R, int64_t Mw, int64_t Nw,
                           int* status, cudaStream_t stream);

// ---- xent.cu
const char* launch_xent_stats(int dtype, const void* logits, int64_t ld, int R, int C,
                              int class_offset, int num_classes, float* rmax, float* rsum,
                              cudaStream_t stream);
const char* launch_xent_loss(int dtype, const void* logits, int64_t ld, const int64_t* target,
                             const float* gmax, const float* gsum, const float* weight, int R, int C,
                             int64_t row_offset, int class_offset, int64_t num_nodes, float* loss,
                             cudaStream_t stream);
const char* launch_xent_grad(int dtype, const void* logits, int64_t ld, const int64_t* target,
                             const float* gmax, const float* gsum, const float* scale, int R, int C,
                             int64_t row_offset, int class_offset, int64_t num_nodes, int num_classes,
                             void* grad, int64_t ldg, cudaStream_t stream);

// ---- adam.cu
constexpr int ADAM_MAX_TENSORS = 24;
struct AdamTensors {
  void* param[ADAM_MAX_TENSORS];
  const void* grad[ADAM_MAX_TENSORS];
  float* exp_avg[ADAM_MAX_TENSORS];
  float* exp_avg_sq[ADAM_MAX_TENSORS];
  float* master[ADAM_MAX_TENSORS];  // nullptr: the parameter itself is fp32
  int64_t numel[ADAM_MAX_TENSORS];
  int chunk_start[ADAM_MAX_TENSORS + 1];
  int is_bf16[ADAM_MAX_TENSORS];
  int count;
};
struct AdamHyper {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;
  int decoupled;
};
constexpr int ADAM_CHUNK = 4096;  // elements per block iteration
const char* launch_adam_multi(const AdamTensors& t, const AdamHyper& h, cudaStream_t stream);

// ---- elementwise.cu
const char* launch_relu_bwd(int dtype, const void* grad, const void* out, void* res, int64_t n,
                            cudaStream_t stream);
const char* launch_prep_weight(int dtype, const void* W, void* Wb, void* WbT, int K, int N,
                               cudaStream_t stream);
const char* launch_wait_flag(const int* flag, int expected, unsigned max_polls, int* status,
                             cudaStream_t stream);

inline const char* last_launch_error() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace plx
