// Plain C++ launch interface of the sm_100a kernels (no torch types): raw device pointers, a
// stream, and a `const char*` result that is nullptr on success or a static error message.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace plx {

enum DType : int { DT_BF16 = 0, DT_F32 = 1 };

// Peer-memory destinations of a fused "compute + push" epilogue (plain stores over NVLink into
// receive buffers that live in other GPUs' memory).  Two modes:
//   seg_rows == 0 (one-shot all-reduce): besides its own output, the kernel stores every result
//     row at the same (row, column) position of every peer's receive slot.
//   seg_rows  > 0 (first half of a two-shot all-reduce, i.e. a reduce-scatter): output row r
//     belongs to group rank r / seg_rows.  Rows of this rank (`me`) go to the local output only;
//     a row of another rank goes ONLY to that rank's receive slot, at row r - owner * seg_rows.
//     base[] lists the peers in group-rank order with `me` left out.
constexpr int MAX_PEERS = 7;
struct PushTargets {
  int n;                  // number of peers (0 = no push)
  void* base[MAX_PEERS];  // receive slot of this rank inside each peer's workspace
  int64_t ld;             // leading dimension of the receive slots (elements)
  int seg_rows;           // rows per owner (0 = broadcast every row)
  int me;                 // this rank's position in the group (seg_rows > 0 only)
  // Debug build of a run (PLEXUS_DEBUG=1): capacity of a receive slot in elements.  A store that
  // would end beyond it is skipped and recorded in the status words (BOUNDS, kernel, row, column);
  // 0 switches the check off.
  int64_t limit_elems;
  int* status;
};

// In-kernel all-reduce of a fused "compute + push" kernel (one-shot form): besides pushing its
// partial result rows into the peers' receive slots (PushTargets), the kernel sums the partials it
// receives itself - no second launch, no flags, no system-scope fences.  The receive slots used for
// this hold a SENTINEL (every byte 0xFF, a bf16 NaN that no conversion from fp32 produces) wherever
// nothing has arrived yet: a warp that has stored rows locally and into the peers' slots later
// re-reads its own rows and the peers' partials of the same rows, treats a 16-byte vector as
// arrived once none of its eight elements is the sentinel, adds the partials in group-rank order,
// applies ReLU / the mask, writes the final rows and puts the sentinel back into the slot for the
// next use of the buffer.  Waiting for a vector is bounded; a timeout is recorded in the status
// words.  n == 0 switches it off.
struct TileReduce {
  int n;                        // peers
  void* slot[MAX_PEERS];        // this rank's sentinel-kept receive slot of every peer (layout of the push)
  int me;                       // position in the group (summation order)
  unsigned long long timeout_ns;
  int* status;
};

// ---- spmm.cu
// CUDA-core SpMM (bf16 or fp32 features), one launch.  Work items, 4 ints each: the pieces of the
// long rows first ({row, -(long id + 1), first nonzero, last nonzero + 1}; a piece's index is also
// the index of its fp32 partial row in `scratch`, spmm_scratch_per_piece() floats each), then
// blocks of whole rows ({first row, last row + 1, 0, 0}).  long_piece_start[num_long + 1] indexes
// the pieces of each long row; long_counter[num_long + 2] (one per long row, then the
// two counters that hand out the items) must be zero and is left zero.  Without the
// in-kernel all-reduce the long rows are summed by a second, small launch; with it the warp that
// delivers the last piece of a row sums them, so that everything happens in one kernel.
int64_t spmm_scratch_per_piece(int dtype, int D);
const char* launch_spmm_csr(int dtype, const int* rowptr, const int* col, const float* val,
                            const void* H, int64_t ldh, void* out, int64_t ldo, const void* mask,
                            int64_t ldm, int D, int row_begin, const int* items, int num_items,
                            int num_pieces, const int* long_piece_start, int num_long, int* long_counter,
                            float* scratch, int64_t scratch_elems, const PushTargets* push,
                            cudaStream_t stream, const TileReduce* reduce = nullptr, int out_rows = 0);

// ---- spmm_mma.cu
// Tensor-core SpMM for bf16 features (any D that is a multiple of 8), one launch for rows of any
// length.  Work items, 4 ints each: the pieces of the long rows first ({row, -(long id + 1), first
// nonzero, last nonzero + 1}; a piece's index is also the index of its fp32 partial row in
// `scratch`), then blocks of whole rows ({first row, last row + 1, 0, 0}).  long_piece_start
// [num_long + 1] indexes the pieces of each long row; long_counter[num_long] must be zero and is
// left zero.  stages: depth of the shared-memory ring of a warp (0 = chosen from the row size).
const char* launch_spmm_mma(const int* rowptr, const int* col, const float* val, const void* H, int64_t ldh,
                            void* out, int64_t ldo, const void* mask, int64_t ldm, int D, int row_begin,
                            const int* items, int num_items, int num_pieces, const int* long_piece_start,
                            int* long_counter, float* scratch, int64_t scratch_elems,
                            const PushTargets* push, int stages, int* status, cudaStream_t stream,
                            const TileReduce* reduce = nullptr, int out_rows = 0);

// ---- gemm_tcgen05.cu
// C[M,N] = A[M,K] . B[N,K]^T ; A, B bf16 row-major (lda/ldb in elements); C bf16 or fp32.
const char* launch_gemm_nt(const void* A, int64_t lda, const void* B, int64_t ldb, void* C,
                           int64_t ldc, int c_dtype, int64_t M, int64_t N, int64_t K, bool relu,
                           int* status, int max_stages, int ctas_limit, int nb_override,
                           const PushTargets* push, const void* mask, int64_t ldm, cudaStream_t stream,
                           const TileReduce* reduce = nullptr);

// mask (same dtype and shape as C, may be null): C = result where mask > 0, else 0.
// out[Mw,Nw] fp32 = A[R,Mw]^T . B[R,Nw]; scratch >= gemm_tn_parts(R)*Mw*Nw floats.
int gemm_tn_parts(int64_t R);
const char* launch_gemm_tn(const void* A, int64_t lda, const void* B, int64_t ldb, float* out,
                           float* scratch, int64_t scratch_elems, int64_t R, int64_t Mw, int64_t Nw,
                           int* status, cudaStream_t stream);

// ---- xent.cu
// stats[2][R]: per-row (max, sum exp) of this class shard; with `loss` (classes not sharded) the
// same launch adds up the loss terms.  xent_combine: statistics of all P class shards
// (pairs[P][2][R]) -> stats[2][R] and the loss terms of the local targets.
struct SlotList;
struct PeerSync;
// push: optional receive slots ([2][R] floats each) of this rank on the peers of the class axis.
const char* launch_xent_stats(int dtype, const void* logits, int64_t ld, int R, int C, int class_offset,
                              int num_classes, float* stats, const int64_t* target, const float* weight,
                              int64_t row_offset, int64_t num_nodes, float* loss, cudaStream_t stream,
                              const SlotList* push = nullptr);
// pairs.ptr[q]: statistics [2][R] of class shard q, rank order.  sync: optional flag barrier first.
const char* launch_xent_combine(int dtype, const void* logits, int64_t ld, const int64_t* target,
                                const SlotList& pairs, const float* weight, int R, int C, int64_t row_offset,
                                int class_offset, int64_t num_nodes, float* stats, float* loss,
                                cudaStream_t stream, const PeerSync* sync = nullptr);
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

// ---- comm_fused.cu
struct SlotList {
  int n;
  void* ptr[MAX_PEERS + 1];
  // For the reducing kernels: ptr[] lists the peers' partials in group-rank order with this rank
  // left out, and `me` is this rank's position in the group.  The local partial is added at that
  // position, so every rank of the group sums in the same order and replicas stay bitwise equal.
  // me < 0: local partial first.
  int me;
};
// Flags of one op: remote_flag[q] is this rank's entry in peer q's flag array (written here),
// local_flag[q] is peer q's entry in this rank's flag array (polled here).
struct PeerSync {
  int n;
  int* remote_flag[MAX_PEERS];
  const int* local_flag[MAX_PEERS];
  int epoch;
  unsigned long long timeout_ns;
  int kernel_id;
  int* status;
};
const char* launch_reduce_slots_bf16(void* out, int64_t ldo, const SlotList& slots, int64_t lds,
                                     int64_t rows, int cols, bool relu, const void* mask, int64_t ldm,
                                     const PeerSync& sync, cudaStream_t stream);
// Flag-free variant: the slots are sentinel-kept (see TileReduce); slots.me = position in the group.
const char* launch_reduce_sentinel_bf16(void* out, int64_t ldo, const SlotList& slots, int64_t lds, int64_t rows,
                                        int cols, bool relu, const void* mask, int64_t ldm, double timeout_ms,
                                        int kernel_id, int* status, int max_blocks, cudaStream_t stream);
const char* launch_reduce_slots_f32(float* out, const SlotList& slots, int64_t n, int op,
                                    const PeerSync& sync, cudaStream_t stream);
const char* launch_push_copy(const void* src, const SlotList& dst, int64_t bytes, cudaStream_t stream);
const char* launch_gather_slots(const SlotList& src, const SlotList& dst, int64_t bytes,
                                const PeerSync& sync, cudaStream_t stream);
// Second half of a two-shot all-reduce.  `out` holds this rank's partial sums of its own row
// segment [row0, row0 + rows); slots hold the peers' partials of the same rows.  The kernel waits
// for the peers (op `sync.epoch`), sums in fp32, applies ReLU / the mask, writes the segment back
// to `out` and stores it into `bcast` (this rank's receive slot of the NEXT op on every peer).
const char* launch_reduce_segment_bf16(void* out, int64_t ldo, int64_t row0, const SlotList& slots,
                                       int64_t lds, int64_t rows, int cols, bool relu, const void* mask,
                                       int64_t ldm, const SlotList& bcast, const PeerSync& sync,
                                       cudaStream_t stream);
// After the wait: copy bytes[q] bytes of slot q to dst.ptr[q] (segments of unequal length).
struct SlotBytes {
  int64_t n[MAX_PEERS + 1];
};
const char* launch_gather_segments(const SlotList& src, const SlotList& dst, const SlotBytes& bytes,
                                   const PeerSync& sync, cudaStream_t stream);
// ---- nvls_reduce.cu
// Middle step of the all-reduce on a symmetric buffer S (same offset on every rank): after the flag
// barrier, reduce `rows` x `cols` bf16 elements that start `elem_off` elements into S and write the
// result (ReLU / mask applied) back to the same place on every rank.  mc != nullptr: multicast
// address of S, the sum is formed inside the switch (multimem.ld_reduce / multimem.st).
// mc == nullptr: `all` lists every rank's S in group-rank order (plain peer loads and stores).
const char* launch_segment_reduce_bf16(void* mc, const SlotList& all, int64_t elem_off, int64_t rows, int cols,
                                       bool relu, const void* mask, int64_t ldm, const PeerSync& sync,
                                       int max_blocks, cudaStream_t stream);
// symmetric workspace over CUDA IPC (one cudaMalloc per rank, handles exchanged by the caller)
const char* symm_alloc(size_t bytes, void** ptr, unsigned char* handle64);
const char* symm_open(const unsigned char* handle64, void** ptr);
const char* symm_close(void* ptr);
const char* symm_free(void* ptr);
const char* symm_fill(void* ptr, int byte, size_t bytes);  // memset on a local workspace

// ---- graph_prep.cu (start-up kernels)
const char* launch_rmat_edges(int64_t num_nodes, int64_t first_edge, int64_t n, uint64_t seed, double a,
                              double b, double c, int64_t* row, int64_t* col, cudaStream_t stream);
const char* launch_gcn_norm(const int64_t* row, const int64_t* col, const float* w, int64_t nnz, float* deg,
                            float* out, cudaStream_t stream);
size_t coo_to_csr_temp_bytes(int64_t nnz, int64_t nrows);
const char* launch_coo_to_csr(const int64_t* row, const int64_t* col, const float* val, int64_t nnz,
                              int64_t nrows, int64_t ncols, int* crow, int* col_out, float* val_out,
                              void* temp, size_t temp_bytes, cudaStream_t stream);
const char* launch_relu_dropout(int dtype, bool backward, const void* x, const void* g, void* out, int64_t n,
                                double p, uint64_t seed, int64_t index_offset, cudaStream_t stream);

// out[i] (fp32, i < n) = entry flat_offset + i of the row-major local block [.., local_cols] at
// (row0, col0) of the zero-padded Kaiming-uniform weight; a pure function of (seed, stream_id, r, c).
const char* launch_weight_init_shard(float* out, int64_t n, int64_t flat_offset, int local_cols, int row0,
                                     int col0, int in_ch, int out_ch, uint64_t seed, uint64_t stream_id,
                                     float bound, cudaStream_t stream);
// Checks rowptr[0..nrows] / col[0..nnz) of an int32 CSR matrix; violations go to the status words.
const char* launch_csr_validate(const int* rowptr, const int* col, int64_t nrows, int64_t ncols, int64_t nnz,
                                int* status, cudaStream_t stream);

inline const char* last_launch_error() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace plx
