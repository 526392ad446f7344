// Python bindings of the sm_100a kernels (module plexus_b200._C): tensor checks, then the plain
// launchers declared in include/plexus_kernels.h on the current CUDA stream.

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cmath>

#include "include/plexus_kernels.h"

namespace {

using torch::Tensor;

int dtype_of(const Tensor& t) {
  if (t.scalar_type() == at::kBFloat16) return plx::DT_BF16;
  TORCH_CHECK(t.scalar_type() == at::kFloat, "expected a bf16 or fp32 tensor");
  return plx::DT_F32;
}

void check(const char* err) { TORCH_CHECK(err == nullptr, err ? err : ""); }

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream(); }

int* status_ptr(const Tensor& status) {
  if (!status.defined() || status.numel() == 0) return nullptr;
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 8);
  return status.data_ptr<int>();
}

// seg_rows > 0 selects the reduce-scatter push (row r goes only to group rank r / seg_rows).
plx::PushTargets make_push(const std::vector<int64_t>& ptrs, int64_t ld, int64_t seg_rows = 0,
                           int64_t me = 0, int64_t limit_elems = 0, int* status = nullptr) {
  plx::PushTargets p = {};
  TORCH_CHECK(ptrs.size() <= static_cast<size_t>(plx::MAX_PEERS), "too many push targets");
  TORCH_CHECK(seg_rows >= 0 && seg_rows < (1ll << 31) && me >= 0 && me <= static_cast<int64_t>(ptrs.size()),
              "bad reduce-scatter push description");
  p.n = static_cast<int>(ptrs.size());
  for (int i = 0; i < p.n; ++i) p.base[i] = reinterpret_cast<void*>(ptrs[i]);
  p.ld = ld;
  p.seg_rows = static_cast<int>(seg_rows);
  p.me = static_cast<int>(me);
  p.limit_elems = limit_elems > 0 ? limit_elems : 0;
  p.status = status;
  return p;
}

// In-kernel all-reduce description: this rank's sentinel-kept receive slots (empty list: off).
plx::TileReduce make_tile_reduce(const std::vector<int64_t>& slots, int64_t me, double timeout_ms) {
  plx::TileReduce r = {};
  TORCH_CHECK(slots.size() <= static_cast<size_t>(plx::MAX_PEERS), "bad in-kernel all-reduce description");
  r.n = static_cast<int>(slots.size());
  for (int i = 0; i < r.n; ++i) r.slot[i] = reinterpret_cast<void*>(slots[i]);
  r.me = static_cast<int>(me);
  r.timeout_ns = static_cast<unsigned long long>(timeout_ms * 1e6);
  return r;
}

plx::SlotList make_slots(const std::vector<int64_t>& ptrs, int64_t me = -1) {
  plx::SlotList s;
  s.me = static_cast<int>(me);
  TORCH_CHECK(ptrs.size() <= static_cast<size_t>(plx::MAX_PEERS + 1), "too many slots");
  s.n = static_cast<int>(ptrs.size());
  for (int i = 0; i < s.n; ++i) s.ptr[i] = reinterpret_cast<void*>(ptrs[i]);
  return s;
}

plx::PeerSync make_sync(const std::vector<int64_t>& remote_flags, const std::vector<int64_t>& local_flags,
                        int64_t epoch, double timeout_ms, int64_t kernel_id, const Tensor& status) {
  plx::PeerSync s;
  TORCH_CHECK(remote_flags.size() == local_flags.size() &&
              remote_flags.size() <= static_cast<size_t>(plx::MAX_PEERS));
  s.n = static_cast<int>(remote_flags.size());
  for (int i = 0; i < s.n; ++i) {
    s.remote_flag[i] = reinterpret_cast<int*>(remote_flags[i]);
    s.local_flag[i] = reinterpret_cast<const int*>(local_flags[i]);
  }
  s.epoch = static_cast<int>(epoch);
  s.timeout_ns = static_cast<unsigned long long>(timeout_ms * 1e6);
  s.kernel_id = static_cast<int>(kernel_id);
  s.status = status_ptr(status);
  return s;
}

const int* int_ptr(const Tensor& t) {
  if (!t.defined() || t.numel() == 0) return nullptr;
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous());
  return t.data_ptr<int>();
}

// Both SpMM kernels take the same arguments; `tensor_core` selects spmm_mma.cu (bf16 only).
void spmm_items(bool tensor_core, const Tensor& rowptr, const Tensor& col, const Tensor& val, const Tensor& H,
                Tensor& out, const c10::optional<Tensor>& mask, int64_t row_begin, const Tensor& items,
                int64_t num_pieces, const Tensor& long_piece_start, Tensor& long_counter, const Tensor& scratch,
                const std::vector<int64_t>& push_ptrs, int64_t push_ld, int64_t stages, int64_t push_seg_rows,
                int64_t push_me, const Tensor& status, const std::vector<int64_t>& red_slots, int64_t red_me,
                double red_timeout_ms, int64_t push_limit_elems) {
  TORCH_CHECK(rowptr.is_cuda() && col.is_cuda() && val.is_cuda() && H.is_cuda() && out.is_cuda());
  TORCH_CHECK(rowptr.scalar_type() == at::kInt && col.scalar_type() == at::kInt,
              "spmm: int32 CSR indices required");
  TORCH_CHECK(val.scalar_type() == at::kFloat, "spmm: fp32 CSR values required");
  TORCH_CHECK(rowptr.is_contiguous() && col.is_contiguous() && val.is_contiguous());
  TORCH_CHECK(H.dim() == 2 && out.dim() == 2 && H.stride(1) == 1 && out.stride(1) == 1);
  TORCH_CHECK(out.scalar_type() == H.scalar_type(), "spmm: out dtype must match H");
  TORCH_CHECK(!tensor_core || H.scalar_type() == at::kBFloat16, "spmm: the tensor-core kernel takes bf16 features");
  const int64_t D = H.size(1);
  TORCH_CHECK(out.size(1) == D, "spmm: bad output shape");
  const void* mptr = nullptr;
  int64_t ldm = 0;
  if (mask.has_value() && mask->defined()) {
    TORCH_CHECK(mask->is_cuda() && mask->scalar_type() == H.scalar_type() && mask->size(1) == D &&
                mask->size(0) == out.size(0) && mask->stride(1) == 1, "spmm: bad mask");
    mptr = mask->data_ptr();
    ldm = mask->stride(0);
  }
  TORCH_CHECK(items.numel() % 4 == 0, "spmm: work items are 4 ints each");
  const int num_items = static_cast<int>(items.numel() / 4);
  float* scr = nullptr;
  int64_t scr_n = 0;
  if (scratch.defined() && scratch.numel() > 0) {
    TORCH_CHECK(scratch.is_cuda() && scratch.scalar_type() == at::kFloat && scratch.is_contiguous());
    scr = scratch.data_ptr<float>();
    scr_n = scratch.numel();
  }
  // one counter per long row, then the two work hand-out counters of the CUDA-core kernel
  TORCH_CHECK(long_counter.defined() && long_counter.numel() >= 2 && long_counter.is_cuda() &&
                  long_counter.scalar_type() == at::kInt && long_counter.is_contiguous(),
              "spmm: counters must be an int32 CUDA tensor of (long rows + 2) zeros");
  int* counters = long_counter.data_ptr<int>();
  const int num_long = static_cast<int>(long_counter.numel() - 2);
  plx::PushTargets push = make_push(push_ptrs, push_ld, push_seg_rows, push_me, push_limit_elems, status_ptr(status));
  TORCH_CHECK(push_seg_rows == 0 || push_seg_rows * (push.n + 1) >= out.size(0),
              "spmm: row segments do not cover the output");
  plx::TileReduce red = make_tile_reduce(red_slots, red_me, red_timeout_ms);
  red.status = status_ptr(status);
  c10::cuda::CUDAGuard guard(H.device());
  if (tensor_core) {
    check(plx::launch_spmm_mma(rowptr.data_ptr<int>(), col.data_ptr<int>(), val.data_ptr<float>(), H.data_ptr(),
                               H.stride(0), out.data_ptr(), out.stride(0), mptr, ldm, static_cast<int>(D),
                               static_cast<int>(row_begin), int_ptr(items), num_items,
                               static_cast<int>(num_pieces), int_ptr(long_piece_start), counters, scr, scr_n,
                               push.n ? &push : nullptr, static_cast<int>(stages), status_ptr(status), stream(),
                               red.n ? &red : nullptr, static_cast<int>(out.size(0))));
  } else {
    check(plx::launch_spmm_csr(dtype_of(H), rowptr.data_ptr<int>(), col.data_ptr<int>(), val.data_ptr<float>(),
                               H.data_ptr(), H.stride(0), out.data_ptr(), out.stride(0), mptr, ldm,
                               static_cast<int>(D), static_cast<int>(row_begin), int_ptr(items), num_items,
                               static_cast<int>(num_pieces), int_ptr(long_piece_start),
                               num_long, counters, scr, scr_n, push.n ? &push : nullptr, stream(), red.n ? &red : nullptr,
                               static_cast<int>(out.size(0))));
  }
}

int64_t spmm_scratch_per_piece(const Tensor& H) {
  return plx::spmm_scratch_per_piece(dtype_of(H), static_cast<int>(H.size(1)));
}

void gemm_nt(const Tensor& A, const Tensor& B, Tensor& C, bool relu, const Tensor& status,
             int64_t max_stages, int64_t ctas_limit, int64_t nb_override,
             const std::vector<int64_t>& push_ptrs, int64_t push_ld, const c10::optional<Tensor>& mask,
             int64_t push_seg_rows, int64_t push_me, const std::vector<int64_t>& red_slots, int64_t red_me,
             double red_timeout_ms, int64_t push_limit_elems) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && C.is_cuda());
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16,
              "gemm_nt: bf16 operands required");
  plx::TileReduce red = make_tile_reduce(red_slots, red_me, red_timeout_ms);
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && C.dim() == 2 && A.size(1) == B.size(1));
  TORCH_CHECK(A.stride(1) == 1 && B.stride(1) == 1 && C.stride(1) == 1);
  TORCH_CHECK(C.size(0) == A.size(0) && C.size(1) == B.size(0), "gemm_nt: bad output shape");
  plx::PushTargets push = make_push(push_ptrs, push_ld, push_seg_rows, push_me, push_limit_elems, status_ptr(status));
  const void* mptr = nullptr;
  int64_t ldm = 0;
  if (mask.has_value() && mask->defined()) {
    TORCH_CHECK(mask->is_cuda() && mask->scalar_type() == C.scalar_type() && mask->sizes() == C.sizes() &&
                mask->stride(1) == 1, "gemm_nt: bad mask");
    mptr = mask->data_ptr();
    ldm = mask->stride(0);
  }
  c10::cuda::CUDAGuard guard(A.device());
  check(plx::launch_gemm_nt(A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), C.data_ptr(),
                            C.stride(0), dtype_of(C), A.size(0), B.size(0), A.size(1), relu,
                            status_ptr(status), static_cast<int>(max_stages),
                            static_cast<int>(ctas_limit), static_cast<int>(nb_override),
                            push.n ? &push : nullptr, mptr, ldm, stream(), red.n ? &red : nullptr));
}

int64_t gemm_tn_parts(int64_t R) { return plx::gemm_tn_parts(R); }

void gemm_tn(const Tensor& A, const Tensor& B, Tensor& out, Tensor& scratch, const Tensor& status) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && out.is_cuda() && scratch.is_cuda());
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16,
              "gemm_tn: bf16 operands required");
  TORCH_CHECK(out.scalar_type() == at::kFloat && scratch.scalar_type() == at::kFloat);
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && A.size(0) == B.size(0) && A.stride(1) == 1 &&
              B.stride(1) == 1 && out.is_contiguous() && scratch.is_contiguous());
  TORCH_CHECK(out.size(0) == A.size(1) && out.size(1) == B.size(1), "gemm_tn: bad output shape");
  c10::cuda::CUDAGuard guard(A.device());
  check(plx::launch_gemm_tn(A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), out.data_ptr<float>(),
                            scratch.data_ptr<float>(), scratch.numel(), A.size(0), A.size(1), B.size(1),
                            status_ptr(status), stream()));
}

static const float* opt_f32(const c10::optional<Tensor>& t, int64_t numel, const char* what) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == numel, what);
  return t->data_ptr<float>();
}

// stats: fp32 [2, R].  With `target` and `loss` (classes not sharded) the loss is added up as well.
void xent_stats(const Tensor& logits, int64_t class_offset, int64_t num_classes, Tensor& stats,
                const c10::optional<Tensor>& target, const c10::optional<Tensor>& weight, int64_t row_offset,
                int64_t num_nodes, const c10::optional<Tensor>& loss, const std::vector<int64_t>& push_ptrs) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1);
  const int64_t R = logits.size(0);
  TORCH_CHECK(stats.is_cuda() && stats.scalar_type() == at::kFloat && stats.is_contiguous() && stats.numel() == 2 * R);
  const int64_t* tptr = nullptr;
  float* lptr = nullptr;
  if (loss.has_value() && loss->defined()) {
    TORCH_CHECK(target.has_value() && target->defined() && target->is_cuda() && target->scalar_type() == at::kLong &&
                target->is_contiguous() && target->numel() == R, "xent_stats: int64 targets, one per row");
    TORCH_CHECK(loss->is_cuda() && loss->scalar_type() == at::kFloat && loss->numel() == 1);
    tptr = target->data_ptr<int64_t>();
    lptr = loss->data_ptr<float>();
  }
  TORCH_CHECK(push_ptrs.size() <= static_cast<size_t>(plx::MAX_PEERS), "xent_stats: too many push targets");
  plx::SlotList push = make_slots(push_ptrs);
  c10::cuda::CUDAGuard guard(logits.device());
  check(plx::launch_xent_stats(dtype_of(logits), logits.data_ptr(), logits.stride(0), static_cast<int>(R),
                               static_cast<int>(logits.size(1)), static_cast<int>(class_offset),
                               static_cast<int>(num_classes), stats.data_ptr<float>(), tptr,
                               opt_f32(weight, R, "xent_stats: fp32 row weights, one per row"), row_offset,
                               num_nodes, lptr, stream(), &push));
}

// pair_ptrs[q]: device address of class shard q's statistics (fp32 [2, R]), rank order -> stats [2, R]
// and the loss.  With flag lists the kernel first runs the flag barrier of op `epoch` (the pairs were
// pushed into this rank's receive slots by the peers' xent_stats launches).
void xent_combine(const Tensor& logits, const Tensor& target, const std::vector<int64_t>& pair_ptrs,
                  const c10::optional<Tensor>& weight, int64_t row_offset, int64_t class_offset, int64_t num_nodes,
                  Tensor& stats, Tensor& loss, const std::vector<int64_t>& remote_flags,
                  const std::vector<int64_t>& local_flags, int64_t epoch, double timeout_ms, const Tensor& status) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1);
  const int64_t R = logits.size(0);
  TORCH_CHECK(target.is_cuda() && target.scalar_type() == at::kLong && target.numel() == R && target.is_contiguous());
  TORCH_CHECK(pair_ptrs.size() >= 1 && pair_ptrs.size() <= static_cast<size_t>(plx::MAX_PEERS + 1),
              "xent_combine: statistics of 1 to 8 class shards");
  for (int64_t p : pair_ptrs) TORCH_CHECK(p != 0 && p % 4 == 0, "xent_combine: bad statistics address");
  TORCH_CHECK(stats.is_cuda() && stats.scalar_type() == at::kFloat && stats.is_contiguous() && stats.numel() == 2 * R);
  TORCH_CHECK(loss.is_cuda() && loss.scalar_type() == at::kFloat && loss.numel() == 1);
  c10::cuda::CUDAGuard guard(logits.device());
  plx::PeerSync sync = {};
  const bool flagged = !remote_flags.empty();
  if (flagged) sync = make_sync(remote_flags, local_flags, epoch, timeout_ms, /*kernel_id=*/5, status);
  check(plx::launch_xent_combine(dtype_of(logits), logits.data_ptr(), logits.stride(0), target.data_ptr<int64_t>(),
                                 make_slots(pair_ptrs), opt_f32(weight, R, "xent_combine: fp32 row weights, one per row"),
                                 static_cast<int>(R), static_cast<int>(logits.size(1)), row_offset,
                                 static_cast<int>(class_offset), num_nodes, stats.data_ptr<float>(),
                                 loss.data_ptr<float>(), stream(), flagged ? &sync : nullptr));
}

void xent_grad(const Tensor& logits, const Tensor& target, const Tensor& gmax, const Tensor& gsum,
               const Tensor& scale, int64_t row_offset, int64_t class_offset, int64_t num_nodes,
               int64_t num_classes, Tensor& grad) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1);
  TORCH_CHECK(scale.is_cuda() && scale.scalar_type() == at::kFloat && scale.numel() == 1);
  TORCH_CHECK(grad.scalar_type() == logits.scalar_type() && grad.stride(1) == 1 &&
              grad.sizes() == logits.sizes());
  TORCH_CHECK(target.scalar_type() == at::kLong && target.is_contiguous());
  c10::cuda::CUDAGuard guard(logits.device());
  check(plx::launch_xent_grad(dtype_of(logits), logits.data_ptr(), logits.stride(0),
                              target.data_ptr<int64_t>(), gmax.data_ptr<float>(), gsum.data_ptr<float>(),
                              scale.data_ptr<float>(), static_cast<int>(logits.size(0)),
                              static_cast<int>(logits.size(1)), row_offset,
                              static_cast<int>(class_offset), num_nodes, static_cast<int>(num_classes),
                              grad.data_ptr(), grad.stride(0), stream()));
}

void adam_multi(std::vector<Tensor> params, std::vector<Tensor> grads, std::vector<Tensor> exp_avgs,
                std::vector<Tensor> exp_avg_sqs, std::vector<c10::optional<Tensor>> masters,
                int64_t step, double lr, double beta1, double beta2, double eps, double weight_decay,
                bool decoupled) {
  const size_t n = params.size();
  TORCH_CHECK(grads.size() == n && exp_avgs.size() == n && exp_avg_sqs.size() == n && masters.size() == n);
  if (n == 0) return;
  plx::AdamHyper h;
  h.lr = static_cast<float>(lr);
  h.beta1 = static_cast<float>(beta1);
  h.beta2 = static_cast<float>(beta2);
  h.eps = static_cast<float>(eps);
  h.weight_decay = static_cast<float>(weight_decay);
  h.bc1 = static_cast<float>(1.0 - std::pow(beta1, static_cast<double>(step)));
  h.bc2 = static_cast<float>(1.0 - std::pow(beta2, static_cast<double>(step)));
  h.decoupled = decoupled ? 1 : 0;
  c10::cuda::CUDAGuard guard(params[0].device());
  for (size_t first = 0; first < n; first += plx::ADAM_MAX_TENSORS) {
    plx::AdamTensors t;
    t.count = static_cast<int>(std::min<size_t>(plx::ADAM_MAX_TENSORS, n - first));
    t.chunk_start[0] = 0;
    for (int i = 0; i < t.count; ++i) {
      const Tensor& p = params[first + i];
      const Tensor& g = grads[first + i];
      const Tensor& m = exp_avgs[first + i];
      const Tensor& v = exp_avg_sqs[first + i];
      TORCH_CHECK(p.is_cuda() && p.is_contiguous() && g.is_contiguous() && g.numel() == p.numel());
      TORCH_CHECK(p.scalar_type() == g.scalar_type(), "adam: grad dtype must match param dtype");
      TORCH_CHECK(p.scalar_type() == at::kFloat || p.scalar_type() == at::kBFloat16);
      TORCH_CHECK(m.scalar_type() == at::kFloat && m.is_contiguous() && m.numel() == p.numel());
      TORCH_CHECK(v.scalar_type() == at::kFloat && v.is_contiguous() && v.numel() == p.numel());
      t.param[i] = p.data_ptr();
      t.grad[i] = g.data_ptr();
      t.exp_avg[i] = m.data_ptr<float>();
      t.exp_avg_sq[i] = v.data_ptr<float>();
      const auto& ms = masters[first + i];
      t.master[i] = nullptr;
      if (ms.has_value() && ms->defined()) {
        TORCH_CHECK(ms->scalar_type() == at::kFloat && ms->is_contiguous() && ms->numel() == p.numel());
        t.master[i] = ms->data_ptr<float>();
      }
      t.numel[i] = p.numel();
      t.is_bf16[i] = p.scalar_type() == at::kBFloat16 ? 1 : 0;
      t.chunk_start[i + 1] =
          t.chunk_start[i] + static_cast<int>((p.numel() + plx::ADAM_CHUNK - 1) / plx::ADAM_CHUNK);
    }
    check(plx::launch_adam_multi(t, h, stream()));
  }
}

void relu_bwd(const Tensor& grad, const Tensor& out, Tensor& res) {
  TORCH_CHECK(grad.is_cuda() && grad.is_contiguous() && out.is_contiguous() && res.is_contiguous());
  TORCH_CHECK(grad.scalar_type() == out.scalar_type() && res.scalar_type() == grad.scalar_type() &&
              grad.numel() == out.numel() && res.numel() == grad.numel());
  c10::cuda::CUDAGuard guard(grad.device());
  check(plx::launch_relu_bwd(dtype_of(grad), grad.data_ptr(), out.data_ptr(), res.data_ptr(),
                             grad.numel(), stream()));
}

void prep_weight(const Tensor& W, const c10::optional<Tensor>& Wb, Tensor& WbT) {
  TORCH_CHECK(W.is_cuda() && W.dim() == 2 && W.is_contiguous() && WbT.is_contiguous());
  const int64_t K = W.size(0), N = W.size(1);
  TORCH_CHECK(WbT.numel() == K * N && WbT.scalar_type() == at::kBFloat16);
  void* wb = nullptr;
  if (Wb.has_value() && Wb->defined()) {
    TORCH_CHECK(Wb->is_contiguous() && Wb->scalar_type() == at::kBFloat16 && Wb->numel() == W.numel());
    wb = Wb->data_ptr();
  }
  c10::cuda::CUDAGuard guard(W.device());
  check(plx::launch_prep_weight(dtype_of(W), W.data_ptr(), wb, WbT.data_ptr(), static_cast<int>(K),
                                static_cast<int>(N), stream()));
}

void wait_flag(const Tensor& flag, int64_t expected, int64_t max_polls, Tensor& status) {
  TORCH_CHECK(flag.is_cuda() && flag.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard guard(flag.device());
  check(plx::launch_wait_flag(flag.data_ptr<int>(), static_cast<int>(expected),
                              static_cast<unsigned>(max_polls), status_ptr(status), stream()));
}

// ---- peer-memory collectives -------------------------------------------------------------
void reduce_slots(Tensor& out, const std::vector<int64_t>& slot_ptrs, int64_t slot_ld, bool relu,
                  const c10::optional<Tensor>& mask, const std::vector<int64_t>& remote_flags,
                  const std::vector<int64_t>& local_flags, int64_t epoch, double timeout_ms,
                  int64_t kernel_id, const Tensor& status, int64_t me) {
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.stride(1) == 1 && out.scalar_type() == at::kBFloat16);
  const void* mptr = nullptr;
  int64_t ldm = 0;
  if (mask.has_value() && mask->defined()) {
    TORCH_CHECK(mask->scalar_type() == at::kBFloat16 && mask->sizes() == out.sizes() && mask->stride(1) == 1);
    mptr = mask->data_ptr();
    ldm = mask->stride(0);
  }
  c10::cuda::CUDAGuard guard(out.device());
  check(plx::launch_reduce_slots_bf16(out.data_ptr(), out.stride(0), make_slots(slot_ptrs, me), slot_ld,
                                      out.size(0), static_cast<int>(out.size(1)), relu, mptr, ldm,
                                      make_sync(remote_flags, local_flags, epoch, timeout_ms, kernel_id, status),
                                      stream()));
}

// Middle step of the two-shot all-reduce: reduce rows [row0, row0 + rows) of `out` with the
// peers' partials and store the result into `bcast_ptrs` (receive slots of the next op).
void reduce_segment(Tensor& out, int64_t row0, int64_t rows, const std::vector<int64_t>& slot_ptrs,
                    int64_t slot_ld, bool relu, const c10::optional<Tensor>& mask,
                    const std::vector<int64_t>& bcast_ptrs, const std::vector<int64_t>& remote_flags,
                    const std::vector<int64_t>& local_flags, int64_t epoch, double timeout_ms,
                    int64_t kernel_id, const Tensor& status, int64_t me) {
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.stride(1) == 1 && out.scalar_type() == at::kBFloat16);
  TORCH_CHECK(row0 >= 0 && rows >= 0 && row0 + rows <= out.size(0), "reduce_segment: bad row range");
  const void* mptr = nullptr;
  int64_t ldm = 0;
  if (mask.has_value() && mask->defined()) {
    TORCH_CHECK(mask->scalar_type() == at::kBFloat16 && mask->sizes() == out.sizes() && mask->stride(1) == 1);
    mptr = mask->data_ptr();
    ldm = mask->stride(0);
  }
  c10::cuda::CUDAGuard guard(out.device());
  check(plx::launch_reduce_segment_bf16(out.data_ptr(), out.stride(0), row0, make_slots(slot_ptrs, me), slot_ld,
                                        rows, static_cast<int>(out.size(1)), relu, mptr, ldm,
                                        make_slots(bcast_ptrs),
                                        make_sync(remote_flags, local_flags, epoch, timeout_ms, kernel_id, status),
                                        stream()));
}

void gather_segments(const std::vector<int64_t>& src_ptrs, const std::vector<int64_t>& dst_ptrs,
                     const std::vector<int64_t>& bytes, const std::vector<int64_t>& remote_flags,
                     const std::vector<int64_t>& local_flags, int64_t epoch, double timeout_ms,
                     int64_t kernel_id, const Tensor& status) {
  TORCH_CHECK(bytes.size() == src_ptrs.size() && bytes.size() <= static_cast<size_t>(plx::MAX_PEERS));
  plx::SlotBytes b = {};
  for (size_t q = 0; q < bytes.size(); ++q) b.n[q] = bytes[q];
  c10::cuda::CUDAGuard guard(status.device());
  check(plx::launch_gather_segments(make_slots(src_ptrs), make_slots(dst_ptrs), b,
                                    make_sync(remote_flags, local_flags, epoch, timeout_ms, kernel_id, status),
                                    stream()));
}

// Reduce this rank's row segment of a symmetric buffer in place on every rank (multimem when
// `mc_ptr` is non-zero, plain peer loads / stores over `all_ptrs` otherwise).  `seg` is the local
// view of the segment (inside buffer all_ptrs[me]); `mask`: the rows of the segment.
void segment_reduce(int64_t mc_ptr, const std::vector<int64_t>& all_ptrs, int64_t me, const Tensor& seg, bool relu,
                    const c10::optional<Tensor>& mask, const std::vector<int64_t>& remote_flags,
                    const std::vector<int64_t>& local_flags, int64_t epoch, double timeout_ms, int64_t kernel_id,
                    const Tensor& status, int64_t max_blocks) {
  TORCH_CHECK(seg.is_cuda() && seg.dim() == 2 && seg.is_contiguous() && seg.scalar_type() == at::kBFloat16,
              "segment_reduce: the segment must be a contiguous bf16 CUDA matrix");
  TORCH_CHECK(all_ptrs.size() >= 1 && all_ptrs.size() <= static_cast<size_t>(plx::MAX_PEERS + 1) && me >= 0 &&
              me < static_cast<int64_t>(all_ptrs.size()));
  const int64_t byte_off = reinterpret_cast<int64_t>(seg.data_ptr()) - all_ptrs[me];
  TORCH_CHECK(byte_off >= 0 && byte_off % 16 == 0, "segment_reduce: the segment does not lie in the local buffer");
  const void* mptr = nullptr;
  int64_t ldm = 0;
  if (mask.has_value() && mask->defined()) {
    TORCH_CHECK(mask->is_cuda() && mask->scalar_type() == at::kBFloat16 && mask->sizes() == seg.sizes() &&
                mask->stride(1) == 1);
    mptr = mask->data_ptr();
    ldm = mask->stride(0);
  }
  c10::cuda::CUDAGuard guard(seg.device());
  check(plx::launch_segment_reduce_bf16(reinterpret_cast<void*>(mc_ptr), make_slots(all_ptrs), byte_off / 2,
                                        seg.size(0), static_cast<int>(seg.size(1)), relu, mptr, ldm,
                                        make_sync(remote_flags, local_flags, epoch, timeout_ms, kernel_id, status),
                                        static_cast<int>(max_blocks), stream()));
}

// Tensor over `numel` elements at a device address of the current device (a workspace of symm_alloc).
Tensor symm_view(int64_t ptr, int64_t numel, at::ScalarType dtype) {
  int dev = 0;
  cudaGetDevice(&dev);
  return at::from_blob(reinterpret_cast<void*>(ptr), {numel},
                       at::TensorOptions().dtype(dtype).device(at::kCUDA, dev));
}

void reduce_sentinel(Tensor& out, const std::vector<int64_t>& slot_ptrs, int64_t slot_ld, bool relu,
                     const c10::optional<Tensor>& mask, double timeout_ms, int64_t kernel_id, const Tensor& status,
                     int64_t me, int64_t max_blocks) {
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.stride(1) == 1 && out.scalar_type() == at::kBFloat16);
  const void* mptr = nullptr;
  int64_t ldm = 0;
  if (mask.has_value() && mask->defined()) {
    TORCH_CHECK(mask->scalar_type() == at::kBFloat16 && mask->sizes() == out.sizes() && mask->stride(1) == 1);
    mptr = mask->data_ptr();
    ldm = mask->stride(0);
  }
  c10::cuda::CUDAGuard guard(out.device());
  check(plx::launch_reduce_sentinel_bf16(out.data_ptr(), out.stride(0), make_slots(slot_ptrs, me), slot_ld,
                                         out.size(0), static_cast<int>(out.size(1)), relu, mptr, ldm, timeout_ms,
                                         static_cast<int>(kernel_id), status_ptr(status),
                                         static_cast<int>(max_blocks), stream()));
}

void reduce_slots_f32(Tensor& out, const std::vector<int64_t>& slot_ptrs, int64_t op,
                      const std::vector<int64_t>& remote_flags, const std::vector<int64_t>& local_flags,
                      int64_t epoch, double timeout_ms, int64_t kernel_id, const Tensor& status, int64_t me) {
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(out.device());
  check(plx::launch_reduce_slots_f32(out.data_ptr<float>(), make_slots(slot_ptrs, me), out.numel(),
                                     static_cast<int>(op),
                                     make_sync(remote_flags, local_flags, epoch, timeout_ms, kernel_id, status),
                                     stream()));
}

void push_copy(const Tensor& src, const std::vector<int64_t>& dst_ptrs) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous());
  c10::cuda::CUDAGuard guard(src.device());
  check(plx::launch_push_copy(src.data_ptr(), make_slots(dst_ptrs), src.numel() * src.element_size(),
                              stream()));
}

void gather_slots(const std::vector<int64_t>& src_ptrs, const std::vector<int64_t>& dst_ptrs, int64_t bytes,
                  const std::vector<int64_t>& remote_flags, const std::vector<int64_t>& local_flags,
                  int64_t epoch, double timeout_ms, int64_t kernel_id, const Tensor& status) {
  c10::cuda::CUDAGuard guard(status.device());
  check(plx::launch_gather_slots(make_slots(src_ptrs), make_slots(dst_ptrs), bytes,
                                 make_sync(remote_flags, local_flags, epoch, timeout_ms, kernel_id, status),
                                 stream()));
}

std::tuple<int64_t, py::bytes> symm_alloc(int64_t bytes) {
  void* p = nullptr;
  unsigned char h[64];
  check(plx::symm_alloc(static_cast<size_t>(bytes), &p, h));
  return {reinterpret_cast<int64_t>(p), py::bytes(reinterpret_cast<const char*>(h), 64)};
}

int64_t symm_open(const std::string& handle) {
  TORCH_CHECK(handle.size() == 64, "IPC handle must be 64 bytes");
  void* p = nullptr;
  check(plx::symm_open(reinterpret_cast<const unsigned char*>(handle.data()), &p));
  return reinterpret_cast<int64_t>(p);
}

void symm_close(int64_t ptr) { check(plx::symm_close(reinterpret_cast<void*>(ptr))); }
void symm_free(int64_t ptr) { check(plx::symm_free(reinterpret_cast<void*>(ptr))); }
void symm_fill(int64_t ptr, int64_t byte, int64_t bytes) {
  check(plx::symm_fill(reinterpret_cast<void*>(ptr), static_cast<int>(byte), static_cast<size_t>(bytes)));
}

// ---- start-up kernels ---------------------------------------------------------------------
std::tuple<Tensor, Tensor> rmat_edges(int64_t num_nodes, int64_t first_edge, int64_t n, int64_t seed,
                                      double a, double b, double c, const Tensor& like) {
  TORCH_CHECK(like.is_cuda());
  c10::cuda::CUDAGuard guard(like.device());
  auto opts = torch::TensorOptions().dtype(at::kLong).device(like.device());
  Tensor row = torch::empty({n}, opts), col = torch::empty({n}, opts);
  check(plx::launch_rmat_edges(num_nodes, first_edge, n, static_cast<uint64_t>(seed), a, b, c,
                               row.data_ptr<int64_t>(), col.data_ptr<int64_t>(), stream()));
  return {row, col};
}

Tensor gcn_norm(const Tensor& edge_index, const c10::optional<Tensor>& weight, int64_t num_nodes) {
  TORCH_CHECK(edge_index.is_cuda() && edge_index.scalar_type() == at::kLong && edge_index.dim() == 2 &&
              edge_index.size(0) == 2 && edge_index.is_contiguous());
  const int64_t nnz = edge_index.size(1);
  const float* w = nullptr;
  if (weight.has_value() && weight->defined()) {
    TORCH_CHECK(weight->scalar_type() == at::kFloat && weight->is_contiguous() && weight->numel() == nnz);
    w = weight->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(edge_index.device());
  auto opts = torch::TensorOptions().dtype(at::kFloat).device(edge_index.device());
  Tensor deg = torch::zeros({num_nodes}, opts), out = torch::empty({nnz}, opts);
  check(plx::launch_gcn_norm(edge_index.data_ptr<int64_t>(), edge_index.data_ptr<int64_t>() + nnz, w, nnz,
                             deg.data_ptr<float>(), out.data_ptr<float>(), stream()));
  return out;
}

std::tuple<Tensor, Tensor, Tensor> coo_to_csr(const Tensor& row, const Tensor& col, const Tensor& val,
                                              int64_t nrows, int64_t ncols) {
  TORCH_CHECK(row.is_cuda() && row.scalar_type() == at::kLong && col.scalar_type() == at::kLong &&
              val.scalar_type() == at::kFloat && row.is_contiguous() && col.is_contiguous() &&
              val.is_contiguous() && row.numel() == col.numel() && row.numel() == val.numel());
  const int64_t nnz = row.numel();
  c10::cuda::CUDAGuard guard(row.device());
  auto iopts = torch::TensorOptions().dtype(at::kInt).device(row.device());
  Tensor crow = torch::zeros({nrows + 1}, iopts), col_out = torch::empty({nnz}, iopts);
  Tensor val_out = torch::empty({nnz}, val.options());
  const size_t tb = plx::coo_to_csr_temp_bytes(nnz, nrows);
  Tensor temp = torch::empty({static_cast<int64_t>(tb)}, torch::TensorOptions().dtype(at::kByte).device(row.device()));
  check(plx::launch_coo_to_csr(row.data_ptr<int64_t>(), col.data_ptr<int64_t>(), val.data_ptr<float>(), nnz,
                               nrows, ncols, crow.data_ptr<int>(), col_out.data_ptr<int>(),
                               val_out.data_ptr<float>(), temp.data_ptr(), tb, stream()));
  return {crow, col_out, val_out};
}

Tensor relu_dropout(const Tensor& x, const c10::optional<Tensor>& grad, double p, int64_t seed,
                    int64_t index_offset) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous());
  const bool bwd = grad.has_value() && grad->defined();
  if (bwd) TORCH_CHECK(grad->is_contiguous() && grad->scalar_type() == x.scalar_type() && grad->numel() == x.numel());
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty_like(x);
  check(plx::launch_relu_dropout(dtype_of(x), bwd, x.data_ptr(), bwd ? grad->data_ptr() : nullptr,
                                 out.data_ptr(), x.numel(), p, static_cast<uint64_t>(seed), index_offset,
                                 stream()));
  return out;
}

void weight_init_shard(Tensor& out, int64_t flat_offset, int64_t local_cols, int64_t row0, int64_t col0,
                       int64_t in_ch, int64_t out_ch, int64_t seed, int64_t stream_id, double bound) {
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(out.device());
  check(plx::launch_weight_init_shard(out.data_ptr<float>(), out.numel(), flat_offset,
                                      static_cast<int>(local_cols), static_cast<int>(row0),
                                      static_cast<int>(col0), static_cast<int>(in_ch), static_cast<int>(out_ch),
                                      static_cast<uint64_t>(seed), static_cast<uint64_t>(stream_id),
                                      static_cast<float>(bound), stream()));
}

void csr_validate(const Tensor& rowptr, const Tensor& col, int64_t nrows, int64_t ncols, const Tensor& status) {
  TORCH_CHECK(rowptr.is_cuda() && col.is_cuda() && rowptr.is_contiguous() && col.is_contiguous());
  TORCH_CHECK(rowptr.scalar_type() == at::kInt && col.scalar_type() == at::kInt, "csr_validate: int32 indices");
  TORCH_CHECK(rowptr.numel() == nrows + 1, "csr_validate: rowptr must have nrows + 1 entries");
  c10::cuda::CUDAGuard guard(col.device());
  check(plx::launch_csr_validate(rowptr.data_ptr<int>(), col.data_ptr<int>(), nrows, ncols, col.numel(),
                                 status_ptr(status), stream()));
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("spmm_items", &spmm_items, "CSR SpMM (CUDA-core or tensor-core kernel), fp32 accumulate");
  m.def("spmm_scratch_per_piece", &spmm_scratch_per_piece);
  m.def("gemm_nt", &gemm_nt, "C = A . B^T on tcgen05 (bf16 in, fp32 accumulate)");
  m.def("gemm_tn_parts", &gemm_tn_parts, "number of row splits gemm_tn uses");
  m.def("gemm_tn", &gemm_tn, "C = A^T . B on tcgen05 with split reduction");
  m.def("xent_stats", &xent_stats);
  m.def("xent_combine", &xent_combine);
  m.def("xent_grad", &xent_grad);
  m.def("adam_multi", &adam_multi);
  m.def("relu_bwd", &relu_bwd);
  m.def("prep_weight", &prep_weight);
  m.def("wait_flag", &wait_flag);
  m.def("rmat_edges", &rmat_edges);
  m.def("gcn_norm", &gcn_norm);
  m.def("coo_to_csr", &coo_to_csr);
  m.def("relu_dropout", &relu_dropout);
  m.def("weight_init_shard", &weight_init_shard);
  m.def("csr_validate", &csr_validate);
  m.def("reduce_slots", &reduce_slots);
  m.def("reduce_slots_f32", &reduce_slots_f32);
  m.def("reduce_sentinel", &reduce_sentinel);
  m.def("reduce_segment", &reduce_segment);
  m.def("segment_reduce", &segment_reduce);
  m.def("gather_segments", &gather_segments);
  m.def("push_copy", &push_copy);
  m.def("gather_slots", &gather_slots);
  m.def("symm_alloc", &symm_alloc);
  m.def("symm_open", &symm_open);
  m.def("symm_close", &symm_close);
  m.def("symm_free", &symm_free);
  m.def("symm_fill", &symm_fill);
  m.def("symm_view", &symm_view);
}
