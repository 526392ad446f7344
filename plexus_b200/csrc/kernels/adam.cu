// Multi-tensor Adam / AdamW: every flat shard (fp32 weights, bf16 feature shard with its fp32
// master copy) is updated by one launch.  Tensor descriptors travel in the kernel argument
// block; a block finds its (tensor, chunk) by a short scan over cumulative chunk counts.
//
// Reference: torch.optim.AdamW at examples/train.py:155-159 (ATen foreach kernels).

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "../include/plexus_kernels.h"

namespace plx {

constexpr int ADAM_THREADS = 256;

__global__ void __launch_bounds__(ADAM_THREADS)
adam_multi_kernel(const AdamTensors t, const AdamHyper h) {
  const int total_chunks = t.chunk_start[t.count];
  for (int chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    int ti = 0;
    while (ti + 1 < t.count && chunk >= t.chunk_start[ti + 1]) ++ti;
    const int64_t base = static_cast<int64_t>(chunk - t.chunk_start[ti]) * ADAM_CHUNK;
    const int64_t rest = t.numel[ti] - base;
    const int64_t n = rest < ADAM_CHUNK ? rest : ADAM_CHUNK;
    float* m = t.exp_avg[ti] + base;
    float* v = t.exp_avg_sq[ti] + base;
    float* w32 = t.master[ti] ? t.master[ti] + base : nullptr;
    for (int i = threadIdx.x; i < n; i += ADAM_THREADS) {
      float g, w;
      if (t.is_bf16[ti]) {
        g = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(t.grad[ti])[base + i]);
        w = w32 ? w32[i] : __bfloat162float(reinterpret_cast<__nv_bfloat16*>(t.param[ti])[base + i]);
      } else {
        g = reinterpret_cast<const float*>(t.grad[ti])[base + i];
        w = reinterpret_cast<float*>(t.param[ti])[base + i];
      }
      if (h.weight_decay != 0.f) {
        if (h.decoupled) w *= 1.f - h.lr * h.weight_decay;
        else g += h.weight_decay * w;
      }
      const float mi = h.beta1 * m[i] + (1.f - h.beta1) * g;
      const float vi = h.beta2 * v[i] + (1.f - h.beta2) * g * g;
      m[i] = mi;
      v[i] = vi;
      w -= (h.lr / h.bc1) * mi / (sqrtf(vi / h.bc2) + h.eps);
      if (t.is_bf16[ti]) {
        if (w32) w32[i] = w;
        reinterpret_cast<__nv_bfloat16*>(t.param[ti])[base + i] = __float2bfloat16_rn(w);
      } else {
        reinterpret_cast<float*>(t.param[ti])[base + i] = w;
      }
    }
  }
}

const char* launch_adam_multi(const AdamTensors& t, const AdamHyper& h, cudaStream_t stream) {
  const int chunks = t.chunk_start[t.count];
  if (chunks == 0) return nullptr;
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  adam_multi_kernel<<<std::min(chunks, sms * 16), ADAM_THREADS, 0, stream>>>(t, h);
  return last_launch_error();
}

}  // namespace plx
