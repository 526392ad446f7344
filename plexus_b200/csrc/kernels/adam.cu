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

__device__ __forceinline__ void adam_update(float& w, float g, float& m, float& v, const AdamHyper& h) {
  if (h.weight_decay != 0.f) {
    if (h.decoupled) w *= 1.f - h.lr * h.weight_decay;
    else g += h.weight_decay * w;
  }
  m = h.beta1 * m + (1.f - h.beta1) * g;
  v = h.beta2 * v + (1.f - h.beta2) * g * g;
  w -= (h.lr / h.bc1) * m / (sqrtf(v / h.bc2) + h.eps);
}

// One chunk of ADAM_CHUNK elements per block iteration; 4 elements per thread per step with
// 16-byte loads of the fp32 streams (8-byte for bf16), scalar code for ragged tails.
__global__ void __launch_bounds__(ADAM_THREADS)
adam_multi_kernel(const AdamTensors t, const AdamHyper h) {
  const int total_chunks = t.chunk_start[t.count];
  for (int chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    int ti = 0;
#pragma unroll 1
    while (ti + 1 < t.count && chunk >= t.chunk_start[ti + 1]) ++ti;
    // copy this tensor's descriptor out of the parameter block with static indexing
    void* param = nullptr;
    const void* grad = nullptr;
    float *em = nullptr, *ev = nullptr, *master = nullptr;
    int64_t numel = 0;
    int is_bf16 = 0, cstart = 0;
#pragma unroll
    for (int k = 0; k < ADAM_MAX_TENSORS; ++k)
      if (k == ti) {
        param = t.param[k];
        grad = t.grad[k];
        em = t.exp_avg[k];
        ev = t.exp_avg_sq[k];
        master = t.master[k];
        numel = t.numel[k];
        is_bf16 = t.is_bf16[k];
        cstart = t.chunk_start[k];
      }
    const int64_t base = static_cast<int64_t>(chunk - cstart) * ADAM_CHUNK;
    const int64_t rest = numel - base;
    const int n = static_cast<int>(rest < ADAM_CHUNK ? rest : ADAM_CHUNK);
    float* m = em + base;
    float* v = ev + base;
    float* w32 = master ? master + base : nullptr;
    // all streams start 16-byte aligned (base is a multiple of 4096 elements, torch allocations are aligned)
    const bool vec_ok = (n % 4 == 0) && (reinterpret_cast<uintptr_t>(m) % 16 == 0) &&
                        (reinterpret_cast<uintptr_t>(v) % 16 == 0) &&
                        (reinterpret_cast<uintptr_t>(param) % 16 == 0) &&
                        (reinterpret_cast<uintptr_t>(grad) % 16 == 0) &&
                        (w32 == nullptr || reinterpret_cast<uintptr_t>(w32) % 16 == 0);
    if (vec_ok) {
      for (int i = threadIdx.x * 4; i < n; i += ADAM_THREADS * 4) {
        float4 m4 = *reinterpret_cast<float4*>(m + i), v4 = *reinterpret_cast<float4*>(v + i);
        float g4[4], w4[4];
        if (is_bf16) {
          const uint2 gr = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(grad) + base + i);
          const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gr);
          float2 a = __bfloat1622float2(gp[0]), b = __bfloat1622float2(gp[1]);
          g4[0] = a.x; g4[1] = a.y; g4[2] = b.x; g4[3] = b.y;
          if (w32) {
            const float4 ww = *reinterpret_cast<const float4*>(w32 + i);
            w4[0] = ww.x; w4[1] = ww.y; w4[2] = ww.z; w4[3] = ww.w;
          } else {
            const uint2 pr = *reinterpret_cast<const uint2*>(reinterpret_cast<__nv_bfloat16*>(param) + base + i);
            const __nv_bfloat162* pp = reinterpret_cast<const __nv_bfloat162*>(&pr);
            float2 c = __bfloat1622float2(pp[0]), d = __bfloat1622float2(pp[1]);
            w4[0] = c.x; w4[1] = c.y; w4[2] = d.x; w4[3] = d.y;
          }
        } else {
          const float4 gg = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grad) + base + i);
          const float4 ww = *reinterpret_cast<const float4*>(reinterpret_cast<float*>(param) + base + i);
          g4[0] = gg.x; g4[1] = gg.y; g4[2] = gg.z; g4[3] = gg.w;
          w4[0] = ww.x; w4[1] = ww.y; w4[2] = ww.z; w4[3] = ww.w;
        }
        float mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) adam_update(w4[k], g4[k], mm[k], vv[k], h);
        *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
        *reinterpret_cast<float4*>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
        if (is_bf16) {
          if (w32) *reinterpret_cast<float4*>(w32 + i) = make_float4(w4[0], w4[1], w4[2], w4[3]);
          uint2 pw;
          __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&pw);
          pp[0] = __floats2bfloat162_rn(w4[0], w4[1]);
          pp[1] = __floats2bfloat162_rn(w4[2], w4[3]);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(param) + base + i) = pw;
        } else {
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(param) + base + i) =
              make_float4(w4[0], w4[1], w4[2], w4[3]);
        }
      }
    } else {
      for (int i = threadIdx.x; i < n; i += ADAM_THREADS) {
        float g, w;
        if (is_bf16) {
          g = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(grad)[base + i]);
          w = w32 ? w32[i] : __bfloat162float(reinterpret_cast<__nv_bfloat16*>(param)[base + i]);
        } else {
          g = reinterpret_cast<const float*>(grad)[base + i];
          w = reinterpret_cast<float*>(param)[base + i];
        }
        float mi = m[i], vi = v[i];
        adam_update(w, g, mi, vi, h);
        m[i] = mi;
        v[i] = vi;
        if (is_bf16) {
          if (w32) w32[i] = w;
          reinterpret_cast<__nv_bfloat16*>(param)[base + i] = __float2bfloat16_rn(w);
        } else {
          reinterpret_cast<float*>(param)[base + i] = w;
        }
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
