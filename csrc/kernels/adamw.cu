// Fused multi-tensor AdamW step (sm_100a): one launch updates every parameter
// of the model.  The optimizer step follows the gradient allreduce on the same
// data; doing it in one pass over (p, g, m, v) keeps the step at its HBM floor of
// 28 bytes per fp32 parameter instead of one launch per tensor.
//
// A device-resident table maps each CTA to (tensor, chunk); tensors are
// addressed through pointer arrays, so parameters stay ordinary, separately
// allocated torch tensors (state_dict and checkpoints are unaffected).
// Numerics follow torch.optim.AdamW (decoupled weight decay):
//   p *= 1 - lr*wd;  m = b1*m + (1-b1)*g;  v = b2*v + (1-b2)*g*g
//   p -= (lr / (1-b1^t)) * m / (sqrt(v) / sqrt(1-b2^t) + eps)
// `grad_scale` is multiplied into g first (loss-scale / deferred averaging).
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels/launch_count.h"
#include "kernels/optim_api.h"

namespace mccl {
namespace kern {

namespace {

__device__ __forceinline__ void adamw_chunk(const AdamWTable& tab, const AdamWHyper& h, int chunk) {
  const int2 ent = tab.chunks[chunk];
  const int t = ent.x;
  const int64_t start = static_cast<int64_t>(ent.y) * kAdamWChunk;
  const int64_t n = tab.sizes[t];
  int64_t end = start + kAdamWChunk;
  if (end > n) end = n;
  float* __restrict__ p = reinterpret_cast<float*>(tab.params[t]);
  const float* __restrict__ g = reinterpret_cast<const float*>(tab.grads[t]);
  float* __restrict__ m = reinterpret_cast<float*>(tab.exp_avg[t]);
  float* __restrict__ v = reinterpret_cast<float*>(tab.exp_avg_sq[t]);
  const float decay = 1.0f - h.lr * h.weight_decay;
  const float one_m_b1 = 1.0f - h.beta1, one_m_b2 = 1.0f - h.beta2;

  auto update = [&](float& pp, float gg, float& mm, float& vv) {
    gg *= h.grad_scale;
    pp *= decay;
    mm = h.beta1 * mm + one_m_b1 * gg;
    vv = h.beta2 * vv + one_m_b2 * gg * gg;
    const float denom = sqrtf(vv) * h.inv_sqrt_bias2 + h.eps;
    pp -= h.step_size * (mm / denom);
  };

  const bool vec_ok = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                        reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15) == 0;
  if (vec_ok) {
    // chunk starts are multiples of 4, so 16-byte alignment carries over
    const int64_t nvec = (end - start) / 4;
    float4* p4 = reinterpret_cast<float4*>(p + start);
    const float4* g4 = reinterpret_cast<const float4*>(g + start);
    float4* m4 = reinterpret_cast<float4*>(m + start);
    float4* v4 = reinterpret_cast<float4*>(v + start);
    for (int64_t i = threadIdx.x; i < nvec; i += blockDim.x) {
      float4 pp = p4[i], gg = __ldcs(g4 + i), mm = m4[i], vv = v4[i];
      update(pp.x, gg.x, mm.x, vv.x);
      update(pp.y, gg.y, mm.y, vv.y);
      update(pp.z, gg.z, mm.z, vv.z);
      update(pp.w, gg.w, mm.w, vv.w);
      p4[i] = pp;
      m4[i] = mm;
      v4[i] = vv;
    }
    for (int64_t i = start + nvec * 4 + threadIdx.x; i < end; i += blockDim.x) update(p[i], g[i], m[i], v[i]);
  } else {
    for (int64_t i = start + threadIdx.x; i < end; i += blockDim.x) update(p[i], g[i], m[i], v[i]);
  }
}

// One chunk per CTA: the grid covers the table.
__global__ void __launch_bounds__(256) adamw_multi_kernel(const AdamWTable tab, AdamWHyper h) {
  adamw_chunk(tab, h, blockIdx.x);
}

// The launcher capped the grid: every CTA walks several chunks (a separate kernel so that the
// uncapped step keeps its register count and occupancy).
__global__ void __launch_bounds__(256) adamw_multi_capped_kernel(const AdamWTable tab, AdamWHyper h) {
  for (int c = blockIdx.x; c < tab.num_chunks; c += gridDim.x) adamw_chunk(tab, h, c);
}

}  // namespace

cudaError_t launch_adamw_multi(const AdamWTable& tab, const AdamWHyper& h, cudaStream_t s, int max_ctas) {
  if (tab.num_chunks <= 0) return cudaSuccess;
  note_launch();
  if (max_ctas > 0 && max_ctas < tab.num_chunks)
    adamw_multi_capped_kernel<<<max_ctas, 256, 0, s>>>(tab, h);
  else
    adamw_multi_kernel<<<tab.num_chunks, 256, 0, s>>>(tab, h);
  return cudaGetLastError();
}

}  // namespace kern
}  // namespace mccl
