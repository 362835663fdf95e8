// Launcher of the fused multi-tensor AdamW kernel (plain C++ header).
#pragma once

#include <cuda_runtime_api.h>
#include <vector_types.h>

#include <cstdint>

namespace mccl {
namespace kern {

constexpr int kAdamWChunk = 16384;  // elements handled by one CTA (multiple of 4)

// All pointers are device pointers; arrays are indexed by tensor id.
struct AdamWTable {
  const uint64_t* params;      // float* per tensor
  const uint64_t* grads;       // const float* per tensor
  const uint64_t* exp_avg;     // float* per tensor
  const uint64_t* exp_avg_sq;  // float* per tensor
  const int64_t* sizes;        // elements per tensor
  const int2* chunks;          // per CTA: {tensor id, chunk index}
  int num_chunks;
};

struct AdamWHyper {
  float lr;
  float beta1, beta2;
  float eps;
  float weight_decay;
  float step_size;       // lr / (1 - beta1^t)
  float inv_sqrt_bias2;  // 1 / sqrt(1 - beta2^t)
  float grad_scale;      // multiplied into every gradient first
};

// `max_ctas` > 0 caps the grid (each CTA then walks several chunks): a step that runs beside other
// kernels (a bucket's update during backward) can be kept to a share of the SMs and of HBM bandwidth.
cudaError_t launch_adamw_multi(const AdamWTable& tab, const AdamWHyper& h, cudaStream_t s, int max_ctas = 0);

}  // namespace kern
}  // namespace mccl
