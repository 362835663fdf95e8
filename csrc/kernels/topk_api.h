// Launchers of the fused top-k compressed allreduce kernels (plain C++ header).
//
// Pipeline for one gradient bucket g (fp32 or bf16) with fp32 residual e:
//   select   a = g + e;  pick the k entries of largest |a| exactly (3-level
//            radix select on the magnitude bits, ties to the lower index);
//            emit them as (u32 index, f32 value) pairs sorted by index;
//            e = a with the k selected entries zeroed          (topk_select)
//            Three passes over the data: adjust + 13-bit histogram (12 B per
//            fp32 element), collect (4 B: per-block counts of the elements
//            above the chosen bin, the elements inside it go to a candidate
//            list on which the remaining 18 bits are resolved), ordered
//            compaction (4 B).  Only if the bin holds more than k elements
//            (heavily tied data) two more full histogram passes and a count
//            pass run instead of the candidate refinement.
//   exchange every rank pushes its k pairs into slot[rank] of every peer's
//            arena over NVLink, release flag                    (exchange)
//   scatter  dense = scale * sum_r sparse_r, written into g: each CTA owns a
//            contiguous index range, zero-fills it and applies the ws sorted
//            lists in rank order without atomics, so every rank produces
//            bit-identical dense results                        (scatter)
// exchange + scatter are one kernel.
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

#include "kernels/api.h"

namespace mccl {
namespace kern {

constexpr int kTopkMaxBlocks = 1024;   // blocks of the ordered compaction
constexpr int kTopkBins0 = 8192;       // bins of the first radix level (13 magnitude bits)
constexpr int kTopkBins12 = 512;       // bins of the second and third level (9 bits each)

struct TopkArgs {
  const void* grad;     // n elements, fp32 or bf16; overwritten with the dense result by scatter
  bool grad_is_bf16;
  float* residual;      // n fp32, in/out
  int64_t n;
  int64_t k;
  void* scratch;        // topk_scratch_bytes() bytes of device memory (any contents)
  void* pairs;          // k * 8 bytes: {u32 index, f32 value}
  float scale;          // applied in scatter
};

// Scratch layout: 3 histograms, the selection state, per-block counts/offsets (about 53 KB).
size_t topk_scratch_bytes();
#ifdef __CUDACC__
__host__ __device__
#endif
inline size_t topk_pad(size_t bytes) { return (bytes + 127) / 128 * 128; }

cudaError_t launch_topk_select(const TopkArgs& a, cudaStream_t s);
// p: arena parameters (ctx[].in = pairs, ctx[].out = dense gradient); count = k.
cudaError_t launch_topk_exchange_scatter(const CollParams& p, const TopkArgs& a, LaunchCfg cfg, cudaStream_t s);
// World size 1: dense = scale * sparse.
cudaError_t launch_topk_local_scatter(const TopkArgs& a, cudaStream_t s);

}  // namespace kern
}  // namespace mccl
