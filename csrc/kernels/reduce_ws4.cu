// One-shot / two-shot allreduce and reduce_scatter kernels for three or four ranks.
#include "kernels/reduce_kernels.cuh"

namespace mccl {
namespace kern {

cudaError_t launch_reduce_ws4(int kind, const CollParams& p, DType dtype, DType wire, int ctas,
                              const LaunchCfg& cfg, cudaStream_t s) {
  return ReduceClass<4>::launch(kind, p, dtype, wire, ctas, cfg, s);
}

}  // namespace kern
}  // namespace mccl
