// Two-shot allreduce / reduce_scatter kernels for three or four ranks.
#include "kernels/twoshot.cuh"

namespace mccl {
namespace kern {

cudaError_t launch_twoshot_ws4(bool allgather, const CollParams& p, DType dtype, DType wire, int ctas,
                               const LaunchCfg& cfg, cudaStream_t s) {
  return TwoShotClass<4>::launch(allgather, p, dtype, wire, ctas, cfg, s);
}

}  // namespace kern
}  // namespace mccl
