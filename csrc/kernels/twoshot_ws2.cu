// Two-shot allreduce / reduce_scatter kernels for exactly two ranks.
#include "kernels/twoshot.cuh"

namespace mccl {
namespace kern {

cudaError_t launch_twoshot_ws2(bool allgather, const CollParams& p, DType dtype, DType wire, int ctas,
                               const LaunchCfg& cfg, cudaStream_t s) {
  return TwoShotClass<2>::launch(allgather, p, dtype, wire, ctas, cfg, s);
}

}  // namespace kern
}  // namespace mccl
