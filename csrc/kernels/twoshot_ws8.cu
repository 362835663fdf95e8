// Two-shot allreduce / reduce_scatter kernels for five to eight ranks.
#include "kernels/twoshot.cuh"

namespace mccl {
namespace kern {

cudaError_t launch_twoshot_ws8(bool allgather, const CollParams& p, DType dtype, DType wire, int ctas,
                               const LaunchCfg& cfg, cudaStream_t s) {
  return TwoShotClass<8>::launch(allgather, p, dtype, wire, ctas, cfg, s);
}

}  // namespace kern
}  // namespace mccl
