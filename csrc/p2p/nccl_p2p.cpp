#include "p2p/nccl_p2p.h"

#ifndef USE_C10D_NCCL
#define USE_C10D_NCCL
#endif
#include <torch/csrc/distributed/c10d/PrefixStore.hpp>
#include <torch/csrc/distributed/c10d/ProcessGroupNCCL.hpp>

namespace mccl {

NcclP2P::NcclP2P(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                 std::chrono::milliseconds timeout) {
  auto opts = c10d::ProcessGroupNCCL::Options::create();
  opts->timeout = timeout;
  auto prefixed = c10::make_intrusive<c10d::PrefixStore>("mccl_p2p", store);
  pg_ = c10::make_intrusive<c10d::ProcessGroupNCCL>(prefixed, rank, size, opts);
}

NcclP2P::~NcclP2P() { shutdown(); }

void NcclP2P::shutdown() {
  if (pg_) {
    try {
      pg_->shutdown();
    } catch (...) {
    }
    pg_.reset();
  }
}

c10::intrusive_ptr<c10d::Work> NcclP2P::send(std::vector<at::Tensor>& tensors, int dst, int tag) {
  return pg_->send(tensors, dst, tag);
}
c10::intrusive_ptr<c10d::Work> NcclP2P::recv(std::vector<at::Tensor>& tensors, int src, int tag) {
  return pg_->recv(tensors, src, tag);
}

}  // namespace mccl
