// Point-to-point transfers of CUDA tensors over NCCL.
//
// send/recv are the one place this backend uses NCCL: torch's ProcessGroupNCCL
// is embedded as a private helper and only its send/recv are called.  It creates
// a two-rank communicator per (src, dst) pair lazily on first use, runs the
// transfer on its own side stream (so it overlaps with collectives in flight on
// the arena lanes) and returns a stream-ordered Work.  Nothing here is on the
// DDP hot path.  NCCL matches messages by order per pair, not by tag.
// Replaces the reference's framed TCP p2p for device tensors
// (reference csrc/backend/ProcessGroupMCCL.cpp:3333-3462).
#pragma once

#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>

#include <chrono>

namespace mccl {

class NcclP2P {
 public:
  NcclP2P(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, std::chrono::milliseconds timeout);
  ~NcclP2P();
  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& tensors, int dst, int tag);
  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& tensors, int src, int tag);
  void shutdown();

 private:
  c10::intrusive_ptr<c10d::Backend> pg_;
};

}  // namespace mccl
