// WorkMCCL: completion handle of one collective.
//
// Host mode (CPU tensors, point-to-point): completed from an engine thread via
// mark_complete / mark_error; wait() blocks on a condition variable and throws
// TimeoutError when `timeout` expires.
//
// Stream mode (CUDA tensors): the collective is a stream-ordered launch on the
// process group's communication stream and `done` is an event recorded behind
// it.  wait() makes the CALLER'S CURRENT STREAM wait for that event and returns
// without blocking the host (blocking only for barrier works or when asked via
// MCCL_BLOCKING_WAIT / a finite timeout, in which case device-side failures
// recorded in the arena status block are raised as exceptions).  getFuture()
// returns a CUDA-aware future that was completed under the communication
// stream, so DistributedDataParallel's reducer, which consumes results only
// through the future, is ordered after the kernel as well.
//
// Parity: reference csrc/backend/WorkMCCL.hpp:16-58 and WorkMCCL.cpp:26-168
// (its MTLSharedEvent consumer release becomes cudaStreamWaitEvent).
#pragma once

#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/distributed/c10d/Work.hpp>

#include <functional>
#include <memory>
#include <string>
#include <vector>

namespace mccl {

class WorkMCCL : public c10d::Work {
 public:
  WorkMCCL(int rank, c10d::OpType op, uint32_t seq, const char* profiling_title,
           std::vector<at::Tensor> outputs, bool stream_mode, c10::DeviceIndex device);
  ~WorkMCCL() override;

  bool isCompleted() override;
  bool isSuccess() const override;
  bool wait(std::chrono::milliseconds timeout = kNoTimeout) override;
  void synchronize() override;
  void abort() override;
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override;
  std::vector<at::Tensor> result() override { return outputs_; }
  uint64_t getSequencenumber() const override { return seq_; }

  // host mode
  void mark_complete();
  void mark_error(const std::string& msg);

  // stream mode: called once the kernels are enqueued on `comm`.
  void attach_stream(c10::cuda::CUDAStream comm, bool blocking_wait);
  // Keeps temporaries alive until the work is waited on / destroyed.
  void stash(std::vector<at::Tensor> tensors) {
    for (auto& t : tensors) stash_.push_back(std::move(t));
  }
  // Runs after the device work is known complete in a blocking wait; may throw.
  void set_health_check(std::function<void()> fn) { health_check_ = std::move(fn); }
  // Cheap test run by every wait(), blocking or not: returns true when the device has already
  // reported a failure (the full health check then runs and throws).
  void set_quick_check(std::function<bool()> fn) { quick_check_ = std::move(fn); }

  uint32_t seq() const { return seq_; }
  bool stream_mode() const { return stream_mode_; }

 private:
  void ensure_future();

  uint32_t seq_;
  std::vector<at::Tensor> outputs_;
  std::vector<at::Tensor> stash_;
  bool stream_mode_;
  c10::DeviceIndex device_;
  bool blocking_wait_ = false;
  std::unique_ptr<at::cuda::CUDAEvent> done_;
  std::unique_ptr<c10::cuda::CUDAStream> comm_;  // stream the collective was enqueued on
  c10::intrusive_ptr<c10::ivalue::Future> future_;
  std::function<void()> health_check_;
  std::function<bool()> quick_check_;
};

}  // namespace mccl
