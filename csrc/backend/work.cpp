#include "backend/work.h"

#include <ATen/core/ivalue.h>
#include <c10/cuda/CUDAGuard.h>

#include <thread>

#include "common/errors.h"
#include "common/log.h"

namespace mccl {

WorkMCCL::WorkMCCL(int rank, c10d::OpType op, uint32_t seq, const char* profiling_title,
                   std::vector<at::Tensor> outputs, bool stream_mode, c10::DeviceIndex device)
    : c10d::Work(rank, op, profiling_title),
      seq_(seq),
      outputs_(std::move(outputs)),
      stream_mode_(stream_mode),
      device_(device) {
  // Host works create their future up front (engine threads and the caller both touch it);
  // stream works build it only if getFuture() is called.
  if (!stream_mode_) ensure_future();
}

WorkMCCL::~WorkMCCL() = default;

void WorkMCCL::ensure_future() {
  if (future_) return;
  if (stream_mode_) {
    future_ = c10::make_intrusive<c10::ivalue::Future>(
        c10::ListType::create(c10::TensorType::get()),
        std::vector<c10::Device>{c10::Device(c10::kCUDA, device_)});
  } else {
    future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
  }
}

void WorkMCCL::attach_stream(c10::cuda::CUDAStream comm, bool blocking_wait) {
  blocking_wait_ = blocking_wait;
  done_ = std::make_unique<at::cuda::CUDAEvent>(cudaEventDisableTiming);
  done_->record(comm);
  comm_ = std::make_unique<c10::cuda::CUDAStream>(comm);
  {
    std::lock_guard<std::mutex> lk(mutex_);
    completed_ = true;  // "enqueued" is the completion notion of stream-ordered work
  }
  cv_.notify_all();
}

bool WorkMCCL::isCompleted() {
  if (stream_mode_) {
    if (!done_) return false;
    return done_->query();
  }
  std::lock_guard<std::mutex> lk(mutex_);
  return completed_;
}

bool WorkMCCL::isSuccess() const {
  std::lock_guard<std::mutex> lk(mutex_);
  return completed_ && !exception_;
}

void WorkMCCL::mark_complete() {
  ensure_future();
  {
    std::lock_guard<std::mutex> lk(mutex_);
    if (completed_) return;
    completed_ = true;
  }
  cv_.notify_all();
  if (!future_->completed()) future_->markCompleted(c10::IValue(outputs_));
}

void WorkMCCL::mark_error(const std::string& msg) {
  if (stream_mode_) {  // enqueued work cannot be recalled; remember the error for wait()
    std::lock_guard<std::mutex> lk(mutex_);
    if (!exception_) exception_ = std::make_exception_ptr(MCCLError(msg));
    return;
  }
  ensure_future();
  std::exception_ptr ep = std::make_exception_ptr(MCCLError(msg));
  {
    std::lock_guard<std::mutex> lk(mutex_);
    if (completed_) return;
    completed_ = true;
    exception_ = ep;
  }
  cv_.notify_all();
  if (!future_->completed()) future_->setError(ep);
}

void WorkMCCL::synchronize() {
  if (!stream_mode_ || !done_) return;
  auto cur = c10::cuda::getCurrentCUDAStream(device_);
  done_->block(cur);
}

bool WorkMCCL::wait(std::chrono::milliseconds timeout) {
  if (stream_mode_) {
    {
      std::lock_guard<std::mutex> lk(mutex_);
      if (exception_) std::rethrow_exception(exception_);
    }
    // A bounded device-side wait that already gave up is visible in host memory: fail now instead
    // of letting the caller consume a result that was never produced.  (A failure that happens
    // after this point is caught by the next wait, the next launch, or the watchdog poll; results
    // between the failure and its detection are undefined.)
    if (quick_check_ && quick_check_() && health_check_) health_check_();
    synchronize();
    const bool blocking = blocking_wait_ || timeout != kNoTimeout;
    if (blocking && done_) {
      if (timeout == kNoTimeout) {
        done_->synchronize();
      } else {
        auto deadline = std::chrono::steady_clock::now() + timeout;
        while (!done_->query()) {
          if (std::chrono::steady_clock::now() > deadline)
            throw TimeoutError("collective seq=" + std::to_string(seq_) + " did not finish within " +
                               std::to_string(timeout.count()) + " ms");
          std::this_thread::sleep_for(std::chrono::microseconds(50));
        }
      }
      if (health_check_) health_check_();
    }
    stash_.clear();
    return true;
  }
  std::unique_lock<std::mutex> lk(mutex_);
  if (timeout == kNoTimeout) {
    cv_.wait(lk, [this] { return completed_; });
  } else if (!cv_.wait_for(lk, timeout, [this] { return completed_; })) {
    throw TimeoutError("operation seq=" + std::to_string(seq_) + " timed out after " +
                       std::to_string(timeout.count()) + " ms");
  }
  if (exception_) std::rethrow_exception(exception_);
  return true;
}

void WorkMCCL::abort() { mark_error("operation aborted"); }

c10::intrusive_ptr<c10::ivalue::Future> WorkMCCL::getFuture() {
  if (stream_mode_ && !future_) {
    ensure_future();
    if (comm_) {
      // Completing the future under the communication stream makes it record its own events
      // there (everything enqueued so far, the collective included); consumers that only look
      // at the future, like DDP's reducer, are then ordered after the kernel.
      c10::cuda::CUDAStreamGuard g(*comm_);
      future_->markCompleted(c10::IValue(outputs_));
    }
    return future_;
  }
  ensure_future();
  return future_;
}

}  // namespace mccl
