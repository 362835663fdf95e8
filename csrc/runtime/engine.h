// HostEngine: bounded FIFO of host-side operations with N worker threads.
//
// `submit(execute, on_complete, on_error)` blocks the caller while the queue is
// at `max_queue_depth` (back-pressure).  Operations START in submission order;
// with more than one worker they may run concurrently.  A worker runs
// `execute`; if it returns normally `on_complete` is called, if it throws
// `on_error(message)` is.  `shutdown()` stops the workers and fails every
// operation still queued through `on_error`, so no Work is left pending.
// On the CUDA path collectives are stream-ordered launches and never pass
// through here; the engine carries CPU-tensor collectives, point-to-point
// operations and abort propagation.
// Parity: reference csrc/runtime/ProgressEngine.hpp:44-46, ProgressEngine.cpp:53-197.
#pragma once

#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace mccl {

class HostEngine {
 public:
  using Fn = std::function<void()>;
  using ErrFn = std::function<void(const std::string&)>;

  HostEngine(std::string name, int workers, size_t max_queue_depth)
      : name_(std::move(name)), max_depth_(max_queue_depth ? max_queue_depth : 1) {
    running_ = true;
    if (workers < 1) workers = 1;
    for (int i = 0; i < workers; ++i) threads_.emplace_back([this] { worker(); });
  }
  ~HostEngine() { shutdown(); }

  // Returns false (after calling on_error) if the engine is shut down.
  bool submit(Fn execute, Fn on_complete, ErrFn on_error) {
    std::unique_lock<std::mutex> lk(mu_);
    not_full_.wait(lk, [this] { return !running_ || queue_.size() < max_depth_; });
    if (!running_) {
      lk.unlock();
      if (on_error) on_error("engine '" + name_ + "' is shut down");
      return false;
    }
    queue_.push_back(Item{std::move(execute), std::move(on_complete), std::move(on_error)});
    submitted_++;
    not_empty_.notify_one();
    return true;
  }

  void shutdown() {
    std::deque<Item> orphans;
    {
      std::lock_guard<std::mutex> g(mu_);
      if (!running_ && threads_.empty()) return;
      running_ = false;
      orphans.swap(queue_);
      not_empty_.notify_all();
      not_full_.notify_all();
    }
    for (auto& t : threads_)
      if (t.joinable()) t.join();
    threads_.clear();
    for (auto& it : orphans)
      if (it.on_error) it.on_error("engine '" + name_ + "' shut down before the operation ran");
  }

  // Blocks until everything submitted so far has finished.
  void drain() {
    std::unique_lock<std::mutex> lk(mu_);
    idle_.wait(lk, [this] { return !running_ || (queue_.empty() && active_ == 0); });
  }

  size_t queue_depth() const {
    std::lock_guard<std::mutex> g(mu_);
    return queue_.size();
  }
  uint64_t submitted() const { return submitted_.load(); }
  uint64_t completed() const { return completed_.load(); }

 private:
  struct Item {
    Fn execute, on_complete;
    ErrFn on_error;
  };

  void worker() {
    for (;;) {
      Item it;
      {
        std::unique_lock<std::mutex> lk(mu_);
        not_empty_.wait(lk, [this] { return !running_ || !queue_.empty(); });
        if (!running_) return;
        it = std::move(queue_.front());
        queue_.pop_front();
        active_++;
        not_full_.notify_one();
      }
      bool ok = true;
      std::string err;
      try {
        if (it.execute) it.execute();
      } catch (const std::exception& e) {
        ok = false;
        err = e.what();
      } catch (...) {
        ok = false;
        err = "unknown exception";
      }
      try {
        if (ok) {
          if (it.on_complete) it.on_complete();
        } else if (it.on_error) {
          it.on_error(err);
        }
      } catch (...) {
      }
      completed_++;
      {
        std::lock_guard<std::mutex> g(mu_);
        active_--;
        if (queue_.empty() && active_ == 0) idle_.notify_all();
      }
    }
  }

  std::string name_;
  size_t max_depth_;
  mutable std::mutex mu_;
  std::condition_variable not_empty_, not_full_, idle_;
  std::deque<Item> queue_;
  std::vector<std::thread> threads_;
  bool running_ = false;
  int active_ = 0;
  std::atomic<uint64_t> submitted_{0}, completed_{0};
};

}  // namespace mccl
