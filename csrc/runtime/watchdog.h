// Deadline watchdog for in-flight collectives.
//
// `watch(seq, name)` registers an operation UNARMED (no deadline) so that an
// operation sitting in a queue behind others can never expire.  `touch(seq)`
// arms or re-arms the deadline (now + timeout); it is called when execution
// starts and at every phase boundary.  `complete(seq)` removes the entry.  A
// monitor thread polls (every `poll_ms`) and calls `on_abort(seq, message)` once
// for the first expired entry; it also runs the optional `poll_hook`, which the
// CUDA path uses to read the device status words written by bounded in-kernel
// waits.  Parity: reference csrc/runtime/Watchdog.hpp:33-46, Watchdog.cpp:33-98.
#pragma once

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>

namespace mccl {

class Watchdog {
 public:
  using Clock = std::chrono::steady_clock;
  using AbortFn = std::function<void(uint32_t, const std::string&)>;
  using PollFn = std::function<void()>;

  Watchdog(std::chrono::milliseconds timeout, AbortFn on_abort,
           std::chrono::milliseconds poll = std::chrono::milliseconds(500));
  ~Watchdog();

  void start();
  void stop();

  void watch(uint32_t seq, const std::string& name);
  void touch(uint32_t seq);
  void complete(uint32_t seq);
  size_t pending() const;
  void set_poll_hook(PollFn fn);
  std::chrono::milliseconds timeout() const { return timeout_; }

 private:
  void loop();

  struct Entry {
    std::string name;
    Clock::time_point deadline;
    bool armed = false;
  };

  std::chrono::milliseconds timeout_;
  std::chrono::milliseconds poll_;
  AbortFn on_abort_;
  PollFn poll_hook_;
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::unordered_map<uint32_t, Entry> entries_;
  std::thread thread_;
  std::atomic<bool> running_{false};
};

}  // namespace mccl
