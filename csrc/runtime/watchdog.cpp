#include "runtime/watchdog.h"

#include "common/log.h"

namespace mccl {

Watchdog::Watchdog(std::chrono::milliseconds timeout, AbortFn on_abort,
                   std::chrono::milliseconds poll)
    : timeout_(timeout), poll_(poll), on_abort_(std::move(on_abort)) {}

Watchdog::~Watchdog() { stop(); }

void Watchdog::start() {
  bool expected = false;
  if (!running_.compare_exchange_strong(expected, true)) return;
  thread_ = std::thread([this] { loop(); });
}

void Watchdog::stop() {
  bool expected = true;
  if (!running_.compare_exchange_strong(expected, false)) return;
  {
    std::lock_guard<std::mutex> g(mu_);
    cv_.notify_all();
  }
  if (thread_.joinable()) thread_.join();
}

void Watchdog::watch(uint32_t seq, const std::string& name) {
  std::lock_guard<std::mutex> g(mu_);
  Entry e;
  e.name = name;
  e.deadline = Clock::time_point::max();
  e.armed = false;
  entries_[seq] = std::move(e);
}

void Watchdog::touch(uint32_t seq) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = entries_.find(seq);
  if (it == entries_.end()) return;
  it->second.deadline = Clock::now() + timeout_;
  it->second.armed = true;
}

void Watchdog::complete(uint32_t seq) {
  std::lock_guard<std::mutex> g(mu_);
  entries_.erase(seq);
}

size_t Watchdog::pending() const {
  std::lock_guard<std::mutex> g(mu_);
  return entries_.size();
}

void Watchdog::set_poll_hook(PollFn fn) {
  std::lock_guard<std::mutex> g(mu_);
  poll_hook_ = std::move(fn);
}

void Watchdog::loop() {
  while (running_.load()) {
    uint32_t expired_seq = 0;
    std::string msg;
    bool fire = false;
    PollFn hook;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait_for(lk, poll_, [this] { return !running_.load(); });
      if (!running_.load()) break;
      auto now = Clock::now();
      for (auto& kv : entries_) {
        if (kv.second.armed && kv.second.deadline <= now) {
          expired_seq = kv.first;
          msg = "watchdog: operation '" + kv.second.name + "' seq=" +
                std::to_string(kv.first) + " exceeded " +
                std::to_string(timeout_.count()) + " ms";
          fire = true;
          break;
        }
      }
      if (fire) entries_.erase(expired_seq);
      hook = poll_hook_;
    }
    if (hook) {
      try {
        hook();
      } catch (const std::exception& e) {
        MCCL_ERROR("watchdog poll hook threw: %s", e.what());
      }
    }
    if (fire) {
      MCCL_ERROR("%s", msg.c_str());
      if (on_abort_) on_abort_(expired_seq, msg);
    }
  }
}

}  // namespace mccl
