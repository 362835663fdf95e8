// Peer liveness monitor.
//
// Every `interval` the monitor asks `is_alive(peer)` for each peer that is
// still considered alive.  The first negative answer marks the peer dead and
// calls `on_death(peer)` exactly once.  The liveness predicate is supplied by
// the process group: it combines the host transport's connection state with a
// heartbeat counter each rank publishes in the c10d Store, so a rank that has
// exited is noticed on the host before the survivors launch another kernel.
// Parity: reference csrc/runtime/HealthMonitor.hpp:24-57 (which only polled the
// transport and never sent its HEARTBEAT frames; this one does probe).
#pragma once

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace mccl {

class HealthMonitor {
 public:
  using AliveFn = std::function<bool(int)>;
  using DeathFn = std::function<void(int)>;
  using BeatFn = std::function<void()>;

  HealthMonitor(int rank, int world_size, std::chrono::milliseconds interval,
                AliveFn is_alive, DeathFn on_death, BeatFn beat = nullptr)
      : rank_(rank), ws_(world_size), interval_(interval),
        is_alive_(std::move(is_alive)), on_death_(std::move(on_death)),
        beat_(std::move(beat)), dead_(world_size, false) {}
  ~HealthMonitor() { stop(); }

  void start() {
    bool e = false;
    if (!running_.compare_exchange_strong(e, true)) return;
    thread_ = std::thread([this] { loop(); });
  }
  void stop() {
    bool e = true;
    if (!running_.compare_exchange_strong(e, false)) return;
    {
      std::lock_guard<std::mutex> g(mu_);
      cv_.notify_all();
    }
    if (thread_.joinable()) thread_.join();
  }
  bool is_dead(int peer) const {
    std::lock_guard<std::mutex> g(mu_);
    return peer >= 0 && peer < ws_ && dead_[peer];
  }
  int dead_count() const {
    std::lock_guard<std::mutex> g(mu_);
    int n = 0;
    for (bool d : dead_) n += d ? 1 : 0;
    return n;
  }
  // Runs one sweep synchronously (used by tests and before kernel launches).
  void check_now() { sweep(); }

 private:
  void sweep() {
    if (beat_) {
      try { beat_(); } catch (...) {}
    }
    for (int p = 0; p < ws_; ++p) {
      if (p == rank_) continue;
      {
        std::lock_guard<std::mutex> g(mu_);
        if (dead_[p]) continue;
      }
      bool alive = true;
      try { alive = is_alive_(p); } catch (...) { alive = false; }
      if (!alive) {
        {
          std::lock_guard<std::mutex> g(mu_);
          if (dead_[p]) continue;
          dead_[p] = true;
        }
        if (on_death_) on_death_(p);
      }
    }
  }
  void loop() {
    while (running_.load()) {
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait_for(lk, interval_, [this] { return !running_.load(); });
      }
      if (!running_.load()) break;
      sweep();
    }
  }

  int rank_, ws_;
  std::chrono::milliseconds interval_;
  AliveFn is_alive_;
  DeathFn on_death_;
  BeatFn beat_;
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::vector<bool> dead_;
  std::thread thread_;
  std::atomic<bool> running_{false};
};

}  // namespace mccl
