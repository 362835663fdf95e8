// Store-backed rendezvous: all-to-all exchange of small opaque values and a
// reusable barrier.
//
// exchange(tag, mine): every rank sets "mccl/<tag>/<rank>" and reads all ranks'
// values (used for host-transport endpoints and arena IPC handles).
// barrier(tag): epoch-keyed -- rank r sets "mccl/barrier/<tag>/<epoch>/<r>" and
// waits for every rank's key of that epoch; the epoch advances locally per tag,
// so the same tag is reusable without deleting keys.  dist.barrier() on CPU
// tensors is this barrier.
// Parity: reference csrc/runtime/Rendezvous.hpp:26-31, Rendezvous.cpp:15-89.
#pragma once

#include <torch/csrc/distributed/c10d/Store.hpp>

#include <chrono>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace mccl {

class Rendezvous {
 public:
  Rendezvous(c10::intrusive_ptr<c10d::Store> store, int rank, int world_size)
      : store_(std::move(store)), rank_(rank), ws_(world_size) {}

  std::vector<std::string> exchange(const std::string& tag, const std::string& mine,
                                    std::chrono::milliseconds timeout) {
    const std::string prefix = "mccl/" + tag + "/";
    store_->set(prefix + std::to_string(rank_), std::vector<uint8_t>(mine.begin(), mine.end()));
    std::vector<std::string> out(ws_);
    for (int r = 0; r < ws_; ++r) {
      if (r == rank_) {
        out[r] = mine;
        continue;
      }
      const std::string key = prefix + std::to_string(r);
      store_->wait({key}, timeout);
      auto v = store_->get(key);
      out[r].assign(v.begin(), v.end());
    }
    return out;
  }

  void barrier(const std::string& tag, std::chrono::milliseconds timeout) {
    uint64_t epoch;
    {
      std::lock_guard<std::mutex> g(mu_);
      epoch = ++epochs_[tag];
    }
    const std::string prefix = "mccl/barrier/" + tag + "/" + std::to_string(epoch) + "/";
    store_->set(prefix + std::to_string(rank_), std::vector<uint8_t>{1});
    std::vector<std::string> keys;
    for (int r = 0; r < ws_; ++r)
      if (r != rank_) keys.push_back(prefix + std::to_string(r));
    if (!keys.empty()) store_->wait(keys, timeout);
  }

  // Small shared flags (abort key, heartbeat counters).
  void put(const std::string& key, const std::string& v) {
    store_->set("mccl/" + key, std::vector<uint8_t>(v.begin(), v.end()));
  }
  bool has(const std::string& key) { return store_->check({"mccl/" + key}); }
  int64_t add(const std::string& key, int64_t delta) { return store_->add("mccl/" + key, delta); }

  c10d::Store& store() { return *store_; }

 private:
  c10::intrusive_ptr<c10d::Store> store_;
  int rank_, ws_;
  std::mutex mu_;
  std::unordered_map<std::string, uint64_t> epochs_;
};

}  // namespace mccl
