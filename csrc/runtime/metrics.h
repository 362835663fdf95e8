// Per-process-group collective metrics.
//
// Each collective is tracked from enqueue (op_start) through execution start
// (op_execute_start) to completion (op_end).  Phase times are accumulated by
// record_phase: `sync` is host time spent ordering the communication stream
// against the producer stream, `network` is the device/host time of the
// transfer phases and `reduce` the time of the reduction/epilogue.  The
// summary exposes exactly the fields of the reference's MetricsSummary
// (reference csrc/runtime/Metrics.hpp:75-89, csrc/backend/Registration.cpp:417-430).
#pragma once

#include <chrono>
#include <cstdint>
#include <deque>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace mccl {

class Metrics {
 public:
  using Clock = std::chrono::steady_clock;

  enum class Phase { SYNC, NETWORK, REDUCE };

  struct OpRecord {
    uint32_t seq = 0;
    std::string name;
    uint64_t bytes = 0;
    double queue_wait_ms = 0;
    double execution_ms = 0;
    double latency_ms = 0;
    double sync_ms = 0, network_ms = 0, reduce_ms = 0;
  };

  struct Summary {
    uint64_t total_ops = 0;
    uint64_t total_bytes_sent = 0;
    uint64_t total_bytes_recv = 0;
    uint64_t total_errors = 0;
    double avg_latency_ms = 0;
    double p50_latency_ms = 0;
    double p99_latency_ms = 0;
    double peak_throughput_gbps = 0;
    double avg_sync_ms = 0;
    double avg_network_ms = 0;
    double avg_reduce_ms = 0;
    double avg_queue_wait_ms = 0;
    double avg_execution_ms = 0;
  };

  static constexpr size_t kHistoryCap = 10000;

  void op_start(uint32_t seq, const std::string& name, uint64_t bytes);
  void op_execute_start(uint32_t seq);
  void record_phase(uint32_t seq, Phase p, double ms);
  void op_end(uint32_t seq);
  // Completion with externally measured (device) execution time.
  void op_end_timed(uint32_t seq, double execution_ms);
  // Completion of an op whose device time was not sampled: counted (ops, bytes) but kept out of
  // the latency statistics, which are over timed ops only.
  void op_end_untimed(uint32_t seq);
  void record_transport_bytes(uint64_t sent, uint64_t recv);
  void record_error();

  Summary summarize() const;
  std::vector<OpRecord> recent_ops(size_t n) const;
  void log_summary() const;
  void reset();

 private:
  struct Live {
    OpRecord rec;
    Clock::time_point t_start;
    Clock::time_point t_exec;
    bool exec_started = false;
  };
  void finish_locked(Live& lv, double exec_ms_override);

  mutable std::mutex mu_;
  std::unordered_map<uint32_t, Live> live_;
  std::deque<OpRecord> history_;
  uint64_t total_ops_ = 0, untimed_ops_ = 0, bytes_sent_ = 0, bytes_recv_ = 0, errors_ = 0;
  double peak_gbps_ = 0;
  // Running sums over all completed ops (not only the capped history).
  double sum_latency_ = 0, sum_sync_ = 0, sum_net_ = 0, sum_reduce_ = 0,
         sum_queue_ = 0, sum_exec_ = 0;
};

}  // namespace mccl
