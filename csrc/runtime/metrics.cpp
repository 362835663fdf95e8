#include "runtime/metrics.h"

#include <algorithm>

#include "common/log.h"

namespace mccl {

static double ms_between(Metrics::Clock::time_point a, Metrics::Clock::time_point b) {
  return std::chrono::duration<double, std::milli>(b - a).count();
}

void Metrics::op_start(uint32_t seq, const std::string& name, uint64_t bytes) {
  std::lock_guard<std::mutex> g(mu_);
  Live lv;
  lv.rec.seq = seq;
  lv.rec.name = name;
  lv.rec.bytes = bytes;
  lv.t_start = Clock::now();
  live_[seq] = std::move(lv);
}

void Metrics::op_execute_start(uint32_t seq) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = live_.find(seq);
  if (it == live_.end()) return;
  it->second.t_exec = Clock::now();
  it->second.exec_started = true;
  it->second.rec.queue_wait_ms = ms_between(it->second.t_start, it->second.t_exec);
}

void Metrics::record_phase(uint32_t seq, Phase p, double ms) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = live_.find(seq);
  if (it == live_.end()) return;
  switch (p) {
    case Phase::SYNC: it->second.rec.sync_ms += ms; break;
    case Phase::NETWORK: it->second.rec.network_ms += ms; break;
    case Phase::REDUCE: it->second.rec.reduce_ms += ms; break;
  }
}

void Metrics::finish_locked(Live& lv, double exec_override) {
  auto now = Clock::now();
  OpRecord& r = lv.rec;
  r.latency_ms = ms_between(lv.t_start, now);
  if (exec_override >= 0) {
    r.execution_ms = exec_override;
  } else {
    r.execution_ms = lv.exec_started ? ms_between(lv.t_exec, now) : r.latency_ms;
  }
  total_ops_++;
  sum_latency_ += r.latency_ms;
  sum_sync_ += r.sync_ms;
  sum_net_ += r.network_ms;
  sum_reduce_ += r.reduce_ms;
  sum_queue_ += r.queue_wait_ms;
  sum_exec_ += r.execution_ms;
  if (r.execution_ms > 0 && r.bytes > 0) {
    double gbps = (static_cast<double>(r.bytes) * 8.0) / (r.execution_ms * 1e6);
    peak_gbps_ = std::max(peak_gbps_, gbps);
  }
  history_.push_back(r);
  if (history_.size() > kHistoryCap) history_.pop_front();
}

void Metrics::op_end(uint32_t seq) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = live_.find(seq);
  if (it == live_.end()) return;
  finish_locked(it->second, -1.0);
  live_.erase(it);
}

void Metrics::op_end_timed(uint32_t seq, double execution_ms) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = live_.find(seq);
  if (it == live_.end()) return;
  finish_locked(it->second, execution_ms);
  live_.erase(it);
}

void Metrics::op_end_untimed(uint32_t seq) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = live_.find(seq);
  if (it == live_.end()) return;
  untimed_ops_++;
  live_.erase(it);
}

void Metrics::record_transport_bytes(uint64_t sent, uint64_t recv) {
  std::lock_guard<std::mutex> g(mu_);
  bytes_sent_ += sent;
  bytes_recv_ += recv;
}

void Metrics::record_error() {
  std::lock_guard<std::mutex> g(mu_);
  errors_++;
}

Metrics::Summary Metrics::summarize() const {
  std::lock_guard<std::mutex> g(mu_);
  Summary s;
  s.total_ops = total_ops_ + untimed_ops_;
  s.total_bytes_sent = bytes_sent_;
  s.total_bytes_recv = bytes_recv_;
  s.total_errors = errors_;
  s.peak_throughput_gbps = peak_gbps_;
  if (total_ops_ > 0) {
    double n = static_cast<double>(total_ops_);
    s.avg_latency_ms = sum_latency_ / n;
    s.avg_sync_ms = sum_sync_ / n;
    s.avg_network_ms = sum_net_ / n;
    s.avg_reduce_ms = sum_reduce_ / n;
    s.avg_queue_wait_ms = sum_queue_ / n;
    s.avg_execution_ms = sum_exec_ / n;
  }
  if (!history_.empty()) {
    std::vector<double> lat;
    lat.reserve(history_.size());
    for (auto& r : history_) lat.push_back(r.latency_ms);
    std::sort(lat.begin(), lat.end());
    auto pick = [&](double q) {
      size_t i = static_cast<size_t>(q * (lat.size() - 1) + 0.5);
      return lat[std::min(i, lat.size() - 1)];
    };
    s.p50_latency_ms = pick(0.50);
    s.p99_latency_ms = pick(0.99);
  }
  return s;
}

std::vector<Metrics::OpRecord> Metrics::recent_ops(size_t n) const {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<OpRecord> out;
  size_t start = history_.size() > n ? history_.size() - n : 0;
  for (size_t i = start; i < history_.size(); ++i) out.push_back(history_[i]);
  return out;
}

void Metrics::log_summary() const {
  Summary s = summarize();
  MCCL_INFO(
      "metrics: ops=%llu sent=%lluB recv=%lluB errors=%llu lat(avg/p50/p99)=%.3f/%.3f/%.3f ms "
      "peak=%.2f Gbps phases(sync/net/reduce)=%.3f/%.3f/%.3f ms queue=%.3f ms exec=%.3f ms",
      (unsigned long long)s.total_ops, (unsigned long long)s.total_bytes_sent,
      (unsigned long long)s.total_bytes_recv, (unsigned long long)s.total_errors,
      s.avg_latency_ms, s.p50_latency_ms, s.p99_latency_ms, s.peak_throughput_gbps,
      s.avg_sync_ms, s.avg_network_ms, s.avg_reduce_ms, s.avg_queue_wait_ms,
      s.avg_execution_ms);
}

void Metrics::reset() {
  std::lock_guard<std::mutex> g(mu_);
  history_.clear();
  total_ops_ = untimed_ops_ = bytes_sent_ = bytes_recv_ = errors_ = 0;
  peak_gbps_ = 0;
  sum_latency_ = sum_sync_ = sum_net_ = sum_reduce_ = sum_queue_ = sum_exec_ = 0;
}

}  // namespace mccl
