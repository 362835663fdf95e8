// Environment-variable accessors and the derived collective limits.
//
// All MCCL_* knobs are read when a process group is constructed (the Python
// MCCLConfig mirrors itself into os.environ before that point).
// Parity: reference csrc/common/CollectiveEnv.hpp:10-68 for the derived limits.
#pragma once

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <string>

namespace mccl {

inline std::string env_str(const char* name, const std::string& dflt = "") {
  const char* v = std::getenv(name);
  return (v && *v) ? std::string(v) : dflt;
}

inline int64_t env_int(const char* name, int64_t dflt) {
  const char* v = std::getenv(name);
  if (!v || !*v) return dflt;
  char* end = nullptr;
  long long r = std::strtoll(v, &end, 10);
  if (end == v) return dflt;
  return static_cast<int64_t>(r);
}

inline double env_double(const char* name, double dflt) {
  const char* v = std::getenv(name);
  if (!v || !*v) return dflt;
  char* end = nullptr;
  double r = std::strtod(v, &end);
  if (end == v) return dflt;
  return r;
}

inline bool env_bool(const char* name, bool dflt) {
  const char* v = std::getenv(name);
  if (!v) return dflt;
  std::string s(v);
  if (s.empty()) return dflt;
  return !(s == "0" || s == "false" || s == "FALSE" || s == "no" || s == "NO" ||
           s == "off" || s == "OFF");
}

// Largest single collective payload one arena slot is sized for.
inline int64_t demux_max_collective_bytes() {
  int64_t v = env_int("MCCL_DEMUX_MAX_COLLECTIVE_BYTES", 64ll << 20);
  return std::max<int64_t>(v, 1 << 20);
}

inline int collective_concurrency_max() {
  int64_t v = env_int("MCCL_MAX_COLLECTIVE_CONCURRENCY", 8);
  return static_cast<int>(std::clamp<int64_t>(v, 1, 16));
}

inline int collective_concurrency_requested() {
  int64_t v = env_int("MCCL_COLLECTIVE_CONCURRENCY", 1);
  return static_cast<int>(std::clamp<int64_t>(v, 1, collective_concurrency_max()));
}

inline int64_t demux_inflight_budget_bytes() {
  int64_t v = env_int("MCCL_DEMUX_INFLIGHT_BUDGET_BYTES", 1ll << 30);
  return std::max<int64_t>(v, 1 << 20);
}

// Collectives allowed in flight at once: 1 below three ranks, otherwise the
// request capped by how many maximum-size payloads fit in the in-flight budget.
inline int effective_collective_concurrency(int world_size) {
  if (world_size < 3) return 1;
  int64_t fit = demux_inflight_budget_bytes() / demux_max_collective_bytes();
  fit = std::max<int64_t>(fit, 1);
  return static_cast<int>(std::min<int64_t>(collective_concurrency_requested(), fit));
}

}  // namespace mccl
