// Process-wide count of kernel launches issued by this library's launchers
// (used by benchmarks to report how many native kernels ran in a timed region).
#pragma once

#include <atomic>
#include <cstdint>

namespace mccl {
namespace kern {

inline std::atomic<uint64_t>& launch_counter() {
  static std::atomic<uint64_t> c{0};
  return c;
}
inline void note_launch(uint64_t n = 1) { launch_counter().fetch_add(n, std::memory_order_relaxed); }

}  // namespace kern
}  // namespace mccl
