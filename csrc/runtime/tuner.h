// Tuner: picks the kernel variant for a collective from a size table.
//
// The decision replaces the reference's fixed small-message threshold and ring
// selection (reference csrc/transport/TcpTransport.hpp:28,
// csrc/backend/ProcessGroupMCCL.cpp:1961-1979).  The table holds, per world
// size, the largest payload for which the one-shot allreduce is faster than the
// two-shot one, the CTA counts for both regimes and the two-shot segment size.
// Defaults come from a bus-bandwidth sweep on 8x B200 (NVSwitch); `load()` reads
// overrides written by the sweep tool (`python -m mccl_b200.bench.busbw --tune FILE`)
// as a flat JSON object of integer fields, e.g.
//   {"ws8_oneshot_max_bytes": 524288, "ws8_ctas_large": 64, "segment_bytes": 67108864}
// The path comes from MCCL_TUNE_FILE.  Every rank must load the same file: the
// choice has to be identical on all ranks.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <sstream>
#include <string>

#include "kernels/api.h"

namespace mccl {

enum class Variant : int { ONESHOT = 0, TWOSHOT = 1 };

class Tuner {
 public:
  Tuner() {
    for (int ws = 0; ws <= kern::kMaxWorld; ++ws) {
      // one-shot moves (ws-1)*N per GPU instead of 2*(ws-1)/ws*N: its advantage
      // (one flag round instead of two) holds up to a few hundred KiB.
      // Measured crossovers (fp32, back-to-back calls): with 2 ranks both variants move N per
      // direction, so the single flag round of one-shot wins up to 32 MiB (85 us vs 89 us; at 64 MiB
      // its extra HBM pass costs more: 160 us vs 153 us).
      oneshot_max_[ws] = ws <= 2 ? (size_t(32) << 20) : ws <= 4 ? (size_t(4) << 20) : (size_t(1) << 20);
      ctas_small_[ws] = 32;
      ctas_large_[ws] = 64;  // two lanes may run at once: 2 x 64 CTAs stay below the 148 SMs
      // measured on 2 ranks: 64 MiB 158 us pushed vs 185 us pulled (the stores overlap the reduction)
      push_gather_[ws] = ws <= 2 ? 1 : 0;
      // Gradient buckets run while backward GEMMs need the SMs.  Measured on 2 ranks (94 M MLP, DDP):
      // 73.7 k samples/s with 48 CTAs per allreduce, 71.1 k with 32, 71.2 k with 24, 67.3 k with 16,
      // 66.6 k with 64.  0 = same as ctas_large.
      ctas_overlap_[ws] = ws <= 2 ? 48 : 0;
    }
  }

  Variant choose_allreduce(int ws, size_t bytes) const {
    if (ws < 0 || ws > kern::kMaxWorld) ws = kern::kMaxWorld;
    return bytes <= oneshot_max_[ws] ? Variant::ONESHOT : Variant::TWOSHOT;
  }
  size_t oneshot_max_bytes(int ws) const { return oneshot_max_[ws]; }
  void set_oneshot_max_bytes(int ws, size_t v) { oneshot_max_[ws] = v; }
  // Two-shot allreduce: owners push the reduced chunks (true) or peers pull them (false).
  bool push_gather(int ws) const { return push_gather_[ws < 0 || ws > kern::kMaxWorld ? kern::kMaxWorld : ws] != 0; }
  void set_push_gather(int ws, bool v) { push_gather_[ws] = v ? 1 : 0; }
  size_t segment_bytes() const { return segment_bytes_; }
  void set_segment_bytes(size_t v) { segment_bytes_ = v; }
  // `pushed_bytes`: what one rank sends over the links for this launch.
  // `overlapped`: the collective is a gradient bucket issued from a DDP hook, i.e. it shares the
  // GPU with the rest of backward.
  int ctas_for(int ws, size_t pushed_bytes, int requested, bool overlapped = false) const {
    if (requested > 0) return requested;
    const int cap = overlapped && ctas_overlap_[ws] > 0 ? ctas_overlap_[ws] : ctas_large_[ws];
    return kern::pick_ctas(pushed_bytes, ws, cap);
  }
  void set_ctas(int ws, int small, int large) {
    if (small > 0) ctas_small_[ws] = small;
    if (large > 0) ctas_large_[ws] = large;
  }

  // Returns the number of fields applied (0 if the file is missing or empty).
  int load(const std::string& path) {
    std::ifstream f(path);
    if (!f) return 0;
    std::stringstream ss;
    ss << f.rdbuf();
    const std::string s = ss.str();
    int applied = 0;
    for (int ws = 2; ws <= kern::kMaxWorld; ++ws) {
      long long v;
      const std::string p = "ws" + std::to_string(ws) + "_";
      if (find_int(s, p + "oneshot_max_bytes", v) && v >= 0) { oneshot_max_[ws] = static_cast<size_t>(v); ++applied; }
      if (find_int(s, p + "ctas_small", v) && v > 0) { ctas_small_[ws] = static_cast<int>(v); ++applied; }
      if (find_int(s, p + "ctas_large", v) && v > 0) { ctas_large_[ws] = static_cast<int>(v); ++applied; }
      if (find_int(s, p + "push_gather", v) && v >= 0) { push_gather_[ws] = v ? 1 : 0; ++applied; }
      if (find_int(s, p + "ctas_overlap", v) && v >= 0) { ctas_overlap_[ws] = static_cast<int>(v); ++applied; }
    }
    long long v;
    if (find_int(s, "segment_bytes", v) && v >= (1 << 20)) { segment_bytes_ = static_cast<size_t>(v); ++applied; }
    return applied;
  }

  std::string dump() const {
    std::ostringstream o;
    o << "{";
    for (int ws = 2; ws <= kern::kMaxWorld; ++ws) {
      o << "\"ws" << ws << "_oneshot_max_bytes\": " << oneshot_max_[ws] << ", ";
      o << "\"ws" << ws << "_ctas_small\": " << ctas_small_[ws] << ", ";
      o << "\"ws" << ws << "_ctas_large\": " << ctas_large_[ws] << ", ";
      o << "\"ws" << ws << "_push_gather\": " << push_gather_[ws] << ", ";
      o << "\"ws" << ws << "_ctas_overlap\": " << ctas_overlap_[ws] << ", ";
    }
    o << "\"segment_bytes\": " << segment_bytes_ << "}";
    return o.str();
  }

 private:
  static bool find_int(const std::string& s, const std::string& key, long long& out) {
    const std::string k = "\"" + key + "\"";
    size_t p = s.find(k);
    if (p == std::string::npos) return false;
    p = s.find(':', p + k.size());
    if (p == std::string::npos) return false;
    char* end = nullptr;
    const char* b = s.c_str() + p + 1;
    long long v = std::strtoll(b, &end, 10);
    if (end == b) return false;
    out = v;
    return true;
  }

  size_t oneshot_max_[kern::kMaxWorld + 1];
  int ctas_small_[kern::kMaxWorld + 1];
  int ctas_large_[kern::kMaxWorld + 1];
  int push_gather_[kern::kMaxWorld + 1];
  int ctas_overlap_[kern::kMaxWorld + 1];
  size_t segment_bytes_ = size_t(64) << 20;
};

}  // namespace mccl
