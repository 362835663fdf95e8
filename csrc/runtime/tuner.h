// Tuner: picks the kernel variant and launch shape of a collective from measured tables.
//
// The decision replaces the reference's fixed small-message threshold and ring selection
// (reference csrc/transport/TcpTransport.hpp:28, csrc/backend/ProcessGroupMCCL.cpp:1961-1979).
// Tables are indexed by world size and, where the crossover depends on it, by the element class
// of the wire type (32-bit and wider / 16-bit).  Per world size they hold
//   allreduce      largest payload for the one-shot kernel, smallest payload for the NVLS kernel
//                  (in-switch reduction), two-shot second half pushed or pulled
//   allgather      smallest per-rank block moved with multimem.st instead of one store per peer
//   broadcast      same for the root's payload
//   all of them    CTA caps (alone / as a gradient bucket that shares the GPU with backward),
//                  segment size, pipeline tile sizes
// Defaults come from bus-bandwidth sweeps on 2, 4 and 8 B200s behind an NVSwitch.  `load()` reads
// overrides written by the sweep tool (`python -m mccl_b200.bench.busbw --tune FILE`) as a flat
// JSON object of integer fields, e.g.
//   {"ws8_oneshot_max_bytes": 524288, "ws8_nvls_min_bytes": 2097152, "segment_bytes": 67108864}
// The path comes from MCCL_TUNE_FILE.  Every rank must load the same file: the choice has to be
// identical on all ranks.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <sstream>
#include <string>

#include "kernels/api.h"

namespace mccl {

enum class Variant : int { ONESHOT = 0, TWOSHOT = 1, NVLS = 2 };

inline const char* variant_name(Variant v) {
  return v == Variant::ONESHOT ? "oneshot" : v == Variant::TWOSHOT ? "twoshot" : "nvls";
}

class Tuner {
 public:
  static constexpr int64_t kNever = -1;

  Tuner() {
    for (int ws = 0; ws <= kern::kMaxWorld; ++ws) {
      for (int cls = 0; cls < 2; ++cls) {
        // one-shot moves (ws-1)*N per GPU instead of 2*(ws-1)/ws*N: its advantage (one flag round
        // instead of two) holds up to a few hundred KiB.  With 2 ranks both variants move N per
        // direction, so one-shot wins up to 32 MiB (85 us vs 89 us; at 64 MiB its extra HBM pass
        // costs more: 160 us vs 153 us).
        oneshot_max_[ws][cls] = ws <= 2 ? (int64_t(32) << 20) : ws <= 4 ? (int64_t(4) << 20) : (int64_t(1) << 20);
        // NVLS moves (1 + 1/ws) * N per direction instead of 2 (ws-1)/ws * N: no gain at 2 ranks,
        // 1.2x at 4 and 1.55x at 8, and it pays two local staging passes.  Measured on 4 ranks: equal to
        // the two-shot kernel within noise from 16 MiB to 1 GiB (231 vs 235 us at 64 MiB), so it is only
        // used from 5 ranks on, above the one-shot range.
        nvls_min_[ws][cls] = ws <= 4 ? kNever : (int64_t(1) << 20) + 1;
      }
      // multimem.st also delivers a copy back to the sender, which costs 1/ws of the ingress.  Measured on
      // 4 ranks: for allgather (every rank sends) the plain peer stores win from 8 MiB up (256 MiB: 367 vs
      // 474 us) and the two are within 2 us below; for broadcast (one sender, and one hop instead of two)
      // multimem.st wins at every size from 16 KiB to 256 MiB (515 vs 662 us at 256 MiB).
      ag_nvls_min_[ws] = kNever;
      bc_nvls_min_[ws] = ws <= 2 ? kNever : (int64_t(16) << 10);
      // Measured on 8 ranks: multimem.st wins up to 8 MiB (1 MiB: 17.6 vs 29.2 us, 8 MiB: 36.7 vs 43.2 us)
      // and loses from 16 MiB up (64 MiB: 186 vs 161 us): one sender's multicast stores run near
      // 385 GB/s there, below what the two-hop peer stores reach.  No ceiling at 3-4 ranks.
      bc_nvls_max_[ws] = ws >= 5 ? (int64_t(8) << 20) : kNever;
      ctas_small_[ws] = 32;
      ctas_large_[ws] = kern::kMaxCtasPerLane;  // two lanes may run at once: 2 x 64 CTAs stay below the 148 SMs
      // measured: 2 ranks 64 MiB 158 us pushed vs 185 us pulled (the stores overlap the reduction);
      // 4 ranks 217 vs 234 us (32 MiB: 121 vs 133 us); 8 ranks 247 vs 255 us (32 MiB: 137 vs 145 us)
      push_gather_[ws] = 1;
      // Gradient buckets run while backward GEMMs need the SMs.  Measured on 2 ranks (94 M MLP, DDP):
      // 73.7 k samples/s with 48 CTAs per allreduce, 71.1 k with 32, 71.2 k with 24, 67.3 k with 16,
      // 66.6 k with 64.  0 = same as ctas_large.
      ctas_overlap_[ws] = ws <= 2 ? 48 : 0;
    }
  }

  // `cls`: 0 for 32-bit and wider wire elements, 1 for 16-bit ones.  `nvls_ok`: the group has an
  // NVLS region and the (dtype, op) pair is one the in-switch reduction supports.
  Variant choose_allreduce(int ws, size_t bytes, int cls = 0, bool nvls_ok = false) const {
    ws = clamp_ws(ws);
    cls = cls ? 1 : 0;
    if (static_cast<int64_t>(bytes) <= oneshot_max_[ws][cls]) return Variant::ONESHOT;
    if (nvls_ok && nvls_min_[ws][cls] >= 0 && static_cast<int64_t>(bytes) >= nvls_min_[ws][cls]) return Variant::NVLS;
    return Variant::TWOSHOT;
  }
  bool allgather_nvls(int ws, size_t bytes_per_rank) const {
    ws = clamp_ws(ws);
    return ag_nvls_min_[ws] >= 0 && static_cast<int64_t>(bytes_per_rank) >= ag_nvls_min_[ws];
  }
  bool broadcast_nvls(int ws, size_t bytes) const {
    ws = clamp_ws(ws);
    return bc_nvls_min_[ws] >= 0 && static_cast<int64_t>(bytes) >= bc_nvls_min_[ws] &&
           (bc_nvls_max_[ws] < 0 || static_cast<int64_t>(bytes) <= bc_nvls_max_[ws]);
  }
  size_t oneshot_max_bytes(int ws, int cls = 0) const { return static_cast<size_t>(oneshot_max_[clamp_ws(ws)][cls ? 1 : 0]); }
  void set_oneshot_max_bytes(int ws, size_t v) { oneshot_max_[ws][0] = oneshot_max_[ws][1] = static_cast<int64_t>(v); }
  int64_t nvls_min_bytes(int ws, int cls = 0) const { return nvls_min_[clamp_ws(ws)][cls ? 1 : 0]; }
  void set_nvls_min_bytes(int ws, int64_t v) { nvls_min_[ws][0] = nvls_min_[ws][1] = v; }
  // Two-shot allreduce: owners push the reduced chunks (true) or peers pull them (false).
  bool push_gather(int ws) const { return push_gather_[clamp_ws(ws)] != 0; }
  void set_push_gather(int ws, bool v) { push_gather_[ws] = v ? 1 : 0; }
  size_t segment_bytes() const { return segment_bytes_; }
  void set_segment_bytes(size_t v) { segment_bytes_ = v; }
  // NVLS allreduce: from this payload on, the staging passes run as separate full-grid kernels
  int64_t nvls_split_min_bytes() const { return nvls_split_min_bytes_; }
  void set_nvls_split_min_bytes(int64_t v) { nvls_split_min_bytes_ = v; }
  int mover_tile_bytes() const { return mover_tile_bytes_; }
  int nvls_tile_bytes() const { return nvls_tile_bytes_; }
  // `pushed_bytes`: what one rank sends over the links for this launch.
  // `overlapped`: the collective is a gradient bucket issued from a DDP hook, i.e. it shares the
  // GPU with the rest of backward.
  int ctas_for(int ws, size_t pushed_bytes, int requested, bool overlapped = false) const {
    ws = clamp_ws(ws);
    if (requested > 0) return requested < kern::kMaxCtasPerLane ? requested : kern::kMaxCtasPerLane;
    const int cap = overlapped && ctas_overlap_[ws] > 0 ? ctas_overlap_[ws] : ctas_large_[ws];
    return kern::pick_ctas(pushed_bytes, ws, cap);
  }
  void set_ctas_overlap(int ws, int v) { ctas_overlap_[ws] = v < kern::kMaxCtasPerLane ? v : kern::kMaxCtasPerLane; }
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
    long long v;
    for (int ws = 2; ws <= kern::kMaxWorld; ++ws) {
      const std::string p = "ws" + std::to_string(ws) + "_";
      if (find_int(s, p + "oneshot_max_bytes", v) && v >= 0) { oneshot_max_[ws][0] = oneshot_max_[ws][1] = v; ++applied; }
      if (find_int(s, p + "oneshot_max_bytes_16bit", v) && v >= 0) { oneshot_max_[ws][1] = v; ++applied; }
      if (find_int(s, p + "nvls_min_bytes", v) && v >= -1) { nvls_min_[ws][0] = nvls_min_[ws][1] = v; ++applied; }
      if (find_int(s, p + "nvls_min_bytes_16bit", v) && v >= -1) { nvls_min_[ws][1] = v; ++applied; }
      if (find_int(s, p + "allgather_nvls_min_bytes", v) && v >= -1) { ag_nvls_min_[ws] = v; ++applied; }
      if (find_int(s, p + "broadcast_nvls_min_bytes", v) && v >= -1) { bc_nvls_min_[ws] = v; ++applied; }
      if (find_int(s, p + "broadcast_nvls_max_bytes", v) && v >= -1) { bc_nvls_max_[ws] = v; ++applied; }
      if (find_int(s, p + "ctas_small", v) && v > 0) { ctas_small_[ws] = static_cast<int>(v); ++applied; }
      if (find_int(s, p + "ctas_large", v) && v > 0) { ctas_large_[ws] = static_cast<int>(std::min<long long>(v, kern::kMaxCtasPerLane)); ++applied; }
      if (find_int(s, p + "push_gather", v) && v >= 0) { push_gather_[ws] = v ? 1 : 0; ++applied; }
      if (find_int(s, p + "ctas_overlap", v) && v >= 0) { ctas_overlap_[ws] = static_cast<int>(std::min<long long>(v, kern::kMaxCtasPerLane)); ++applied; }
    }
    if (find_int(s, "segment_bytes", v) && v >= (1 << 20)) { segment_bytes_ = static_cast<size_t>(v); ++applied; }
    if (find_int(s, "mover_tile_bytes", v) && v >= 0) { mover_tile_bytes_ = static_cast<int>(v); ++applied; }
    if (find_int(s, "nvls_split_min_bytes", v) && v >= -1) { nvls_split_min_bytes_ = v; ++applied; }
    if (find_int(s, "nvls_tile_bytes", v) && v >= 0) { nvls_tile_bytes_ = static_cast<int>(v); ++applied; }
    return applied;
  }

  std::string dump() const {
    std::ostringstream o;
    o << "{";
    for (int ws = 2; ws <= kern::kMaxWorld; ++ws) {
      const std::string p = "\"ws" + std::to_string(ws) + "_";
      o << p << "oneshot_max_bytes\": " << oneshot_max_[ws][0] << ", ";
      o << p << "oneshot_max_bytes_16bit\": " << oneshot_max_[ws][1] << ", ";
      o << p << "nvls_min_bytes\": " << nvls_min_[ws][0] << ", ";
      o << p << "nvls_min_bytes_16bit\": " << nvls_min_[ws][1] << ", ";
      o << p << "allgather_nvls_min_bytes\": " << ag_nvls_min_[ws] << ", ";
      o << p << "broadcast_nvls_min_bytes\": " << bc_nvls_min_[ws] << ", ";
      o << p << "broadcast_nvls_max_bytes\": " << bc_nvls_max_[ws] << ", ";
      o << p << "ctas_small\": " << ctas_small_[ws] << ", ";
      o << p << "ctas_large\": " << ctas_large_[ws] << ", ";
      o << p << "push_gather\": " << push_gather_[ws] << ", ";
      o << p << "ctas_overlap\": " << ctas_overlap_[ws] << ", ";
    }
    o << "\"segment_bytes\": " << segment_bytes_ << ", \"mover_tile_bytes\": " << mover_tile_bytes_
      << ", \"nvls_tile_bytes\": " << nvls_tile_bytes_ << ", \"nvls_split_min_bytes\": " << nvls_split_min_bytes_ << "}";
    return o.str();
  }

 private:
  static int clamp_ws(int ws) { return ws < 0 || ws > kern::kMaxWorld ? kern::kMaxWorld : ws; }
  // Finds `"key": <int>`; the key must be delimited by quotes so that a key that is a prefix of
  // another one does not match it.
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

  int64_t oneshot_max_[kern::kMaxWorld + 1][2];
  int64_t nvls_min_[kern::kMaxWorld + 1][2];
  int64_t ag_nvls_min_[kern::kMaxWorld + 1];
  int64_t bc_nvls_min_[kern::kMaxWorld + 1];
  int64_t bc_nvls_max_[kern::kMaxWorld + 1];  // -1: no ceiling
  int ctas_small_[kern::kMaxWorld + 1];
  int ctas_large_[kern::kMaxWorld + 1];
  int push_gather_[kern::kMaxWorld + 1];
  int ctas_overlap_[kern::kMaxWorld + 1];
  size_t segment_bytes_ = size_t(64) << 20;
  // measured on 2 ranks (64 MiB broadcast: 160 us with 128 KiB tiles, 132 us with 512 KiB, 117 us with
  // 2 MiB; 16 MiB allgather: 34 / 35 / 49 us): every tile costs a system-scope fence on the sender
  int mover_tile_bytes_ = 1 << 20;
  int nvls_tile_bytes_ = 0;  // 0: kernel default
  int64_t nvls_split_min_bytes_ = int64_t(8) << 20;
};

}  // namespace mccl
