// Cross-GPU signalling primitives: release stores to a peer's signal pad,
// acquire polls of the local pad, and the bounded wait every kernel uses.
//
// Protocol.  A producer CTA finishes its payload stores (to local or peer
// memory), executes __syncthreads(), and then ONE thread per destination does
// fence.acq_rel.sys + st.release.sys of the epoch into the destination's flag.
// A consumer thread polls the flag in its own arena with ld.acquire.sys until
// the epoch appears, then the CTA executes __syncthreads() before touching the
// payload.  Flags are compared with wrap-safe signed arithmetic.
//
// No wait is unbounded: after `wait_ns` nanoseconds of polling the waiter
// records {code, seq, phase, peer} in the status block and returns false; the
// calling kernel then skips its remaining phases and exits normally, leaving the
// context usable.  The status block lives in device memory; the host copies it
// out on a side stream (watchdog poll, Work::wait) and fails the collective.
#pragma once

#include <cstdint>

#include "kernels/api.h"

namespace mccl {
namespace kern {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool epoch_reached(uint32_t seen, uint32_t want) {
  return static_cast<int32_t>(seen - want) >= 0;
}

// Signal values are (epoch << 12) + count: pipelined kernels publish a running
// tile count inside one epoch, plain kernels publish kSigDone.  Values grow
// monotonically across epochs (4095 tiles per CTA per epoch at most).
constexpr uint32_t kSigDone = 4095;
__device__ __forceinline__ uint32_t sig_value(uint32_t seq, uint32_t count) { return (seq << 12) + count; }

__device__ __forceinline__ int lane_of(uint32_t seq) { return static_cast<int>(seq & (kNumLanes - 1)); }
__device__ __forceinline__ uint32_t* entered_flag(char* arena, int lane, int src) {
  return reinterpret_cast<uint32_t*>(arena + kEnteredOffset) + lane * kMaxWorld + src;
}
__device__ __forceinline__ uint32_t* sig_flag(char* arena, int lane, int phase, int cta, int src) {
  return reinterpret_cast<uint32_t*>(arena + kSigOffset) +
         ((static_cast<size_t>(lane) * kNumPhases + phase) * kMaxCtas + cta) * kMaxWorld + src;
}

__device__ __forceinline__ void report_failure(uint32_t* status, uint32_t code, uint32_t seq,
                                               uint32_t phase, uint32_t peer) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0u, code) == 0u) {
    status[1] = seq;
    status[2] = phase;
    status[3] = peer;
    __threadfence();
    // Words 4-5 hold the device address of a host-mapped mirror (0: none).  The first failure is
    // copied there with plain stores, code last, so the host can see it without touching a stream.
    const unsigned long long mirror = *reinterpret_cast<const unsigned long long*>(status + kStatusMirrorWord);
    if (mirror != 0ull) {
      volatile uint32_t* h = reinterpret_cast<volatile uint32_t*>(mirror);
      h[1] = seq;
      h[2] = phase;
      h[3] = peer;
      __threadfence_system();
      h[0] = code;
      __threadfence_system();
    }
  }
}

// Polls `flag` (local arena) until it reaches `want`.  Returns false on timeout.
__device__ __forceinline__ bool wait_epoch(const uint32_t* flag, uint32_t want,
                                           unsigned long long wait_ns, uint32_t* status,
                                           uint32_t phase, uint32_t peer) {
  if (epoch_reached(ld_acquire_sys(flag), want)) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (epoch_reached(ld_acquire_sys(flag), want)) return true;
    if ((++spins & 0x3FFu) == 0) {
      if (globaltimer_ns() - t0 > wait_ns) {
        report_failure(status, ERR_WAIT_TIMEOUT, want, phase, peer);
        return false;
      }
      // Another CTA already failed: give up quickly so the kernel drains.
      if (status != nullptr && *reinterpret_cast<volatile uint32_t*>(status) != 0u) return false;
    }
    __nanosleep(20);
  }
}

}  // namespace kern
}  // namespace mccl
