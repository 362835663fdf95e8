// SymmetricArena: the per-process-group block of device memory that peers write
// into and read from directly over NVLink.
//
// Every rank allocates  [signal pad | data buffer 0..3]  with
// cudaMalloc (outside torch's caching allocator, so the allocation is a whole
// IPC-exportable block), zeroes the signal pad, publishes a
// cudaIpcMemHandle through the c10d Store and maps every peer's block with
// cudaIpcOpenMemHandle (which also enables peer access).  Ranks must share a
// host and be P2P-capable; `open_peers` reports failure instead of throwing so
// the process group can agree, collectively, to fall back to host staging.
//
// Collectives take consecutive epochs; epoch e runs in lane e % 2 (one stream
// per lane, so two consecutive collectives overlap) and uses data buffer e % 4.
// The credit protocol in the kernels (enter_collective) guarantees that epoch e
// never touches a buffer a peer may still be using for epoch e-4, so no trailing
// barrier is needed and flags are never reset.
//
// An emulation constructor builds `ws` arenas on ONE device for single-GPU
// tests: the same kernels then run as one cooperative launch with grid.y = ws.
//
// This is the B200 replacement for the reference's host staging buffers and
// blit copies (reference csrc/metal/MPSInterop.mm:53-230,511-685).
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>
#include <string>
#include <vector>

#include "kernels/api.h"

namespace mccl {

class SymmetricArena {
 public:
  // Real arena of this rank on the current device.
  SymmetricArena(int rank, int world_size, size_t parity_bytes);
  // Emulated: all `world_size` arenas on the current device.
  static SymmetricArena* make_emulated(int world_size, size_t parity_bytes);
  ~SymmetricArena();

  // Opaque bytes to publish to peers (IPC handle + identity).
  std::string export_handle() const;
  // handles[r] from every rank.  Returns "" on success or the reason it failed.
  std::string open_peers(const std::vector<std::string>& handles);

  int rank() const { return rank_; }
  int world_size() const { return ws_; }
  size_t parity_bytes() const { return parity_bytes_; }
  bool emulated() const { return emulated_; }
  bool ready() const { return ready_; }

  // Takes the next epoch and fills the arena part of `p` for local rank
  // (real) or all ranks (emulated).  in/out pointers are left to the caller.
  uint32_t next_epoch() { return ++epoch_; }
  uint32_t epoch() const { return epoch_; }
  void fill_params(kern::CollParams& p, uint32_t epoch) const;

  uint32_t* status_device(int r = 0) const { return status_[emulated_ ? r : 0]; }
  // Copies the status block of rank r out (synchronous on `stream`).
  void read_status(uint32_t out[kern::kStatusWords], cudaStream_t stream, int r = 0) const;
  void clear_status(cudaStream_t stream);
  // True once a kernel of this (real, non-emulated) arena has recorded a failure.  Reads a
  // host-mapped mirror of the status block: no stream, no synchronisation, callable from any thread.
  bool device_failed() const { return status_host_ != nullptr && status_host_[0] != 0u; }
  // Phase-stamp capture (off by default): fill_params passes the buffer to the kernels.
  void enable_stamps(bool on);
  // Stamps of arena epoch `epoch` (default: the latest one).  The stamps live in host-mapped memory,
  // one slot per epoch in a ring of kStampRing; the caller makes sure the kernel has finished.
  void read_stamps(unsigned long long out[kern::kStampSlots], cudaStream_t stream, int r = 0,
                   int64_t epoch = -1) const;
  bool stamps_enabled() const { return stamps_on_; }
  static constexpr int kStampRing = 64;
  char* base(int r) const { return bases_[r]; }

 private:
  SymmetricArena() = default;
  int rank_ = 0, ws_ = 1;
  size_t parity_bytes_ = 0;
  size_t total_bytes_ = 0;
  bool emulated_ = false;
  bool ready_ = false;
  int device_ = 0;
  uint32_t epoch_ = 0;
  std::vector<char*> bases_;       // [ws]; bases_[rank_] is the local allocation
  std::vector<bool> opened_;       // peers mapped through IPC (to close)
  std::vector<uint32_t*> status_;  // device status blocks (1 real, ws emulated)
  volatile uint32_t* status_host_ = nullptr;  // pinned, device-mapped mirror of status_[0][0..3] (real arenas)
  std::vector<unsigned long long*> stamps_;      // host addresses of the pinned stamp rings
  std::vector<unsigned long long*> stamps_dev_;  // the same memory as the device sees it
  bool stamps_on_ = false;
};

}  // namespace mccl
