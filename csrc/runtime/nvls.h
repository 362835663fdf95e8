// NvlsRegion: per-process-group device buffers bound to an NVLink multicast object (NVLS).
//
// Every rank allocates the same amount of physical device memory with the virtual-memory API,
// all ranks bind theirs at offset 0 of ONE multicast object created by rank 0, and every rank maps
// both its own memory (`uc()`: plain accesses, local only) and the multicast object (`mc()`):
// a `multimem.st` on an mc address writes every rank's copy through the NVSwitch, a
// `multimem.ld_reduce` returns the sum over all copies, added inside the switch.  The kernels
// that use it are in kernels/nvls.cu and the byte movers of kernels/collectives.cu; signal pads
// and the point-to-point kernels stay on the cudaIpc arena (runtime/arena.h).
//
// Set-up is collective and never throws on an unsupported system: every step is followed by an
// agreement round through the caller's exchange function, and one failure anywhere makes every
// rank release what it holds and return nullptr with the reason (the group then keeps using the
// peer-memory kernels).  The multicast handle travels from rank 0 to the peers as a POSIX file
// descriptor over abstract-namespace Unix datagram sockets (SCM_RIGHTS); driver entry points are
// resolved at run time through the CUDA runtime, so the library has no link-time dependency on
// libcuda and loads on machines without a driver.
//
// Tear-down order matters on NVLink: a rank must not release memory that is still bound while
// peers may issue multicast accesses.  `release()` unmaps and unbinds explicitly; the process group
// calls it after all ranks have drained their streams and met at a host-side rendezvous.
//
// The reference has no counterpart (its bandwidth path is a TCP ring,
// reference csrc/backend/ProcessGroupMCCL.cpp:1712-1959).
#pragma once

#include <cstddef>
#include <functional>
#include <memory>
#include <string>
#include <vector>

namespace mccl {

class NvlsRegion {
 public:
  // All-gather of one small string per rank, keyed by `tag` (a c10d Store exchange in practice).
  using Exchange = std::function<std::vector<std::string>(const std::string& tag, const std::string& mine)>;

  // Collective.  `buffer_bytes` per buffer, `nbuffers` buffers per rank; the current CUDA device is
  // used.  Returns nullptr and fills `why` when NVLS is unavailable or any rank failed.
  // `tag`: distinguishes several regions created through the same exchange (it prefixes the keys).
  static std::unique_ptr<NvlsRegion> create(int rank, int world_size, size_t buffer_bytes, int nbuffers,
                                            const std::string& tag, const Exchange& exchange, std::string* why);
  // Cheap local test: does this device report multicast support (and can the entry points be resolved)?
  static bool device_supported(std::string* why);

  ~NvlsRegion();
  void release();  // idempotent; unmap + unbind + free
  // Ends the multicast side only (unmap the multicast alias, unbind, drop the object) and keeps this
  // rank's own memory mapped: for regions that hold tensors which may outlive the process group.
  void release_multicast_keep_memory();
  size_t total_bytes() const;

  char* uc() const { return uc_; }
  char* mc() const { return mc_; }
  size_t buffer_bytes() const { return buffer_bytes_; }
  int nbuffers() const { return nbuffers_; }
  size_t buffer_offset(unsigned epoch) const { return static_cast<size_t>(epoch % nbuffers_) * buffer_bytes_; }

 private:
  NvlsRegion() = default;
  struct Impl;
  std::unique_ptr<Impl> impl_;
  char* uc_ = nullptr;
  char* mc_ = nullptr;
  size_t buffer_bytes_ = 0;
  int nbuffers_ = 0;
};

}  // namespace mccl
