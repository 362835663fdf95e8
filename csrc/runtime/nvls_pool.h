// NvlsUserPool: device memory for user tensors that is bound to an NVLink multicast object, so that a
// collective on such a tensor needs no staging at all: the NVLS allreduce reduces it in the switch
// and writes the result back in place (kernels/nvls.cu, nvls_inplace_kernel).
//
// The pool is one NvlsRegion (runtime/nvls.h) per device plus a first-fit free list.  It is handed to
// torch as a pluggable allocator behind a torch.cuda.MemPool: DistributedDataParallel built inside
// `torch.cuda.use_mem_pool(pool)` places its gradient buckets here (mccl_b200.parallel.wrap_ddp does
// that).  Every rank allocates the same sizes in the same order, so a tensor sits at the same offset
// of every rank's region, which is what a multicast address needs; the process group checks the
// offsets across ranks the first time it sees a tensor.  Requests the pool cannot serve fall back to
// cudaMalloc (such tensors simply take the staged path).
//
// The region's own memory is never unmapped while the process lives: tensors may outlive the
// process group.  Only the multicast binding ends with the group.
//
// The reference has no counterpart.
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>
#include <map>
#include <memory>
#include <mutex>
#include <set>

#include "runtime/nvls.h"

namespace mccl {

// First-fit allocator over the offsets [0, size): 512-byte granules, free blocks coalesce on release.
class RangeAllocator {
 public:
  static constexpr size_t kAlign = 512;
  void reset(size_t size) {
    free_.clear();
    used_.clear();
    if (size) free_[0] = size;
  }
  // Offset of a block of at least `bytes`, or -1.
  long long alloc(size_t bytes) {
    if (bytes == 0) return -1;
    const size_t need = (bytes + kAlign - 1) / kAlign * kAlign;
    for (auto it = free_.begin(); it != free_.end(); ++it) {
      if (it->second < need) continue;
      const size_t off = it->first, len = it->second;
      free_.erase(it);
      if (len > need) free_[off + need] = len - need;
      used_[off] = need;
      return static_cast<long long>(off);
    }
    return -1;
  }
  // False if `off` is not the start of a live block.
  bool release(size_t off) {
    auto it = used_.find(off);
    if (it == used_.end()) return false;
    size_t len = it->second, start = off;
    used_.erase(it);
    auto nxt = free_.lower_bound(start);
    if (nxt != free_.end() && nxt->first == start + len) {  // merge with the block behind
      len += nxt->second;
      nxt = free_.erase(nxt);
    }
    if (nxt != free_.begin()) {  // merge with the block in front
      auto prv = std::prev(nxt);
      if (prv->first + prv->second == start) {
        start = prv->first;
        len += prv->second;
        free_.erase(prv);
      }
    }
    free_[start] = len;
    return true;
  }
  size_t bytes_in_use() const {
    size_t n = 0;
    for (auto& kv : used_) n += kv.second;
    return n;
  }
  size_t free_blocks() const { return free_.size(); }

 private:
  std::map<size_t, size_t> free_;  // offset -> length, coalesced
  std::map<size_t, size_t> used_;  // offset -> length
};

class NvlsUserPool {
 public:
  static NvlsUserPool& get(int device);

  // Takes ownership of a freshly created single-buffer region.  False if the device already has one.
  bool attach(std::unique_ptr<NvlsRegion> region);
  bool active() const { return region_ != nullptr && region_->mc() != nullptr; }
  void end_multicast();  // the owning process group shuts down

  void* alloc(size_t bytes);     // nullptr: no room (or no region)
  bool release(void* p);         // true if p came from this pool
  bool contains(const void* p, size_t bytes) const;
  size_t offset_of(const void* p) const { return static_cast<size_t>(static_cast<const char*>(p) - base_); }
  char* uc() const { return base_; }
  char* mc() const { return region_ ? region_->mc() : nullptr; }
  size_t size() const { return size_; }
  size_t bytes_in_use() const;

 private:
  mutable std::mutex mu_;
  std::unique_ptr<NvlsRegion> region_;
  char* base_ = nullptr;
  size_t size_ = 0;
  RangeAllocator ranges_;
};

}  // namespace mccl

extern "C" {
// torch.cuda.memory.CUDAPluggableAllocator entry points.
void* mccl_nvls_pool_alloc(ssize_t size, int device, cudaStream_t stream);
void mccl_nvls_pool_free(void* ptr, size_t size, int device, cudaStream_t stream);
}
