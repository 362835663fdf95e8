// Reusable host staging buffers.
//
// `acquire(n)` returns the smallest free buffer that holds n bytes (best fit);
// if none fits, a new one is allocated with 25 % head-room (the head-room is
// capped at 256 MiB) so that slightly larger follow-up requests reuse it.
// Buffers return to the pool when their PooledBuffer handle dies.  `trim()`
// frees every idle buffer; `total_allocated()` reports bytes held (idle and in
// use).  The process-wide `staging_memory_pool()` backs the host transport's
// receive scratch and the CPU collectives' temporaries; its buffers are page
// aligned (4 KiB) so they can be pinned for asynchronous device copies.
// Parity: reference csrc/runtime/MemoryPool.hpp:16-79, MemoryPool.cpp:20-126.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <map>
#include <mutex>

namespace mccl {

class MemoryPool;

class PooledBuffer {
 public:
  PooledBuffer() = default;
  PooledBuffer(MemoryPool* pool, void* p, size_t cap) : pool_(pool), ptr_(p), cap_(cap) {}
  PooledBuffer(const PooledBuffer&) = delete;
  PooledBuffer& operator=(const PooledBuffer&) = delete;
  PooledBuffer(PooledBuffer&& o) noexcept { swap(o); }
  PooledBuffer& operator=(PooledBuffer&& o) noexcept {
    if (this != &o) {
      release();
      swap(o);
    }
    return *this;
  }
  ~PooledBuffer() { release(); }

  void* data() const { return ptr_; }
  template <typename T> T* as() const { return static_cast<T*>(ptr_); }
  size_t capacity() const { return cap_; }
  explicit operator bool() const { return ptr_ != nullptr; }
  void release();

 private:
  void swap(PooledBuffer& o) {
    std::swap(pool_, o.pool_);
    std::swap(ptr_, o.ptr_);
    std::swap(cap_, o.cap_);
  }
  MemoryPool* pool_ = nullptr;
  void* ptr_ = nullptr;
  size_t cap_ = 0;
};

class MemoryPool {
 public:
  explicit MemoryPool(size_t alignment = 4096) : align_(alignment) {}
  ~MemoryPool() { trim(); }

  PooledBuffer acquire(size_t nbytes) {
    if (nbytes == 0) nbytes = 1;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = free_.lower_bound(nbytes);  // best fit: smallest capacity >= nbytes
      if (it != free_.end()) {
        void* p = it->second;
        size_t cap = it->first;
        free_.erase(it);
        in_use_ += cap;
        return PooledBuffer(this, p, cap);
      }
    }
    size_t extra = nbytes / 4;
    const size_t kMaxExtra = size_t(256) << 20;
    if (extra > kMaxExtra) extra = kMaxExtra;
    size_t cap = round_up(nbytes + extra);
    void* p = nullptr;
    if (posix_memalign(&p, align_, cap) != 0 || !p) {
      cap = round_up(nbytes);
      if (posix_memalign(&p, align_, cap) != 0 || !p) throw std::bad_alloc();
    }
    std::lock_guard<std::mutex> g(mu_);
    total_ += cap;
    in_use_ += cap;
    return PooledBuffer(this, p, cap);
  }

  void give_back(void* p, size_t cap) {
    std::lock_guard<std::mutex> g(mu_);
    in_use_ -= cap;
    free_.emplace(cap, p);
  }

  // Frees idle buffers; buffers currently handed out are untouched.
  void trim() {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& kv : free_) {
      std::free(kv.second);
      total_ -= kv.first;
    }
    free_.clear();
  }

  size_t total_allocated() const {
    std::lock_guard<std::mutex> g(mu_);
    return total_;
  }
  size_t bytes_in_use() const {
    std::lock_guard<std::mutex> g(mu_);
    return in_use_;
  }
  size_t idle_buffers() const {
    std::lock_guard<std::mutex> g(mu_);
    return free_.size();
  }

 private:
  size_t round_up(size_t n) const { return (n + align_ - 1) / align_ * align_; }
  size_t align_;
  mutable std::mutex mu_;
  std::multimap<size_t, void*> free_;
  size_t total_ = 0;
  size_t in_use_ = 0;
};

inline void PooledBuffer::release() {
  if (pool_ && ptr_) pool_->give_back(ptr_, cap_);
  pool_ = nullptr;
  ptr_ = nullptr;
  cap_ = 0;
}

inline MemoryPool& staging_memory_pool() {
  static MemoryPool* pool = new MemoryPool(4096);  // leaked on purpose: outlives static dtors
  return *pool;
}

}  // namespace mccl
