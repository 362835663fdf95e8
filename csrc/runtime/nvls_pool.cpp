#include "runtime/nvls_pool.h"

#include <sys/types.h>

#include "common/log.h"

namespace mccl {

namespace {
constexpr int kMaxDevices = 64;
}  // namespace

NvlsUserPool& NvlsUserPool::get(int device) {
  static NvlsUserPool pools[kMaxDevices];
  return pools[device >= 0 && device < kMaxDevices ? device : 0];
}

bool NvlsUserPool::attach(std::unique_ptr<NvlsRegion> region) {
  std::lock_guard<std::mutex> g(mu_);
  if (region_ || !region) return false;
  base_ = region->uc();
  size_ = region->buffer_bytes() * static_cast<size_t>(region->nbuffers());
  region_ = std::move(region);
  ranges_.reset(size_);
  return true;
}

void NvlsUserPool::end_multicast() {
  std::lock_guard<std::mutex> g(mu_);
  if (region_) region_->release_multicast_keep_memory();
}

void* NvlsUserPool::alloc(size_t bytes) {
  std::lock_guard<std::mutex> g(mu_);
  if (!region_) return nullptr;
  const long long off = ranges_.alloc(bytes);
  return off < 0 ? nullptr : base_ + off;
}

bool NvlsUserPool::release(void* p) {
  std::lock_guard<std::mutex> g(mu_);
  if (!region_ || p < base_ || p >= base_ + size_) return false;
  ranges_.release(static_cast<size_t>(static_cast<char*>(p) - base_));
  return true;  // inside the region: ours, whether or not it was a live block
}

bool NvlsUserPool::contains(const void* p, size_t bytes) const {
  std::lock_guard<std::mutex> g(mu_);
  if (!region_) return false;
  const char* c = static_cast<const char*>(p);
  return c >= base_ && bytes <= size_ && c + bytes <= base_ + size_;
}

size_t NvlsUserPool::bytes_in_use() const {
  std::lock_guard<std::mutex> g(mu_);
  return ranges_.bytes_in_use();
}

}  // namespace mccl

extern "C" __attribute__((visibility("default"))) void* mccl_nvls_pool_alloc(ssize_t size, int device, cudaStream_t) {
  if (size <= 0) return nullptr;
  void* p = mccl::NvlsUserPool::get(device).alloc(static_cast<size_t>(size));
  if (p != nullptr) return p;
  // no multicast-bound room: ordinary device memory (the tensor then takes the staged paths)
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != device) cudaSetDevice(device);
  void* q = nullptr;
  cudaError_t e = cudaMalloc(&q, static_cast<size_t>(size));
  if (prev != device && prev >= 0) cudaSetDevice(prev);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return q;
}

extern "C" __attribute__((visibility("default"))) void mccl_nvls_pool_free(void* ptr, size_t, int device, cudaStream_t) {
  if (ptr == nullptr) return;
  if (mccl::NvlsUserPool::get(device).release(ptr)) return;
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != device) cudaSetDevice(device);
  cudaFree(ptr);
  if (prev != device && prev >= 0) cudaSetDevice(prev);
}
