#include "runtime/arena.h"

#include <unistd.h>

#include <cstring>

#include "common/errors.h"
#include "common/log.h"

namespace mccl {

namespace {

struct ExportRecord {
  cudaIpcMemHandle_t handle;
  char hostname[64];
  int32_t pid;
  int32_t device;
  uint64_t total_bytes;
};

std::string host_identity() {
  char buf[64];
  std::memset(buf, 0, sizeof(buf));
  gethostname(buf, sizeof(buf) - 1);
  return std::string(buf);
}

}  // namespace

SymmetricArena::SymmetricArena(int rank, int world_size, size_t parity_bytes)
    : rank_(rank), ws_(world_size), parity_bytes_(parity_bytes) {
  MCCL_CHECK(world_size >= 1 && world_size <= kern::kMaxWorld,
             "symmetric arena supports 1.." << kern::kMaxWorld << " ranks, got " << world_size);
  MCCL_CUDA_CHECK(cudaGetDevice(&device_));
  total_bytes_ = kern::kSignalBytes + kern::kNumParity * parity_bytes_;
  bases_.assign(ws_, nullptr);
  opened_.assign(ws_, false);
  void* p = nullptr;
  MCCL_CUDA_CHECK(cudaMalloc(&p, total_bytes_));
  bases_[rank_] = static_cast<char*>(p);
  MCCL_CUDA_CHECK(cudaMemset(p, 0, kern::kSignalBytes));
  uint32_t* st = nullptr;
  MCCL_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&st), kern::kStatusWords * sizeof(uint32_t)));
  MCCL_CUDA_CHECK(cudaMemset(st, 0, kern::kStatusWords * sizeof(uint32_t)));
  status_.push_back(st);
  // host-visible mirror of the first failure (optional: without it the status is still polled)
  void* hp = nullptr;
  if (cudaHostAlloc(&hp, kern::kStatusWords * sizeof(uint32_t), cudaHostAllocMapped) == cudaSuccess) {
    std::memset(hp, 0, kern::kStatusWords * sizeof(uint32_t));
    void* dp = nullptr;
    if (cudaHostGetDevicePointer(&dp, hp, 0) == cudaSuccess) {
      status_host_ = static_cast<volatile uint32_t*>(hp);
      const unsigned long long addr = reinterpret_cast<unsigned long long>(dp);
      MCCL_CUDA_CHECK(cudaMemcpy(st + kern::kStatusMirrorWord, &addr, sizeof(addr), cudaMemcpyHostToDevice));
    } else {
      cudaGetLastError();
      cudaFreeHost(hp);
    }
  } else {
    cudaGetLastError();
  }
  MCCL_CUDA_CHECK(cudaDeviceSynchronize());
  if (ws_ == 1) ready_ = true;
}

SymmetricArena* SymmetricArena::make_emulated(int world_size, size_t parity_bytes) {
  MCCL_CHECK(world_size >= 1 && world_size <= kern::kMaxWorld, "bad emulated world size");
  auto* a = new SymmetricArena();
  a->rank_ = 0;
  a->ws_ = world_size;
  a->parity_bytes_ = parity_bytes;
  a->emulated_ = true;
  a->total_bytes_ = kern::kSignalBytes + kern::kNumParity * parity_bytes;
  MCCL_CUDA_CHECK(cudaGetDevice(&a->device_));
  a->bases_.assign(world_size, nullptr);
  a->opened_.assign(world_size, false);
  for (int r = 0; r < world_size; ++r) {
    void* p = nullptr;
    MCCL_CUDA_CHECK(cudaMalloc(&p, a->total_bytes_));
    a->bases_[r] = static_cast<char*>(p);
    MCCL_CUDA_CHECK(cudaMemset(p, 0, kern::kSignalBytes));
    uint32_t* st = nullptr;
    MCCL_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&st), kern::kStatusWords * sizeof(uint32_t)));
    MCCL_CUDA_CHECK(cudaMemset(st, 0, kern::kStatusWords * sizeof(uint32_t)));
    a->status_.push_back(st);
  }
  MCCL_CUDA_CHECK(cudaDeviceSynchronize());
  a->ready_ = true;
  return a;
}

SymmetricArena::~SymmetricArena() {
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(device_);
  for (int r = 0; r < static_cast<int>(bases_.size()); ++r) {
    if (!bases_[r]) continue;
    if (opened_[r]) {
      cudaIpcCloseMemHandle(bases_[r]);
    } else if (emulated_ || r == rank_) {
      cudaFree(bases_[r]);
    }
  }
  for (auto* s : status_)
    if (s) cudaFree(s);
  if (status_host_) cudaFreeHost(const_cast<uint32_t*>(status_host_));
  for (auto* s : stamps_)
    if (s) cudaFreeHost(s);
  if (prev >= 0) cudaSetDevice(prev);
}

std::string SymmetricArena::export_handle() const {
  ExportRecord rec;
  std::memset(&rec, 0, sizeof(rec));
  MCCL_CUDA_CHECK(cudaIpcGetMemHandle(&rec.handle, bases_[rank_]));
  std::string h = host_identity();
  std::strncpy(rec.hostname, h.c_str(), sizeof(rec.hostname) - 1);
  rec.pid = static_cast<int32_t>(getpid());
  rec.device = device_;
  rec.total_bytes = total_bytes_;
  return std::string(reinterpret_cast<const char*>(&rec), sizeof(rec));
}

std::string SymmetricArena::open_peers(const std::vector<std::string>& handles) {
  if (static_cast<int>(handles.size()) != ws_) return "handle list size mismatch";
  const std::string me = host_identity();
  for (int r = 0; r < ws_; ++r) {
    if (r == rank_) continue;
    if (handles[r].size() != sizeof(ExportRecord)) return "malformed arena handle from rank " + std::to_string(r);
    ExportRecord rec;
    std::memcpy(&rec, handles[r].data(), sizeof(rec));
    if (me != rec.hostname)
      return "rank " + std::to_string(r) + " runs on host '" + rec.hostname + "', this rank on '" + me +
             "': peer memory needs one NVLink domain";
    if (rec.total_bytes != total_bytes_) return "arena size differs on rank " + std::to_string(r);
    if (rec.pid == static_cast<int32_t>(getpid()))
      return "rank " + std::to_string(r) + " lives in this process; IPC mapping needs one process per GPU";
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, rec.handle, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();  // clear the sticky-less error
      return std::string("cudaIpcOpenMemHandle(rank ") + std::to_string(r) + "): " + cudaGetErrorString(e);
    }
    bases_[r] = static_cast<char*>(p);
    opened_[r] = true;
  }
  ready_ = true;
  return "";
}

void SymmetricArena::fill_params(kern::CollParams& p, uint32_t epoch) const {
  p.seq = epoch;
  p.parity_offset = kern::kSignalBytes + static_cast<size_t>(epoch % kern::kNumParity) * parity_bytes_;
  p.parity_capacity = parity_bytes_;
  const int nctx = emulated_ ? ws_ : 1;
  for (int i = 0; i < nctx; ++i) {
    kern::RankCtx& c = p.ctx[i];
    c.rank = emulated_ ? i : rank_;
    c.ws = ws_;
    for (int r = 0; r < kern::kMaxWorld; ++r) c.arena[r] = r < ws_ ? bases_[r] : nullptr;
    c.status = status_[i];
    c.stamps = (stamps_on_ && i < static_cast<int>(stamps_dev_.size()))
                   ? stamps_dev_[i] + static_cast<size_t>(epoch % kStampRing) * kern::kStampSlots
                   : nullptr;
    c.nvls_uc = nullptr;
    c.nvls_mc = nullptr;
  }
}

void SymmetricArena::read_status(uint32_t out[kern::kStatusWords], cudaStream_t stream, int r) const {
  MCCL_CUDA_CHECK(cudaMemcpyAsync(out, status_[emulated_ ? r : 0], kern::kStatusWords * sizeof(uint32_t),
                                  cudaMemcpyDeviceToHost, stream));
  MCCL_CUDA_CHECK(cudaStreamSynchronize(stream));
}

void SymmetricArena::enable_stamps(bool on) {
  if (on && stamps_.empty()) {
    const size_t bytes = static_cast<size_t>(kStampRing) * kern::kStampSlots * sizeof(unsigned long long);
    for (size_t i = 0; i < status_.size(); ++i) {
      void* hp = nullptr;
      void* dp = nullptr;
      MCCL_CUDA_CHECK(cudaHostAlloc(&hp, bytes, cudaHostAllocMapped));
      std::memset(hp, 0, bytes);
      MCCL_CUDA_CHECK(cudaHostGetDevicePointer(&dp, hp, 0));
      stamps_.push_back(static_cast<unsigned long long*>(hp));
      stamps_dev_.push_back(static_cast<unsigned long long*>(dp));
    }
  }
  stamps_on_ = on;
}

void SymmetricArena::read_stamps(unsigned long long out[kern::kStampSlots], cudaStream_t stream, int r,
                                 int64_t epoch) const {
  (void)stream;
  for (int i = 0; i < kern::kStampSlots; ++i) out[i] = 0;
  if (stamps_.empty()) return;
  const uint32_t e = epoch < 0 ? epoch_ : static_cast<uint32_t>(epoch);
  const volatile unsigned long long* src =
      stamps_[emulated_ ? r : 0] + static_cast<size_t>(e % kStampRing) * kern::kStampSlots;
  for (int i = 0; i < kern::kStampSlots; ++i) out[i] = src[i];
}

void SymmetricArena::clear_status(cudaStream_t stream) {
  // words 0-3 only: the mirror address in words 4-5 stays
  for (auto* s : status_) MCCL_CUDA_CHECK(cudaMemsetAsync(s, 0, kern::kStatusMirrorWord * sizeof(uint32_t), stream));
  if (status_host_)
    for (int i = 0; i < kern::kStatusMirrorWord; ++i) status_host_[i] = 0u;
}

}  // namespace mccl
