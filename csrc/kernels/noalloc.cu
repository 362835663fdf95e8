// Allocation-free top-k selection: see noalloc.h for the contract.
//
// The scratch the selection kernels need is a file-scope device array.  Host
// code cannot hand that symbol to a kernel directly (on the host the name is
// only a stand-in, not a device address), so the first call on each device asks
// the runtime for the array's device address, with that device current, and
// every launch passes that address on.
#include "kernels/noalloc.h"

#include <cstdio>
#include <mutex>

#include "kernels/topk_api.h"

namespace {

constexpr size_t kScratchBytes = 64 * 1024;  // >= mccl::kern::topk_scratch_bytes(), checked at set-up
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_noalloc_topk_scratch[kScratchBytes];

std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {nullptr};
thread_local char g_err[256] = {0};

int fail(int code, const char* msg) {
  std::snprintf(g_err, sizeof(g_err), "%s", msg);
  return code;
}

// Device address of the scratch array on the current device (looked up once per device).
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(2, cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(1, "device index out of range");
  std::lock_guard<std::mutex> g(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    if (mccl::kern::topk_scratch_bytes() > kScratchBytes) return fail(2, "built-in scratch array is too small");
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_topk_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return fail(2, e != cudaSuccess ? cudaGetErrorString(e) : "cudaGetSymbolAddress returned null");
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int mccl_topk_select_noalloc(const float* grad, float* residual,
                                                                              long long n, long long k,
                                                                              void* pairs_out, cudaStream_t stream) {
  g_err[0] = 0;
  if (grad == nullptr || residual == nullptr || pairs_out == nullptr) return fail(1, "null pointer argument");
  if (n < 1 || n > MCCL_NOALLOC_TOPK_MAX_N) {
    char msg[128];
    std::snprintf(msg, sizeof(msg), "n = %lld is outside 1..%lld", n, (long long)MCCL_NOALLOC_TOPK_MAX_N);
    return fail(1, msg);
  }
  if (k < 1 || k > n) {
    char msg[128];
    std::snprintf(msg, sizeof(msg), "k = %lld is outside 1..n (n = %lld)", k, n);
    return fail(1, msg);
  }
  // The scratch array that is used belongs to the CURRENT device, so the caller's buffers must
  // live there too: a launch with another GPU's scratch would fail or, with peer access on,
  // silently work on the wrong GPU's array.
  {
    int cur = -1;
    cudaError_t ce = cudaGetDevice(&cur);
    if (ce != cudaSuccess) return fail(2, cudaGetErrorString(ce));
    const void* bufs[3] = {grad, residual, pairs_out};
    const char* names[3] = {"grad", "residual", "pairs_out"};
    for (int i = 0; i < 3; ++i) {
      cudaPointerAttributes at;
      ce = cudaPointerGetAttributes(&at, bufs[i]);
      if (ce != cudaSuccess) {
        cudaGetLastError();
        return fail(2, cudaGetErrorString(ce));
      }
      if ((at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) && at.device != cur) {
        char msg[160];
        std::snprintf(msg, sizeof(msg), "%s lives on device %d but device %d is current: make the buffers' device current",
                      names[i], at.device, cur);
        return fail(1, msg);
      }
    }
  }
  void* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  mccl::kern::TopkArgs a;
  a.grad = grad;
  a.grad_is_bf16 = false;
  a.residual = residual;
  a.n = n;
  a.k = k;
  a.scratch = scratch;  // the selection starts by clearing the histograms and state it uses
  a.pairs = pairs_out;
  a.scale = 1.0f;
  cudaError_t e = mccl::kern::launch_topk_select(a, stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(2, cudaGetErrorString(e));
  }
  return 0;
}

extern "C" __attribute__((visibility("default"))) const char* mccl_noalloc_last_error(void) { return g_err; }
