#include "runtime/nvls.h"

#include <cuda.h>
#include <cuda_runtime_api.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <cstdint>
#include <cstring>
#include <random>
#include <sstream>

#include "common/log.h"

namespace mccl {

namespace {

// Driver API entry points, resolved through the runtime (no link-time libcuda dependency).
struct Driver {
  decltype(&cuDeviceGet) DeviceGet = nullptr;
  decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
  decltype(&cuGetErrorString) GetErrorString = nullptr;
  decltype(&cuMulticastGetGranularity) MulticastGetGranularity = nullptr;
  decltype(&cuMulticastCreate) MulticastCreate = nullptr;
  decltype(&cuMulticastAddDevice) MulticastAddDevice = nullptr;
  decltype(&cuMulticastBindMem) MulticastBindMem = nullptr;
  decltype(&cuMulticastUnbind) MulticastUnbind = nullptr;
  decltype(&cuMemGetAllocationGranularity) MemGetAllocationGranularity = nullptr;
  decltype(&cuMemCreate) MemCreate = nullptr;
  decltype(&cuMemRelease) MemRelease = nullptr;
  decltype(&cuMemExportToShareableHandle) MemExportToShareableHandle = nullptr;
  decltype(&cuMemImportFromShareableHandle) MemImportFromShareableHandle = nullptr;
  decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
  decltype(&cuMemAddressFree) MemAddressFree = nullptr;
  decltype(&cuMemMap) MemMap = nullptr;
  decltype(&cuMemUnmap) MemUnmap = nullptr;
  decltype(&cuMemSetAccess) MemSetAccess = nullptr;

  template <typename Fn>
  static bool one(const char* name, Fn* out) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || p == nullptr ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return false;
    }
    *out = reinterpret_cast<Fn>(p);
    return true;
  }
  std::string load() {
#define MCCL_DRV(sym)                                            \
  if (!one("cu" #sym, &sym)) return "driver entry point cu" #sym " not available";
    MCCL_DRV(DeviceGet)
    MCCL_DRV(DeviceGetAttribute)
    MCCL_DRV(GetErrorString)
    MCCL_DRV(MulticastGetGranularity)
    MCCL_DRV(MulticastCreate)
    MCCL_DRV(MulticastAddDevice)
    MCCL_DRV(MulticastBindMem)
    MCCL_DRV(MulticastUnbind)
    MCCL_DRV(MemGetAllocationGranularity)
    MCCL_DRV(MemCreate)
    MCCL_DRV(MemRelease)
    MCCL_DRV(MemExportToShareableHandle)
    MCCL_DRV(MemImportFromShareableHandle)
    MCCL_DRV(MemAddressReserve)
    MCCL_DRV(MemAddressFree)
    MCCL_DRV(MemMap)
    MCCL_DRV(MemUnmap)
    MCCL_DRV(MemSetAccess)
#undef MCCL_DRV
    return "";
  }
  std::string err(const char* what, CUresult r) const {
    const char* s = nullptr;
    if (GetErrorString) GetErrorString(r, &s);
    std::ostringstream o;
    o << what << " failed: " << (s ? s : "unknown error") << " (" << static_cast<int>(r) << ")";
    return o.str();
  }
};

// ---- file-descriptor passing over abstract Unix datagram sockets ------------------------------
socklen_t abstract_addr(const std::string& name, sockaddr_un* a) {
  std::memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  const size_t n = std::min(name.size(), sizeof(a->sun_path) - 2);
  std::memcpy(a->sun_path + 1, name.data(), n);  // sun_path[0] == 0: abstract namespace, no file
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}

int bound_socket(const std::string& name) {
  int s = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (s < 0) return -1;
  sockaddr_un a;
  const socklen_t len = abstract_addr(name, &a);
  if (bind(s, reinterpret_cast<sockaddr*>(&a), len) != 0) {
    close(s);
    return -1;
  }
  return s;
}

bool send_fd(int sock, const std::string& to, int fd) {
  sockaddr_un a;
  const socklen_t len = abstract_addr(to, &a);
  char payload = 'F';
  iovec iov{&payload, 1};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  std::memset(ctrl, 0, sizeof(ctrl));
  msghdr m{};
  m.msg_name = &a;
  m.msg_namelen = len;
  m.msg_iov = &iov;
  m.msg_iovlen = 1;
  m.msg_control = ctrl;
  m.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&m);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
  return sendmsg(sock, &m, 0) == 1;
}

int recv_fd(int sock, int timeout_ms) {
  pollfd p{sock, POLLIN, 0};
  if (poll(&p, 1, timeout_ms) <= 0) return -1;
  char payload = 0;
  iovec iov{&payload, 1};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  std::memset(ctrl, 0, sizeof(ctrl));
  msghdr m{};
  m.msg_iov = &iov;
  m.msg_iovlen = 1;
  m.msg_control = ctrl;
  m.msg_controllen = sizeof(ctrl);
  if (recvmsg(sock, &m, MSG_CMSG_CLOEXEC) != 1) return -1;
  for (cmsghdr* c = CMSG_FIRSTHDR(&m); c != nullptr; c = CMSG_NXTHDR(&m, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
      int fd = -1;
      std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
      return fd;
    }
  }
  return -1;
}

size_t round_up_to(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace

struct NvlsRegion::Impl {
  Driver d;
  int device = 0;
  CUdevice cudev = 0;
  size_t total = 0;
  CUmemGenericAllocationHandle mc_handle = 0, mem_handle = 0;
  bool have_mc = false, have_mem = false, bound = false;
  CUdeviceptr uc_va = 0, mc_va = 0;
  bool uc_mapped = false, mc_mapped = false;
};

bool NvlsRegion::device_supported(std::string* why) {
  Driver d;
  std::string e = d.load();
  int dev = 0;
  if (e.empty() && cudaGetDevice(&dev) != cudaSuccess) e = "no current CUDA device";
  if (e.empty()) {
    cudaFree(nullptr);  // make sure the primary context exists
    CUdevice cd;
    int ok = 0;
    CUresult r = d.DeviceGet(&cd, dev);
    if (r != CUDA_SUCCESS) e = d.err("cuDeviceGet", r);
    else if ((r = d.DeviceGetAttribute(&ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cd)) != CUDA_SUCCESS)
      e = d.err("cuDeviceGetAttribute(MULTICAST_SUPPORTED)", r);
    else if (!ok) e = "device reports no NVLink multicast support";
    else if ((r = d.DeviceGetAttribute(&ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cd)) !=
                 CUDA_SUCCESS ||
             !ok)
      e = "POSIX file-descriptor memory handles are not supported";
  }
  if (why) *why = e;
  return e.empty();
}

std::unique_ptr<NvlsRegion> NvlsRegion::create(int rank, int ws, size_t buffer_bytes, int nbuffers,
                                               const std::string& uid_hint, const Exchange& exchange_raw,
                                               std::string* why) {
  const Exchange exchange = [&](const std::string& tag, const std::string& mine) {
    return exchange_raw(uid_hint + "/" + tag, mine);
  };
  std::unique_ptr<NvlsRegion> reg(new NvlsRegion());
  reg->impl_ = std::make_unique<Impl>();
  Impl& im = *reg->impl_;
  reg->buffer_bytes_ = buffer_bytes;
  reg->nbuffers_ = nbuffers;
  int sock = -1;

  // One agreement round: every rank reports "" or its error; any error ends the set-up everywhere.
  auto agree = [&](const std::string& tag, const std::string& local, std::vector<std::string>* all_out = nullptr) {
    std::vector<std::string> all = exchange(tag, local.empty() ? std::string("ok") : "E" + local);
    std::string bad;
    for (int r = 0; r < ws && bad.empty(); ++r)
      if (all[r].rfind("ok", 0) != 0) bad = "rank " + std::to_string(r) + ": " + (all[r].empty() ? "?" : all[r].substr(1));
    if (all_out) *all_out = std::move(all);
    return bad;
  };
  auto fail = [&](const std::string& e) -> std::unique_ptr<NvlsRegion> {
    if (sock >= 0) close(sock);
    reg->release();
    if (why) *why = e;
    return nullptr;
  };

  // ---- exchange 0: local capability + rank 0's unique id for the socket names ---------------------
  std::string e;
  if (!device_supported(&e)) { /* e set */ }
  if (e.empty()) e = im.d.load();
  if (e.empty() && cudaGetDevice(&im.device) != cudaSuccess) e = "no current CUDA device";
  if (e.empty()) {
    CUresult r = im.d.DeviceGet(&im.cudev, im.device);
    if (r != CUDA_SUCCESS) e = im.d.err("cuDeviceGet", r);
  }
  std::string uid;
  {
    static std::atomic<unsigned> counter{0};
    std::random_device rd;
    std::ostringstream o;
    o << uid_hint << "-" << getpid() << "-" << counter.fetch_add(1) << "-" << std::hex << rd();
    uid = o.str();
  }
  {
    std::vector<std::string> got = exchange("nvls_uid", (e.empty() ? "ok" : "E" + e) + std::string("|") + uid);
    std::string bad;
    for (int r = 0; r < ws && bad.empty(); ++r)
      if (got[r].rfind("ok|", 0) != 0) bad = "rank " + std::to_string(r) + ": " + got[r].substr(0, got[r].find('|'));
    if (!bad.empty()) return fail(bad);
    uid = got[0].substr(3);  // everybody uses rank 0's id
  }
  auto sock_name = [&](int r) { return "mccl-nvls-" + uid + "-" + std::to_string(r); };

  // ---- exchange 1: sockets bound everywhere; rank 0 creates and exports the multicast object ------
  CUmulticastObjectProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.numDevices = static_cast<unsigned>(ws);
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  prop.size = buffer_bytes * static_cast<size_t>(nbuffers);
  CUmemAllocationProp aprop;
  std::memset(&aprop, 0, sizeof(aprop));
  aprop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  aprop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  aprop.location.id = im.device;
  aprop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  int export_fd = -1;
  {
    size_t g_mc = 0, g_mem = 0;
    CUresult r = im.d.MulticastGetGranularity(&g_mc, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED);
    if (r != CUDA_SUCCESS) e = im.d.err("cuMulticastGetGranularity", r);
    if (e.empty() && (r = im.d.MemGetAllocationGranularity(&g_mem, &aprop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED)) !=
                         CUDA_SUCCESS)
      e = im.d.err("cuMemGetAllocationGranularity", r);
    gran = std::max(g_mc, g_mem);
    if (e.empty() && gran == 0) e = "zero allocation granularity";
  }
  if (e.empty()) {
    im.total = round_up_to(prop.size, gran);
    prop.size = im.total;
    sock = bound_socket(sock_name(rank));
    if (sock < 0) e = std::string("cannot bind the handle-passing socket: ") + std::strerror(errno);
  }
  if (e.empty() && rank == 0) {
    CUresult r = im.d.MulticastCreate(&im.mc_handle, &prop);
    if (r != CUDA_SUCCESS) e = im.d.err("cuMulticastCreate", r);
    else {
      im.have_mc = true;
      r = im.d.MemExportToShareableHandle(&export_fd, im.mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      if (r != CUDA_SUCCESS) e = im.d.err("cuMemExportToShareableHandle", r);
    }
  }
  {
    // ranks also compare the size they derived: it must be the same everywhere
    std::vector<std::string> got = exchange("nvls_create", (e.empty() ? "ok" : "E" + e) + std::string("|") + std::to_string(im.total));
    std::string bad;
    for (int r = 0; r < ws && bad.empty(); ++r) {
      if (got[r].rfind("ok|", 0) != 0) bad = "rank " + std::to_string(r) + ": " + got[r].substr(1, got[r].find('|') - 1);
      else if (got[r].substr(3) != std::to_string(im.total)) bad = "rank " + std::to_string(r) + " derived another region size";
    }
    if (!bad.empty()) {
      if (export_fd >= 0) close(export_fd);
      return fail(bad);
    }
  }

  // ---- exchange 2: the handle reaches every rank; every rank adds its device -----------------------
  if (rank == 0) {
    for (int r = 1; r < ws && e.empty(); ++r)
      if (!send_fd(sock, sock_name(r), export_fd)) e = std::string("sending the multicast handle to rank ") + std::to_string(r) + ": " + std::strerror(errno);
    if (export_fd >= 0) close(export_fd);
  } else {
    int fd = recv_fd(sock, 20000);
    if (fd < 0) e = "multicast handle from rank 0 did not arrive";
    else {
      CUresult r = im.d.MemImportFromShareableHandle(&im.mc_handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                     CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      close(fd);
      if (r != CUDA_SUCCESS) e = im.d.err("cuMemImportFromShareableHandle", r);
      else im.have_mc = true;
    }
  }
  close(sock);
  sock = -1;
  if (e.empty()) {
    CUresult r = im.d.MulticastAddDevice(im.mc_handle, im.cudev);
    if (r != CUDA_SUCCESS) e = im.d.err("cuMulticastAddDevice", r);
  }
  {
    std::string bad = agree("nvls_add", e);
    if (!bad.empty()) return fail(bad);
  }

  // ---- exchange 3: physical memory, bind, map ------------------------------------------------------
  {
    CUresult r = im.d.MemCreate(&im.mem_handle, im.total, &aprop, 0);
    if (r != CUDA_SUCCESS) e = im.d.err("cuMemCreate", r);
    else im.have_mem = true;
    if (e.empty()) {
      r = im.d.MulticastBindMem(im.mc_handle, 0, im.mem_handle, 0, im.total, 0);
      if (r != CUDA_SUCCESS) e = im.d.err("cuMulticastBindMem", r);
      else im.bound = true;
    }
    CUmemAccessDesc acc;
    std::memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = im.device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    if (e.empty()) {
      if ((r = im.d.MemAddressReserve(&im.uc_va, im.total, gran, 0, 0)) != CUDA_SUCCESS) e = im.d.err("cuMemAddressReserve", r);
      else if ((r = im.d.MemMap(im.uc_va, im.total, 0, im.mem_handle, 0)) != CUDA_SUCCESS) e = im.d.err("cuMemMap(unicast)", r);
      else {
        im.uc_mapped = true;
        if ((r = im.d.MemSetAccess(im.uc_va, im.total, &acc, 1)) != CUDA_SUCCESS) e = im.d.err("cuMemSetAccess(unicast)", r);
      }
    }
    if (e.empty()) {
      if ((r = im.d.MemAddressReserve(&im.mc_va, im.total, gran, 0, 0)) != CUDA_SUCCESS) e = im.d.err("cuMemAddressReserve", r);
      else if ((r = im.d.MemMap(im.mc_va, im.total, 0, im.mc_handle, 0)) != CUDA_SUCCESS) e = im.d.err("cuMemMap(multicast)", r);
      else {
        im.mc_mapped = true;
        if ((r = im.d.MemSetAccess(im.mc_va, im.total, &acc, 1)) != CUDA_SUCCESS) e = im.d.err("cuMemSetAccess(multicast)", r);
      }
    }
    if (e.empty()) {
      if (cudaMemset(reinterpret_cast<void*>(im.uc_va), 0, im.total) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        e = std::string("clearing the region: ") + cudaGetErrorString(cudaGetLastError());
      }
    }
  }
  {
    std::string bad = agree("nvls_bind", e);
    if (!bad.empty()) return fail(bad);
  }
  reg->uc_ = reinterpret_cast<char*>(im.uc_va);
  reg->mc_ = reinterpret_cast<char*>(im.mc_va);
  MCCL_INFO("rank %d: NVLS region ready: %d buffers x %zu MiB bound to one multicast object over %d GPUs", rank, nbuffers,
            buffer_bytes >> 20, ws);
  return reg;
}

void NvlsRegion::release() {
  if (!impl_) return;
  Impl& im = *impl_;
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(im.device);
  if (im.mc_mapped) im.d.MemUnmap(im.mc_va, im.total);
  if (im.mc_va) im.d.MemAddressFree(im.mc_va, im.total);
  if (im.bound) im.d.MulticastUnbind(im.mc_handle, im.cudev, 0, im.total);
  if (im.uc_mapped) im.d.MemUnmap(im.uc_va, im.total);
  if (im.uc_va) im.d.MemAddressFree(im.uc_va, im.total);
  if (im.have_mem) im.d.MemRelease(im.mem_handle);
  if (im.have_mc) im.d.MemRelease(im.mc_handle);
  im.mc_mapped = im.uc_mapped = im.bound = im.have_mem = im.have_mc = false;
  im.mc_va = im.uc_va = 0;
  uc_ = mc_ = nullptr;
  if (prev >= 0) cudaSetDevice(prev);
  impl_.reset();
}

void NvlsRegion::release_multicast_keep_memory() {
  if (!impl_) return;
  Impl& im = *impl_;
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(im.device);
  if (im.mc_mapped) im.d.MemUnmap(im.mc_va, im.total);
  if (im.mc_va) im.d.MemAddressFree(im.mc_va, im.total);
  if (im.bound) im.d.MulticastUnbind(im.mc_handle, im.cudev, 0, im.total);
  if (im.have_mc) im.d.MemRelease(im.mc_handle);
  im.mc_mapped = im.bound = im.have_mc = false;
  im.mc_va = 0;
  mc_ = nullptr;
  if (prev >= 0) cudaSetDevice(prev);
}

size_t NvlsRegion::total_bytes() const { return impl_ ? impl_->total : 0; }

NvlsRegion::~NvlsRegion() { release(); }

}  // namespace mccl
