// CUDA data path of ProcessGroupMCCL: stream-ordered launches of the fused
// collective kernels over the SymmetricArena.
//
// Ordering (replaces the reference's MTLSharedEvent fences,
// reference csrc/metal/EventSync.mm:123-234):
//   producer fence   cudaEventRecord(current stream) + cudaStreamWaitEvent(comm)
//   kernel(s)        on the high-priority communication stream, one epoch each
//   consumer release event recorded behind the kernels; Work::wait and the
//                    CUDA-aware Future make consumers wait for it on-device
// With MCCL_OVERLAP_COMM=0 the kernels run on the caller's stream instead.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime_api.h>
#include <nvtx3/nvToolsExt.h>

#include <set>

#include "backend/process_group.h"
#include "backend/tensor_checks.h"
#include "common/log.h"
#include "kernels/topk_api.h"
#include "runtime/nvls.h"
#include "runtime/nvls_pool.h"

namespace mccl {

struct ProcessGroupMCCL::CudaState {
  c10::DeviceIndex dev = 0;
  // One communication stream per lane: epoch e launches on lanes[e % 2], so two
  // consecutive collectives (two DDP buckets) overlap each other's sync gaps.
  std::vector<c10::cuda::CUDAStream> lanes;
  cudaEvent_t lane_done[kern::kNumLanes] = {nullptr, nullptr};   // recorded behind the lane's latest epoch
  cudaStream_t lane_last[kern::kNumLanes] = {nullptr, nullptr};  // stream that epoch was launched on
  bool lane_used[kern::kNumLanes] = {false, false};
  cudaEvent_t join_ev = nullptr;
  cudaStream_t poll_stream = nullptr;
  std::unique_ptr<SymmetricArena> arena;
  std::unique_ptr<NvlsRegion> nvls;  // multicast-bound buffers (nullptr: not supported / switched off)
  bool user_pool = false;       // this group owns the device's multicast-bound tensor pool
  std::set<size_t> pool_offsets_ok;  // tensor offsets in that pool already checked to agree on every rank
  std::set<size_t> pool_offsets_bad; // offsets that differ between ranks: those tensors take the staged paths
  bool p2p = false;
  bool stamps_always = false;  // MCCL_PHASE_STAMPS=1: every collective stamps, not only the timed ones
  std::string why_not;
  at::cuda::CUDAEvent fence{cudaEventDisableTiming};
  struct Pending {
    uint32_t seq;
    cudaEvent_t start, end;
    const char* name;     // collective, for the INFO line
    const char* algo;     // kernel variant
    uint64_t bytes;       // payload of this rank
    double bus_factor;    // busbw = bytes / t * bus_factor
    double sync_ms;       // host time spent fencing streams for this collective
    bool stamps;          // phase stamps were captured for it
    int64_t stamp_epoch;  // arena epoch of its last launch
  };
  std::deque<Pending> pending;
  std::vector<cudaEvent_t> free_events;
  std::mutex pending_mu;
  uint32_t last_status[kern::kStatusWords] = {0};

  cudaEvent_t get_event() {
    if (!free_events.empty()) {
      cudaEvent_t e = free_events.back();
      free_events.pop_back();
      return e;
    }
    cudaEvent_t e;
    MCCL_CUDA_CHECK(cudaEventCreate(&e));
    return e;
  }
  ~CudaState() {
    c10::cuda::OptionalCUDAGuard g(dev);
    for (auto& p : pending) {
      cudaEventDestroy(p.start);
      cudaEventDestroy(p.end);
    }
    for (auto e : free_events) cudaEventDestroy(e);
    for (auto e : lane_done)
      if (e) cudaEventDestroy(e);
    if (join_ev) cudaEventDestroy(join_ev);
    nvls.reset();
    arena.reset();
    if (poll_stream) cudaStreamDestroy(poll_stream);
  }
};

std::string ProcessGroupMCCL::data_plane() const {
  if (getSize() == 1) return "local";
  if (!cuda_) return "uninitialised";
  return cuda_->p2p ? (cuda_->nvls ? "nvlink-p2p+nvls" : "nvlink-p2p") : "host-staged";
}

bool ProcessGroupMCCL::device_failed_quick() const {
  const SymmetricArena* a = arena_quick_.load(std::memory_order_acquire);
  return a != nullptr && a->device_failed();
}

// Ordered tear-down of the NVLS region.  Memory bound to a multicast object must not disappear
// while a peer can still issue a multimem access to it, so: drain this rank's communication
// streams, meet the peers at a host-side rendezvous (bounded: a peer that is gone cannot be waited
// for), and only then unmap and unbind.
void ProcessGroupMCCL::release_nvls() {
  std::lock_guard<std::mutex> g(cuda_mu_);
  if (!cuda_ || (!cuda_->nvls && !cuda_->user_pool)) return;
  c10::cuda::OptionalCUDAGuard guard(cuda_->dev);
  for (auto& l : cuda_->lanes) cudaStreamSynchronize(l.stream());
  cudaDeviceSynchronize();
  cudaGetLastError();
  try {
    rendezvous_->exchange("nvls_bye", "bye", std::chrono::milliseconds(env_int("MCCL_NVLS_BYE_TIMEOUT_MS", 5000)));
  } catch (const std::exception& e) {
    MCCL_WARN("rank %d: peers did not all reach the NVLS tear-down rendezvous (%s); releasing anyway", getRank(), e.what());
  }
  if (cuda_->user_pool) {
    // tensors in the pool may outlive this group: only the multicast side ends here
    NvlsUserPool::get(cuda_->dev).end_multicast();
    cuda_->user_pool = false;
  }
  if (cuda_->nvls) {
    cuda_->nvls->release();
    cuda_->nvls.reset();
  }
}

// Collective: creates the device's pool of multicast-bound memory for user tensors (gradient
// buckets) on this group.  Returns false, on every rank alike, when NVLS is not available.
bool ProcessGroupMCCL::create_nvls_user_pool(int64_t bytes, c10::DeviceIndex dev) {
  if (getSize() < 2 || options_->nvls == "0" || options_->nvls == "off") return false;
  ensure_cuda(dev);
  std::lock_guard<std::mutex> g(cuda_mu_);
  if (!cuda_->p2p) return false;
  if (cuda_->user_pool) return true;
  c10::cuda::CUDAGuard guard(dev);
  const auto timeout = std::chrono::milliseconds(env_int("MCCL_CONNECT_TIMEOUT_MS", 30000));
  std::string why;
  if (NvlsUserPool::get(dev).active()) why = "another process group already owns this device's pool";
  // agree first: one rank that cannot must keep all of them off the path
  auto votes = rendezvous_->exchange("nvls_pool_vote", why.empty() ? "ok" : why, timeout);
  for (auto& v : votes)
    if (v != "ok") {
      MCCL_WARN("rank %d: no multicast-bound tensor pool (%s)", getRank(), v.c_str());
      return false;
    }
  auto region = NvlsRegion::create(
      getRank(), getSize(), static_cast<size_t>(bytes), 1, "pool",
      [this, timeout](const std::string& tag, const std::string& mine) { return rendezvous_->exchange(tag, mine, timeout); }, &why);
  if (!region) {
    MCCL_INFO("rank %d: no multicast-bound tensor pool (%s)", getRank(), why.c_str());
    return false;
  }
  cuda_->user_pool = NvlsUserPool::get(dev).attach(std::move(region));
  return cuda_->user_pool;
}

void ProcessGroupMCCL::ensure_cuda(c10::DeviceIndex dev) {
  std::lock_guard<std::mutex> g(cuda_mu_);
  if (cuda_) {
    MCCL_CHECK(cuda_->dev == dev, "this process group is bound to cuda:" << int(cuda_->dev)
                                                                         << " but got a tensor on cuda:" << int(dev));
    return;
  }
  c10::cuda::CUDAGuard guard(dev);
  auto st = std::make_shared<CudaState>();
  st->dev = dev;
  for (int l = 0; l < kern::kNumLanes; ++l) {
    st->lanes.push_back(c10::cuda::getStreamFromPool(/*isHighPriority=*/true, dev));
    MCCL_CUDA_CHECK(cudaEventCreateWithFlags(&st->lane_done[l], cudaEventDisableTiming));
  }
  MCCL_CHECK(st->lanes[0] != st->lanes[1], "stream pool returned one stream twice");
  MCCL_CUDA_CHECK(cudaEventCreateWithFlags(&st->join_ev, cudaEventDisableTiming));
  MCCL_CUDA_CHECK(cudaStreamCreateWithFlags(&st->poll_stream, cudaStreamNonBlocking));

  const int ws = getSize();
  std::string local_reason;
  if (options_->algo == "staged") {
    local_reason = "MCCL_ALGO=staged";
  } else if (ws > kern::kMaxWorld) {
    local_reason = "world size " + std::to_string(ws) + " exceeds one NVLink domain of " + std::to_string(kern::kMaxWorld);
  } else {
    try {
      st->arena = std::make_unique<SymmetricArena>(getRank(), ws, static_cast<size_t>(options_->arena_bytes));
    } catch (const std::exception& e) {
      local_reason = e.what();
    }
  }
  const auto timeout = std::chrono::milliseconds(env_int("MCCL_CONNECT_TIMEOUT_MS", 30000));
  // First exchange: publish handles (or the reason there is none).
  std::string mine = st->arena ? ("H" + st->arena->export_handle()) : ("X" + local_reason);
  auto all = rendezvous_->exchange("arena", mine, timeout);
  if (local_reason.empty()) {
    std::vector<std::string> handles(ws);
    for (int r = 0; r < ws; ++r) {
      if (all[r].empty() || all[r][0] != 'H') {
        local_reason = "rank " + std::to_string(r) + " has no arena: " + (all[r].empty() ? "" : all[r].substr(1));
        break;
      }
      handles[r] = all[r].substr(1);
    }
    if (local_reason.empty()) local_reason = st->arena->open_peers(handles);
  }
  // Second exchange: agree. One failure anywhere puts every rank on the host-staged path.
  auto answers = rendezvous_->exchange("arena_ok", local_reason.empty() ? "ok" : local_reason, timeout);
  st->p2p = true;
  for (int r = 0; r < ws; ++r)
    if (answers[r] != "ok") {
      st->p2p = false;
      st->why_not = "rank " + std::to_string(r) + ": " + answers[r];
      break;
    }
  if (!st->p2p) {
    st->arena.reset();
    MCCL_WARN("rank %d: peer-memory data plane unavailable (%s); CUDA collectives are staged through host memory",
              getRank(), st->why_not.c_str());
    ensure_transport();
  } else {
    MCCL_INFO("rank %d: NVLink peer arena mapped on %d ranks (%lld MiB x2 per rank)", getRank(), ws,
              (long long)(options_->arena_bytes >> 20));
  }
  // Phase stamps (seven %globaltimer reads by one thread per kernel) feed the reduce/network split of
  // the metrics for the timed collectives; MCCL_PHASE_STAMPS=0 switches them off.
  if (st->arena && (device_timing_ > 0 || env_bool("MCCL_PHASE_STAMPS", false)) && env_bool("MCCL_PHASE_STAMPS", true))
    st->arena->enable_stamps(true);
  st->stamps_always = std::getenv("MCCL_PHASE_STAMPS") != nullptr && env_bool("MCCL_PHASE_STAMPS", false);
  // NVLS region: collective set-up with agreement rounds, so either every rank has it or none.
  if (st->p2p && ws >= 2 && options_->nvls != "0" && options_->nvls != "off") {
    std::string why;
    st->nvls = NvlsRegion::create(
        getRank(), ws, static_cast<size_t>(options_->nvls_bytes), kern::kNumParity, "pg",
        [this, timeout](const std::string& tag, const std::string& mine) { return rendezvous_->exchange(tag, mine, timeout); },
        &why);
    if (!st->nvls) {
      if (options_->nvls == "1" || options_->nvls == "on" || options_->algo == "nvls")
        MCCL_WARN("rank %d: NVLS requested but unavailable (%s); using the peer-memory kernels", getRank(), why.c_str());
      else
        MCCL_INFO("rank %d: NVLS not used (%s)", getRank(), why.c_str());
    }
  }
  arena_quick_.store(st->arena.get(), std::memory_order_release);
  cuda_ = std::move(st);
}

std::vector<int64_t> ProcessGroupMCCL::last_phase_stamps() {
  std::vector<int64_t> out;
  std::lock_guard<std::mutex> g(cuda_mu_);
  if (!cuda_ || !cuda_->arena) return out;
  c10::cuda::CUDAGuard guard(cuda_->dev);
  for (auto& l : cuda_->lanes) MCCL_CUDA_CHECK(cudaStreamSynchronize(l.stream()));
  unsigned long long st[kern::kStampSlots];
  cuda_->arena->read_stamps(st, cuda_->poll_stream);
  for (auto v : st) out.push_back(static_cast<int64_t>(v));
  return out;
}

// Retires collectives whose end event has fired: device time -> metrics, watchdog entry closed,
// events back to the pool.  Never blocks.
void ProcessGroupMCCL::drain_finished() {
  if (!cuda_) return;
  CudaState& cs = *cuda_;
  std::lock_guard<std::mutex> pg(cs.pending_mu);
  while (!cs.pending.empty()) {
    auto& p = cs.pending.front();
    cudaError_t q = cudaEventQuery(p.end);
    if (q == cudaErrorNotReady) {
      cudaGetLastError();
      break;
    }
    float ms = 0.f;
    if (q == cudaSuccess && cudaEventElapsedTime(&ms, p.start, p.end) != cudaSuccess) {
      cudaGetLastError();
      ms = 0.f;
    }
    // Phase split: SYNC = host time spent ordering streams, REDUCE = device time of the reduction
    // phase when the in-kernel stamps are on (stamp 3 -> 4), NETWORK = the rest of the device time.
    double reduce_ms = 0.0;
    if (p.stamps && cs.arena) {
      unsigned long long st[kern::kStampSlots];
      try {
        cs.arena->read_stamps(st, cs.poll_stream, 0, p.stamp_epoch);
        // share of the kernel spent between "peers' data seen" and "reduction done"; for a
        // segmented collective the last segment's share stands for all of them
        if (st[0] != 0 && st[3] >= st[0] && st[4] > st[3] && st[6] >= st[4] && st[6] > st[0])
          reduce_ms = ms * static_cast<double>(st[4] - st[3]) / static_cast<double>(st[6] - st[0]);
      } catch (const std::exception&) {
      }
    }
    metrics_.record_phase(p.seq, Metrics::Phase::SYNC, p.sync_ms);
    metrics_.record_phase(p.seq, Metrics::Phase::REDUCE, reduce_ms);
    metrics_.record_phase(p.seq, Metrics::Phase::NETWORK, ms - reduce_ms);
    metrics_.op_end_timed(p.seq, ms);
    if (log_enabled(LogLevel::INFO) && p.name != nullptr)
      MCCL_INFO("%s seq=%u algo=%s bytes=%llu device_us=%.1f busbw=%.2f GB/s", p.name, p.seq, p.algo ? p.algo : "-",
                (unsigned long long)p.bytes, ms * 1e3, ms > 0.f ? static_cast<double>(p.bytes) * p.bus_factor / (ms * 1e6) : 0.0);
    watchdog_->complete(p.seq);
    cs.free_events.push_back(p.start);
    cs.free_events.push_back(p.end);
    cs.pending.pop_front();
  }
}

void ProcessGroupMCCL::poll_device(bool must) {
  // The watchdog polls opportunistically; a blocking wait must not miss a status that another
  // thread is reading right now, so it queues behind that thread instead of giving up.
  std::unique_lock<std::mutex> g(cuda_mu_, std::defer_lock);
  if (must) g.lock();
  else if (!g.try_lock()) return;
  if (!cuda_) return;
  CudaState& cs = *cuda_;
  c10::cuda::OptionalCUDAGuard guard(cs.dev);
  // 1. finished collectives -> metrics + watchdog
  drain_finished();
  // 2. device status block (bounded waits that gave up)
  if (cs.arena && !poisoned_.load()) {
    uint32_t st[kern::kStatusWords] = {0};
    try {
      cs.arena->read_status(st, cs.poll_stream);
    } catch (const std::exception& e) {
      g.unlock();
      poison(std::string("device status read failed: ") + e.what(), true);
      return;
    }
    if (st[0] != kern::ERR_NONE) {
      std::memcpy(cs.last_status, st, sizeof(st));
      std::ostringstream o;
      o << "device-side wait timed out: arena epoch " << st[1] << " phase " << st[2] << " waiting for rank " << st[3]
        << " (limit " << options_->device_wait_us << " us)";
      g.unlock();
      metrics_.record_error();
      poison(o.str(), /*tell_peers=*/true);
    }
  }
}

void ProcessGroupMCCL::device_health_check() {
  poll_device(/*must=*/true);
  if (poisoned_.load()) throw MCCLError("collective failed: " + poison_reason());
}

namespace {

double ms_since(std::chrono::steady_clock::time_point t0) {
  return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
}

}  // namespace

#define MCCL_LAUNCH_CHECK(expr)                                                       \
  do {                                                                                \
    cudaError_t _le = (expr);                                                         \
    if (_le != cudaSuccess) {                                                         \
      cudaGetLastError();                                                             \
      throw DeviceError(std::string(#expr) + ": " + cudaGetErrorString(_le));         \
    }                                                                                 \
  } while (0)

// Shared prologue/epilogue of every arena collective.
//
// Stream discipline.  Every launch takes the next arena epoch e; its lane is
// e % 2.  With overlap on, the launch goes to that lane's stream (or, for
// `serial` collectives that reuse temporaries between launches, always to lane
// stream 0); with overlap off, to the caller's current stream.  Whatever the
// stream, epochs of one lane stay ordered: a launch on a stream other than the
// one its lane last used first waits for an event recorded (at that moment) on
// the lane's previous stream.  The kernels' buffer-reuse credit relies on
// exactly this ordering.
//
// The host path is kept short because small collectives are bounded by it:
// streams are fenced only when they are first used by the collective, device
// timing events are recorded only when MCCL_DEVICE_TIMING is on, and the Work's
// CUDA future is materialised only if somebody asks for it.
struct CudaPath {
  ProcessGroupMCCL& pg;
  ProcessGroupMCCL::CudaState& cs;
  c10::intrusive_ptr<WorkMCCL> work;
  uint32_t seq;
  c10::cuda::CUDAStream caller;
  c10::cuda::CUDAStream stream;  // stream of the current epoch (valid after params())
  bool serial;
  bool overlap;
  bool timing;
  bool fenced = false;           // producer event recorded on the caller's stream
  int cur_lane = -1;
  cudaStream_t used[kern::kNumLanes + 1] = {nullptr, nullptr, nullptr};
  int n_used = 0;
  std::vector<at::Tensor> kept;
  cudaEvent_t ev_start = nullptr, ev_end = nullptr;
  bool skip = false;
  std::function<void(cudaStream_t)> epilogue;  // enqueued behind the collective, covered by the Work
  const char* op_name;
  const char* algo = nullptr;    // kernel variant of the last launch (INFO line)
  uint64_t payload;
  double bus_factor = 1.0;       // busbw = payload / t * bus_factor
  double sync_ms = 0.0;          // host time spent in producer fences
  bool reducing = false;         // the kernels of this collective write reduction-phase stamps
  int64_t last_epoch = -1;
  bool range_open = false;

  CudaPath(ProcessGroupMCCL& pg_, c10d::OpType op, const char* name, uint64_t bytes, std::vector<at::Tensor> outs,
           c10::DeviceIndex dev, bool serial_ = false)
      : pg(pg_), cs(*pg_.cuda_), seq(pg_.next_seq()), caller(c10::cuda::getCurrentCUDAStream(dev)),
        stream(caller), serial(serial_ || pg_.options_->lanes < 2), overlap(pg_.options_->overlap_comm),
        timing(pg_.device_timing_ > 0 && (pg_.timing_tick_++ % static_cast<uint32_t>(pg_.device_timing_)) == 0),
        op_name(name), payload(bytes) {
    // a bounded device-side wait that gave up earlier poisons the group before anything new is enqueued
    if (pg.device_failed_quick()) pg.poll_device(/*must=*/true);
    pg.check_alive(name);
    nvtxRangePushA(name);  // one range per collective around its launches (visible to attached profilers)
    range_open = true;
    work = c10::make_intrusive<WorkMCCL>(pg.getRank(), op, seq, pg.profile_titles_ ? name : nullptr, std::move(outs),
                                         /*stream_mode=*/true, dev);
    pg.metrics_.op_start(seq, name, bytes);
    pg.watchdog_->watch(seq, name);
    if (overlap && serial) use_stream(cs.lanes[0]);  // temporaries of serial collectives live on lane stream 0
    skip = pg.skip_next_launch_.exchange(false);
  }

  ~CudaPath() {
    if (range_open) nvtxRangePop();
  }

  // First use of `s` by this collective: order it behind the producer and tell the allocator.
  void use_stream(c10::cuda::CUDAStream s) {
    stream = s;
    for (int i = 0; i < n_used; ++i)
      if (used[i] == s.stream()) return;
    used[n_used++] = s.stream();
    if (s != caller) {
      const auto t0 = timing ? std::chrono::steady_clock::now() : std::chrono::steady_clock::time_point();
      if (!fenced) {
        cs.fence.record(caller);
        fenced = true;
      }
      cs.fence.block(s);
      for (auto& t : kept) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), s);
      if (timing) sync_ms += ms_since(t0);
    }
    if (n_used == 1) {
      pg.metrics_.op_execute_start(seq);
      pg.watchdog_->touch(seq);
      if (timing) {
        {
          std::lock_guard<std::mutex> g(cs.pending_mu);
          ev_start = cs.get_event();
          ev_end = cs.get_event();
        }
        MCCL_CUDA_CHECK(cudaEventRecord(ev_start, s.stream()));
      }
    }
  }

  void close_epoch() {
    if (cur_lane < 0) return;
    cs.lane_last[cur_lane] = stream.stream();
    cs.lane_used[cur_lane] = true;
    cur_lane = -1;
  }

  // Takes the next epoch, selects its stream and returns the kernel parameters.
  kern::CollParams params() {
    close_epoch();
    kern::CollParams p;
    std::memset(&p, 0, sizeof(p));
    const uint32_t epoch = cs.arena->next_epoch();
    cs.arena->fill_params(p, epoch);
    const int lane = static_cast<int>(epoch % kern::kNumLanes);
    use_stream(overlap ? (serial ? cs.lanes[0] : cs.lanes[lane]) : caller);
    if (cs.lane_used[lane] && cs.lane_last[lane] != stream.stream()) {
      // the lane's previous epoch ran on another stream: order this one behind it
      MCCL_CUDA_CHECK(cudaEventRecord(cs.lane_done[lane], cs.lane_last[lane]));
      MCCL_CUDA_CHECK(cudaStreamWaitEvent(stream.stream(), cs.lane_done[lane], 0));
    }
    cur_lane = lane;
    last_epoch = epoch;
    p.scale = 1.0f;
    p.wait_ns = static_cast<unsigned long long>(pg.options_->device_wait_us) * 1000ull;
    p.tiles = static_cast<int>(pg.options_->tiles);
    p.tile_bytes = static_cast<int>(pg.options_->tile_bytes);
    p.debug_checks = pg.options_->debug_checks ? 1 : 0;
    if (!timing && !cs.stamps_always) p.ctx[0].stamps = nullptr;  // stamps are read back for timed collectives only
    if (cs.nvls) {
      p.ctx[0].nvls_uc = cs.nvls->uc();
      p.ctx[0].nvls_mc = cs.nvls->mc();
      p.nvls_offset = cs.nvls->buffer_offset(epoch);
      p.nvls_capacity = cs.nvls->buffer_bytes();
    }
    return p;
  }

  // Orders the current epoch's stream behind everything both lanes have been given so far
  // (a barrier must not complete before earlier collectives of the group).
  void wait_all_lanes() {
    for (int l = 0; l < kern::kNumLanes; ++l)
      if (cs.lane_used[l] && cs.lane_last[l] != stream.stream()) {
        MCCL_CUDA_CHECK(cudaEventRecord(cs.lane_done[l], cs.lane_last[l]));
        MCCL_CUDA_CHECK(cudaStreamWaitEvent(stream.stream(), cs.lane_done[l], 0));
      }
  }

  kern::LaunchCfg cfg(size_t bytes, bool overlapped = false) {
    kern::LaunchCfg c;
    c.ctas = pg.tuner_.ctas_for(cs.arena->world_size(), bytes, static_cast<int>(pg.options_->comm_ctas), overlapped);
    return c;
  }

  // The tensor will be touched on the communication streams this collective uses.
  void keep(const at::Tensor& t) {
    if (!t.defined() || !t.is_cuda()) return;
    kept.push_back(t);
    for (int i = 0; i < n_used; ++i)
      if (used[i] != caller.stream())
        for (auto& l : cs.lanes)
          if (l.stream() == used[i]) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), l);
  }

  c10::intrusive_ptr<c10d::Work> finish(bool blocking = false) {
    close_epoch();
    if (n_used == 0) use_stream(caller);  // nothing was launched: complete on the caller's stream
    // join: the stream of the last launch waits for the other streams this collective used
    for (int i = 0; i < n_used; ++i) {
      if (used[i] == stream.stream()) continue;
      MCCL_CUDA_CHECK(cudaEventRecord(cs.join_ev, used[i]));
      MCCL_CUDA_CHECK(cudaStreamWaitEvent(stream.stream(), cs.join_ev, 0));
    }
    if (epilogue) {
      c10::cuda::CUDAStreamGuard sg(stream);
      epilogue(stream.stream());
    }
    if (timing) {
      MCCL_CUDA_CHECK(cudaEventRecord(ev_end, stream.stream()));
      bool crowded;
      {
        std::lock_guard<std::mutex> g(cs.pending_mu);
        cs.pending.push_back({seq, ev_start, ev_end, op_name, algo, payload, bus_factor, sync_ms,
                              reducing && cs.arena && cs.arena->stamps_enabled(), last_epoch});
        crowded = cs.pending.size() > 64;
      }
      if (crowded) pg.drain_finished();  // keep the event pool small between watchdog polls
    } else {
      pg.metrics_.op_end_untimed(seq);  // counted, not part of the latency statistics
      pg.watchdog_->complete(seq);
    }
    ProcessGroupMCCL* self = &pg;
    work->set_health_check([self] { self->device_health_check(); });
    work->set_quick_check([self] { return self->device_failed_quick(); });
    if (range_open) {
      nvtxRangePop();
      range_open = false;
    }
    work->attach_stream(stream, blocking || pg.options_->blocking_wait);
    return work;
  }
};

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::staged_via_host(
    c10d::OpType op, std::vector<at::Tensor> cuda_tensors,
    std::function<c10::intrusive_ptr<c10d::Work>(std::vector<at::Tensor>&)> fn, bool copy_back) {
  std::vector<at::Tensor> host;
  for (auto& t : cuda_tensors) host.push_back(t.to(at::kCPU));
  auto w = fn(host);
  w->wait();
  if (copy_back)
    for (size_t i = 0; i < host.size(); ++i) cuda_tensors[i].copy_(host[i]);
  return completed_work(op, cuda_tensors, nullptr);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::cuda_allreduce(at::Tensor& t, c10d::ReduceOp::RedOpType op,
                                                                float prescale,
                                                                std::function<void(cudaStream_t)> epilogue,
                                                                bool overlapped) {
  const auto dev = t.device().index();
  ensure_cuda(dev);
  if (!cuda_->p2p) {
    auto w = staged_via_host(
        c10d::OpType::ALLREDUCE, {t},
        [this, op](std::vector<at::Tensor>& h) {
          c10d::AllreduceOptions o;
          o.reduceOp = op;
          return allreduce(h, o);
        },
        true);
    if (prescale != 1.0f) t.mul_(prescale);
    if (epilogue) epilogue(c10::cuda::getCurrentCUDAStream(dev).stream());
    return w;
  }
  c10::cuda::CUDAGuard guard(dev);
  const int ws = getSize();
  const kern::DType dt = to_kern_dtype(t.scalar_type());
  kern::DType wire = dt;
  const bool summing = op == c10d::ReduceOp::SUM || op == c10d::ReduceOp::AVG;
  if (dt == kern::F32 && summing) {
    if (options_->wire_dtype == "bf16") wire = kern::BF16;
    else if (options_->wire_dtype == "fp16" || options_->compression == CompressionMode::FP16) wire = kern::F16;
  }
  const size_t esz = t.element_size();
  const size_t wsz = kern::dtype_size(wire);
  const int64_t n = t.numel();
  CudaPath cp(*this, c10d::OpType::ALLREDUCE, "mccl:all_reduce", t.nbytes(), {t}, dev);
  cp.epilogue = std::move(epilogue);
  cp.keep(t);
  cp.reducing = true;
  cp.bus_factor = 2.0 * (ws - 1) / ws;

  // Tensor inside the multicast-bound pool (a DDP bucket built by wrap_ddp): reduce it in place, in
  // the switch, with no staging and a grid sized for this rank's chunk only.  With two ranks the
  // in-switch reduction moves as many bytes as the peer-memory kernels and measured slower at every
  // size (256 MiB: 750 us against 499 us), so there it is used only when the threshold is set by hand.
  const int64_t inplace_min = env_int("MCCL_NVLS_INPLACE_MIN_BYTES", ws <= 2 ? -1 : (1 << 20));
  if (cuda_->user_pool && wire == dt && kern::nvls_allreduce_supported(dt, dt, to_kern_op(op)) &&
      options_->algo != "oneshot" && options_->algo != "twoshot" && t.nbytes() % 16 == 0 &&
      (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0 &&
      inplace_min >= 0 && t.nbytes() >= static_cast<size_t>(inplace_min)) {
    NvlsUserPool& pool = NvlsUserPool::get(dev);
    if (pool.active() && pool.contains(t.data_ptr(), t.nbytes())) {
      const size_t off = pool.offset_of(t.data_ptr());
      if (!cuda_->pool_offsets_ok.count(off) && !cuda_->pool_offsets_bad.count(off)) {
        // first sight of this tensor: every rank must hold it at the same offset (same allocation
        // order everywhere); checked once through the Store, then remembered
        const auto timeout = std::chrono::milliseconds(env_int("MCCL_CONNECT_TIMEOUT_MS", 30000));
        auto all = rendezvous_->exchange("nvls_pool_off/" + std::to_string(pool_checks_++),
                                         std::to_string(off) + ":" + std::to_string(t.nbytes()), timeout);
        bool same = true;
        for (auto& v : all) same = same && v == all[0];
        if (same) cuda_->pool_offsets_ok.insert(off);
        else cuda_->pool_offsets_bad.insert(off);
      }
      if (cuda_->pool_offsets_ok.count(off)) {
        kern::CollParams p = cp.params();
        p.ctx[0].in = t.data_ptr();
        p.ctx[0].out = t.data_ptr();
        p.ctx[0].nvls_uc = pool.uc();
        p.ctx[0].nvls_mc = pool.mc();
        p.nvls_offset = off;
        p.nvls_capacity = pool.size();
        p.count = n;
        p.op = to_kern_op(op);
        p.scale = (op == c10d::ReduceOp::AVG ? 1.0f / ws : 1.0f) * prescale;
        // each rank's SMs only move its own chunk (the switch does the fan-in and fan-out): a small grid.
        // Measured on 4 ranks, 94 M MLP under DDP: 88.1 k samples/s with 16 CTAs, 86.9 k with 32, 81.6 k with 64.
        // MCCL_NVLS_INPLACE_CTAS_ALONE: the grid when the caller says nothing overlaps (default: the same).
        kern::LaunchCfg lc = cp.cfg(t.nbytes() / ws, overlapped);
        const int64_t grid_cap = env_int("MCCL_NVLS_INPLACE_CTAS", 16);
        lc.ctas = std::min<int>(lc.ctas, static_cast<int>(overlapped ? grid_cap : env_int("MCCL_NVLS_INPLACE_CTAS_ALONE", grid_cap)));
        if (!cp.skip) MCCL_LAUNCH_CHECK(kern::launch_allreduce_nvls_inplace(p, dt, lc, cp.stream.stream()));
        cp.algo = "nvls-inplace";
        const uint64_t sent = t.nbytes() + t.nbytes() / ws;
        metrics_.record_transport_bytes(sent, sent);
        return cp.finish();
      }
    }
  }

  const int cls = wsz <= 2 ? 1 : 0;
  const bool nvls_ok = cuda_->nvls != nullptr && kern::nvls_allreduce_supported(dt, wire, to_kern_op(op)) &&
                       options_->algo != "oneshot" && options_->algo != "twoshot";
  // Segment so that every launch fits one parity buffer (and one NVLS buffer when that path is taken).
  const size_t cap = cuda_->arena->parity_bytes();
  size_t seg_bytes = std::min(tuner_.segment_bytes(), cap * ws / (ws + 1));
  const bool whole_nvls = nvls_ok && (options_->algo == "nvls" ||
                                      tuner_.choose_allreduce(ws, static_cast<size_t>(n) * wsz, cls, true) == Variant::NVLS);
  if (whole_nvls) seg_bytes = std::min(seg_bytes, cuda_->nvls->buffer_bytes() / 4096 * 4096);
  int64_t seg_elems = static_cast<int64_t>(seg_bytes / wsz);
  seg_elems = std::max<int64_t>(seg_elems / 256 * 256, 256);
  char* base = static_cast<char*>(t.data_ptr());
  uint64_t sent = 0;
  for (int64_t off = 0; off < n; off += seg_elems) {
    const int64_t cnt = std::min(seg_elems, n - off);
    const size_t wire_bytes = static_cast<size_t>(cnt) * wsz;
    Variant v = tuner_.choose_allreduce(ws, wire_bytes, cls, nvls_ok);
    if (options_->algo == "oneshot") v = Variant::ONESHOT;
    if (options_->algo == "twoshot") v = Variant::TWOSHOT;
    if (options_->algo == "nvls" && nvls_ok) v = Variant::NVLS;
    if (v == Variant::NVLS && kern::nvls_allreduce_stage_bytes(wire_bytes, ws) > cuda_->nvls->buffer_bytes()) v = Variant::TWOSHOT;
    if (v == Variant::ONESHOT && kern::oneshot_arena_bytes(wire_bytes, ws) > cap) v = Variant::TWOSHOT;
    MCCL_CHECK(v == Variant::NVLS || kern::twoshot_arena_bytes(wire_bytes, ws) <= cap, "segment does not fit the arena");
    bool push = options_->gather == "push" || (options_->gather == "auto" && tuner_.push_gather(ws));
    if (push && kern::twoshot_arena_bytes(wire_bytes, ws, true) > cap) push = false;
    kern::CollParams p = cp.params();
    p.push_gather = push ? 1 : 0;
    p.ctx[0].in = base + off * esz;
    p.ctx[0].out = base + off * esz;
    p.count = cnt;
    p.op = to_kern_op(op);
    p.scale = (op == c10d::ReduceOp::AVG ? 1.0f / ws : 1.0f) * prescale;
    if (v == Variant::NVLS && p.tile_bytes == 0) p.tile_bytes = tuner_.nvls_tile_bytes();
    const int64_t split_min = options_->nvls_split_min_bytes >= -1 ? options_->nvls_split_min_bytes : tuner_.nvls_split_min_bytes();
    const bool nvls_split = v == Variant::NVLS && split_min >= 0 && static_cast<int64_t>(wire_bytes) >= split_min;
    if (!cp.skip) {
      if (v == Variant::ONESHOT)
        MCCL_LAUNCH_CHECK(kern::launch_allreduce_oneshot(p, dt, wire, cp.cfg(wire_bytes * (ws - 1), overlapped), cp.stream.stream()));
      else if (v == Variant::NVLS)
        MCCL_LAUNCH_CHECK(kern::launch_allreduce_nvls(p, dt, wire, cp.cfg(wire_bytes, overlapped), cp.stream.stream(), nvls_split));
      else
        MCCL_LAUNCH_CHECK(kern::launch_allreduce_twoshot(p, dt, wire, cp.cfg(wire_bytes, overlapped), cp.stream.stream()));
    }
    cp.algo = nvls_split ? "nvls-split" : variant_name(v);
    sent += v == Variant::ONESHOT ? wire_bytes * (ws - 1)
            : v == Variant::NVLS  ? wire_bytes + wire_bytes / ws
                                  : 2 * wire_bytes * (ws - 1) / ws;
    MCCL_DEBUG("allreduce seq=%u epoch=%u %s bytes=%zu wire=%d", cp.seq, p.seq, variant_name(v), wire_bytes, int(wire));
  }
  metrics_.record_transport_bytes(sent, sent);
  return cp.finish();
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::cuda_broadcast(at::Tensor& t, int root) {
  const auto dev = t.device().index();
  ensure_cuda(dev);
  if (!cuda_->p2p) {
    return staged_via_host(
        c10d::OpType::BROADCAST, {t},
        [this, root](std::vector<at::Tensor>& h) {
          c10d::BroadcastOptions o;
          o.rootRank = root;
          return broadcast(h, o);
        },
        getRank() != root);
  }
  c10::cuda::CUDAGuard guard(dev);
  CudaPath cp(*this, c10d::OpType::BROADCAST, "mccl:broadcast", t.nbytes(), {t}, dev);
  cp.keep(t);
  const int ws = getSize();
  const size_t nbytes = t.nbytes();
  const bool nvls = cuda_->nvls != nullptr && options_->algo != "oneshot" && options_->algo != "twoshot" &&
                    (options_->algo == "nvls" || tuner_.broadcast_nvls(ws, nbytes));
  const size_t cap = (nvls ? std::min(cuda_->arena->parity_bytes(), cuda_->nvls->buffer_bytes()) : cuda_->arena->parity_bytes()) / 256 * 256;
  char* base = static_cast<char*>(t.data_ptr());
  for (size_t off = 0; off < nbytes; off += cap) {
    const size_t cnt = std::min(cap, nbytes - off);
    kern::CollParams p = cp.params();
    p.ctx[0].in = base + off;
    p.ctx[0].out = base + off;
    p.count = static_cast<int64_t>(cnt);
    p.root = root;
    p.use_nvls = nvls ? 1 : 0;
    if (p.tile_bytes == 0) p.tile_bytes = tuner_.mover_tile_bytes();
    if (!cp.skip) MCCL_LAUNCH_CHECK(kern::launch_broadcast(p, cp.cfg(cnt), cp.stream.stream()));
  }
  cp.algo = nvls ? "nvls" : (ws == 2 || nbytes <= (256u << 10)) ? "direct" : "twohop";
  if (getRank() == root) metrics_.record_transport_bytes(nbytes, 0);
  else metrics_.record_transport_bytes(nvls ? 0 : nbytes * (ws - 2) / (ws - 1), nbytes);
  return cp.finish();
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::cuda_allgather(at::Tensor& out_flat, const at::Tensor& in,
                                                                std::vector<at::Tensor>* scatter_to) {
  const auto dev = in.device().index();
  ensure_cuda(dev);
  const int ws = getSize();
  if (!cuda_->p2p) {
    at::Tensor hin = in.to(at::kCPU);
    std::vector<at::Tensor> houts;
    for (int r = 0; r < ws; ++r) houts.push_back(at::empty_like(hin));
    std::vector<std::vector<at::Tensor>> ol{houts};
    std::vector<at::Tensor> il{hin};
    allgather(ol, il)->wait();
    for (int r = 0; r < ws; ++r) {
      if (scatter_to) (*scatter_to)[r].copy_(ol[0][r]);
      else out_flat.narrow(0, r * in.numel(), in.numel()).copy_(ol[0][r].reshape({-1}));
    }
    return completed_work(c10d::OpType::ALLGATHER, scatter_to ? *scatter_to : std::vector<at::Tensor>{out_flat}, nullptr);
  }
  c10::cuda::CUDAGuard guard(dev);
  std::vector<at::Tensor> outs = scatter_to ? *scatter_to : std::vector<at::Tensor>{out_flat};
  // with a temporary that is scattered afterwards everything stays on one stream; otherwise the
  // slices of a large gather alternate lanes like the segments of a large allreduce
  CudaPath cp(*this, c10d::OpType::ALLGATHER, "mccl:all_gather", in.nbytes() * ws, outs, dev, /*serial=*/scatter_to != nullptr);
  at::Tensor flat = out_flat;
  if (scatter_to) {
    c10::cuda::CUDAStreamGuard sg(cp.stream);  // temporary belongs to the stream that uses it
    flat = at::empty({static_cast<int64_t>(ws) * in.numel()}, in.options());
  }
  cp.keep(in);
  cp.keep(flat);
  cp.bus_factor = static_cast<double>(ws - 1) / ws;
  const size_t nbytes = in.nbytes();
  const bool nvls = cuda_->nvls != nullptr && options_->algo != "oneshot" && options_->algo != "twoshot" &&
                    (options_->algo == "nvls" || tuner_.allgather_nvls(ws, nbytes));
  // one launch stages ws blocks in every rank's staging buffer: larger blocks go slice by slice, each
  // slice landing at its final place (the kernel takes the distance between ranks' blocks in `out`)
  const size_t stage = nvls ? std::min(cuda_->arena->parity_bytes(), cuda_->nvls->buffer_bytes()) : cuda_->arena->parity_bytes();
  const size_t cap = std::max<size_t>((stage / ws) / 256 * 256, 256);
  const char* ibase = static_cast<const char*>(in.data_ptr());
  char* obase = static_cast<char*>(flat.data_ptr());
  for (size_t off = 0; off < nbytes; off += cap) {
    const size_t cnt = std::min(cap, nbytes - off);
    kern::CollParams p = cp.params();
    p.ctx[0].in = ibase + off;
    p.ctx[0].out = obase + off;
    p.count = static_cast<int64_t>(cnt);
    p.out_pitch = static_cast<int64_t>(nbytes);
    p.use_nvls = nvls ? 1 : 0;
    if (p.tile_bytes == 0) p.tile_bytes = tuner_.mover_tile_bytes();
    MCCL_CHECK(kern::allgather_stage_bytes(cnt, ws) <= stage, "allgather slice does not fit the staging buffer");
    if (!cp.skip) MCCL_LAUNCH_CHECK(kern::launch_allgather(p, cp.cfg(cnt * ws), cp.stream.stream()));
  }
  cp.algo = nvls ? "nvls-push" : "push";
  if (scatter_to) {
    c10::cuda::CUDAStreamGuard sg(cp.stream);
    for (int r = 0; r < ws; ++r) {
      cp.keep((*scatter_to)[r]);
      (*scatter_to)[r].reshape({-1}).copy_(flat.narrow(0, r * in.numel(), in.numel()), /*non_blocking=*/true);
    }
  }
  metrics_.record_transport_bytes(nbytes * (ws - 1), nbytes * (ws - 1));
  return cp.finish();
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::cuda_reduce_scatter(at::Tensor& out, const at::Tensor& in_flat,
                                                                     c10d::ReduceOp::RedOpType op) {
  const auto dev = out.device().index();
  ensure_cuda(dev);
  const int ws = getSize();
  if (!cuda_->p2p) {
    at::Tensor hin = in_flat.to(at::kCPU);
    at::Tensor hout = at::empty({out.numel()}, hin.options());
    c10d::ReduceScatterOptions o;
    o.reduceOp = op;
    _reduce_scatter_base(hout, hin, o)->wait();
    out.reshape({-1}).copy_(hout);
    return completed_work(c10d::OpType::REDUCE_SCATTER, {out}, nullptr);
  }
  c10::cuda::CUDAGuard guard(dev);
  const kern::DType dt = to_kern_dtype(out.scalar_type());
  const size_t esz = out.element_size();
  const int64_t n = out.numel();
  CudaPath cp(*this, c10d::OpType::REDUCE_SCATTER, "mccl:reduce_scatter", in_flat.nbytes(), {out}, dev);
  cp.keep(in_flat);
  cp.keep(out);
  cp.algo = "push";
  cp.reducing = true;
  cp.bus_factor = static_cast<double>(ws - 1) / ws;
  const size_t cap = cuda_->arena->parity_bytes();
  // slot = one chunk slice; ws slots per parity buffer.  Chunks larger than a slot go in slices:
  // launch i reduces elements [off, off + cnt) of every chunk, reading them in place (chunk q
  // starts at in + q * n: the kernel's chunk pitch), and consecutive launches alternate lanes.
  int64_t seg_elems = static_cast<int64_t>(std::min(tuner_.segment_bytes(), cap) / ws / esz) / 256 * 256;
  seg_elems = std::max<int64_t>(seg_elems, 256);
  const char* ibase = static_cast<const char*>(in_flat.data_ptr());
  char* obase = static_cast<char*>(out.data_ptr());
  for (int64_t off = 0; off < n; off += seg_elems) {
    const int64_t cnt = std::min(seg_elems, n - off);
    kern::CollParams p = cp.params();
    p.ctx[0].in = ibase + off * esz;
    p.ctx[0].out = obase + off * esz;
    p.count = cnt;
    p.chunk_pitch = n;
    p.op = to_kern_op(op);
    p.scale = op == c10d::ReduceOp::AVG ? 1.0f / ws : 1.0f;
    if (!cp.skip) MCCL_LAUNCH_CHECK(kern::launch_reduce_scatter(p, dt, dt, cp.cfg(cnt * esz * ws), cp.stream.stream()));
  }
  metrics_.record_transport_bytes(out.nbytes() * (ws - 1), out.nbytes() * (ws - 1));
  return cp.finish();
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::cuda_barrier() {
  const auto dev = cuda_->dev;
  c10::cuda::CUDAGuard guard(dev);
  CudaPath cp(*this, c10d::OpType::BARRIER, "mccl:barrier", 0, {}, dev);
  cp.algo = "flags";
  kern::CollParams p = cp.params();
  cp.wait_all_lanes();
  if (!cp.skip) MCCL_LAUNCH_CHECK(kern::launch_barrier(p, kern::LaunchCfg{}, cp.stream.stream()));
  return cp.finish(/*blocking=*/true);
}

// ---------------------------------------------------------------------------
// Fused top-k compressed allreduce (select -> sparse allgather -> scatter-add
// with error feedback).  Semantics: standard sparse allgather, identical dense
// result on every rank (the reference's 2-rank path mixed a decompressed peer
// with an uncompressed local tensor: reference
// csrc/backend/ProcessGroupMCCL.cpp:1692-1708; not reproduced).
// ---------------------------------------------------------------------------
c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::allreduce_topk(at::Tensor& grad, at::Tensor& residual, double ratio,
                                                                float scale) {
  check_alive("allreduce_topk");
  check_tensor(grad, "allreduce_topk");
  MCCL_CHECK_TENSOR(grad.is_cuda(), "allreduce_topk: CUDA tensors only");
  MCCL_CHECK_TENSOR(grad.scalar_type() == at::kFloat || grad.scalar_type() == at::kBFloat16,
                    "allreduce_topk: float32 or bfloat16 gradients");
  MCCL_CHECK_TENSOR(residual.is_cuda() && residual.scalar_type() == at::kFloat && residual.is_contiguous() &&
                        residual.numel() == grad.numel(),
                    "allreduce_topk: residual must be a float32 CUDA tensor of the gradient's size");
  MCCL_CHECK_TENSOR(ratio > 0.0 && ratio <= 1.0, "allreduce_topk: ratio must be in (0, 1]");
  const auto dev = grad.device().index();
  const int ws = getSize();
  const int64_t n = grad.numel();
  MCCL_CHECK_TENSOR(n > 0 && n < (int64_t(1) << 31), "allreduce_topk: element count out of range");
  const bool bf16 = grad.scalar_type() == at::kBFloat16;
  c10::cuda::CUDAGuard guard(dev);

  if (ws > 1) ensure_cuda(dev);
  const bool p2p = ws > 1 && cuda_ && cuda_->p2p;
  MCCL_CHECK(ws == 1 || p2p, "allreduce_topk needs the NVLink peer data plane (" << data_plane() << ")");
  auto k_for = [ratio](int64_t cnt) {
    int64_t k = std::max<int64_t>(1, static_cast<int64_t>(std::floor(static_cast<double>(cnt) * ratio)));
    return std::min(k, cnt);
  };
  // One exchange stages ws lists of k pairs in every rank's arena buffer.  A bucket whose lists do not
  // fit is cut into equal segments, each selected and exchanged on its own (top-k per segment).
  int64_t seg = n;
  if (p2p) {
    const size_t cap = cuda_->arena->parity_bytes();
    while (kern::topk_pad(static_cast<size_t>(k_for(seg)) * 8) * ws > cap) seg = (seg / 2 + 1023) / 1024 * 1024;
    MCCL_CHECK(seg >= 1024, "top-k payload cannot be made to fit the arena");
  }

  cudaStream_t stream;
  std::unique_ptr<CudaPath> cp;
  at::Tensor scratch, pairs;
  if (p2p) {
    cp = std::make_unique<CudaPath>(*this, c10d::OpType::ALLREDUCE, "mccl:all_reduce_topk",
                                    static_cast<uint64_t>(k_for(n)) * 8 * ws, std::vector<at::Tensor>{grad}, dev,
                                    /*serial=*/true);
    stream = cp->stream.stream();  // serial collectives run on lane stream 0 (or the caller's stream)
    cp->keep(grad);
    cp->keep(residual);
    cp->algo = "topk";
    cp->bus_factor = static_cast<double>(ws - 1);
  } else {
    stream = c10::cuda::getCurrentCUDAStream(dev).stream();
  }
  {
    // scratch: radix histograms + counters; pairs: this rank's (idx,val) list of the largest segment
    c10::cuda::CUDAStreamGuard sg(p2p ? cp->stream : c10::cuda::getCurrentCUDAStream(dev));
    scratch = at::empty({static_cast<int64_t>(kern::topk_scratch_bytes())}, grad.options().dtype(at::kByte));
    pairs = at::empty({k_for(std::min(seg, n)) * 2}, grad.options().dtype(at::kInt));
  }
  const size_t gsz = grad.element_size();
  uint64_t sent = 0;
  for (int64_t off = 0; off < n; off += seg) {
    const int64_t cnt = std::min(seg, n - off);
    const int64_t k = k_for(cnt);
    kern::TopkArgs a;
    a.grad = static_cast<char*>(grad.data_ptr()) + off * gsz;
    a.grad_is_bf16 = bf16;
    a.residual = residual.data_ptr<float>() + off;
    a.n = cnt;
    a.k = k;
    a.scratch = scratch.data_ptr();
    a.pairs = pairs.data_ptr();
    a.scale = scale;
    if (!(cp && cp->skip)) MCCL_LAUNCH_CHECK(kern::launch_topk_select(a, stream));
    if (p2p) {
      kern::CollParams p = cp->params();
      p.ctx[0].in = pairs.data_ptr();
      p.ctx[0].out = const_cast<void*>(a.grad);
      p.count = k;
      p.scale = scale;
      if (!cp->skip) MCCL_LAUNCH_CHECK(kern::launch_topk_exchange_scatter(p, a, cp->cfg(static_cast<size_t>(k) * 8 * ws), stream));
      sent += static_cast<uint64_t>(k) * 8 * (ws - 1);
    } else {
      MCCL_LAUNCH_CHECK(kern::launch_topk_local_scatter(a, stream));
    }
  }
  if (p2p) {
    metrics_.record_transport_bytes(sent, sent);
    return cp->finish();
  }
  return completed_work(c10d::OpType::ALLREDUCE, {grad}, nullptr);
}

}  // namespace mccl
