#include "backend/process_group.h"

#include <c10/util/irange.h>

#include <algorithm>
#include <cstring>

#include "backend/tensor_checks.h"
#include "common/env.h"
#include "common/log.h"
#include "cpu/reduce.h"
#include "p2p/nccl_p2p.h"
#include "runtime/mempool.h"

namespace mccl {

// c10d::OpType names the collective kind; wire::OpType is the frame-header op code.
namespace wire = ::mccl;

// ---------------------------------------------------------------------------
// active group (module-level metrics accessors)
// ---------------------------------------------------------------------------
static std::mutex g_pg_mu;
static ProcessGroupMCCL* g_active_pg = nullptr;

void set_active_pg(ProcessGroupMCCL* pg) {
  std::lock_guard<std::mutex> g(g_pg_mu);
  g_active_pg = pg;
}
void clear_active_pg(ProcessGroupMCCL* pg) {
  std::lock_guard<std::mutex> g(g_pg_mu);
  if (g_active_pg == pg) g_active_pg = nullptr;
}
ProcessGroupMCCL* active_pg_locked(std::unique_lock<std::mutex>& lk) {
  lk = std::unique_lock<std::mutex>(g_pg_mu);
  return g_active_pg;
}

c10::intrusive_ptr<ProcessGroupMCCL> createProcessGroupMCCL(
    const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, std::chrono::milliseconds timeout) {
  auto opts = MCCLOptions::from_env(timeout);
  return c10::make_intrusive<ProcessGroupMCCL>(store, rank, size, opts);
}

// ---------------------------------------------------------------------------
// construction / teardown
// ---------------------------------------------------------------------------
ProcessGroupMCCL::ProcessGroupMCCL(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                                   c10::intrusive_ptr<MCCLOptions> options)
    : c10d::Backend(rank, size), store_(store), options_(std::move(options)) {
  MCCL_CHECK(size >= 1 && rank >= 0 && rank < size, "bad rank/size " << rank << "/" << size);
  MCCL_TRACE("ctor: begin");
  if (std::getenv("MCCL_SYNC_MODE"))
    MCCL_WARN("MCCL_SYNC_MODE was removed: ordering is always stream/event based");
  if (std::getenv("MCCL_ALLREDUCE_ALGO"))
    MCCL_WARN("MCCL_ALLREDUCE_ALGO was removed: use MCCL_ALGO (auto|oneshot|twoshot|staged)");

  if (options_->gather != "auto" && options_->gather != "pull" && options_->gather != "push") {
    MCCL_WARN("MCCL_GATHER=%s is not one of auto|pull|push: using auto", options_->gather.c_str());
    options_->gather = "auto";
  }
  if (options_->algo != "auto" && options_->algo != "oneshot" && options_->algo != "twoshot" && options_->algo != "nvls" &&
      options_->algo != "staged") {
    MCCL_WARN("MCCL_ALGO=%s is not one of auto|oneshot|twoshot|nvls|staged: using auto", options_->algo.c_str());
    options_->algo = "auto";
  }
  device_timing_ = static_cast<int>(std::max<int64_t>(0, env_int("MCCL_DEVICE_TIMING", 8)));
  profile_titles_ = env_bool("MCCL_PROFILE_TITLES", false);
  compressor_ = make_compressor(options_->compression, options_->topk_ratio);
  std::string tune = env_str("MCCL_TUNE_FILE", "");
  if (!tune.empty()) {
    int n = tuner_.load(tune);
    MCCL_INFO("tuner: %d fields loaded from %s", n, tune.c_str());
  }
  if (env_int("MCCL_SEGMENT_BYTES", 0) >= (1 << 20)) tuner_.set_segment_bytes(static_cast<size_t>(env_int("MCCL_SEGMENT_BYTES", 0)));
  if (options_->oneshot_max_bytes >= 0)
    for (int ws = 0; ws <= kern::kMaxWorld; ++ws)
      tuner_.set_oneshot_max_bytes(ws, static_cast<size_t>(options_->oneshot_max_bytes));
  if (options_->nvls_min_bytes >= -1)
    for (int ws = 0; ws <= kern::kMaxWorld; ++ws) tuner_.set_nvls_min_bytes(ws, options_->nvls_min_bytes);
  if (env_int("MCCL_OVERLAP_CTAS", -1) >= 0)  // grid cap of collectives that share the GPU with backward (DDP buckets)
    for (int ws = 0; ws <= kern::kMaxWorld; ++ws) tuner_.set_ctas_overlap(ws, static_cast<int>(env_int("MCCL_OVERLAP_CTAS", 0)));
  if (options_->comm_ctas > kern::kMaxCtasPerLane) {
    MCCL_WARN("MCCL_COMM_CTAS=%lld exceeds the %d CTAs one lane may use (two lanes must stay co-resident): clamped",
              (long long)options_->comm_ctas, kern::kMaxCtasPerLane);
    options_->comm_ctas = kern::kMaxCtasPerLane;
  }

  MCCL_TRACE("ctor: tuner ok");
  rendezvous_ = std::make_unique<Rendezvous>(store_, rank, size);
  collective_engine_ = std::make_unique<HostEngine>("mccl_engine", 1, static_cast<size_t>(options_->max_queue_depth));
  p2p_engine_ = std::make_unique<HostEngine>("mccl_p2p", 2, static_cast<size_t>(options_->max_queue_depth));

  watchdog_ = std::make_unique<Watchdog>(
      options_->watchdog_timeout,
      [this](uint32_t seq, const std::string& msg) {
        metrics_.record_error();
        poison(msg + " (seq " + std::to_string(seq) + ")", /*tell_peers=*/true);
      });
  MCCL_TRACE("ctor: engines+watchdog ok");
  watchdog_->set_poll_hook([this] { poll_device(); });
  watchdog_->start();
  MCCL_TRACE("ctor: watchdog started");

  if (size > 1 && env_str("MCCL_HOST_TRANSPORT", "eager") != "lazy") ensure_transport();

  if (size > 1) {
    health_ = std::make_unique<HealthMonitor>(
        rank, size, options_->heartbeat_interval,
        [this](int peer) {
          std::lock_guard<std::mutex> g(transport_init_mu_);
          return !transport_ || transport_->is_peer_connected(peer);
        },
        [this](int peer) {
          if (shut_down_.load()) return;
          metrics_.record_error();
          poison("rank " + std::to_string(peer) + " is no longer reachable", /*tell_peers=*/false);
        },
        [this] {
          std::lock_guard<std::mutex> g(transport_init_mu_);
          if (transport_) transport_->send_heartbeat();
        });
    health_->start();
  }

  MCCL_TRACE("ctor: before describe");
  MCCL_INFO("%s", describe().c_str());
  set_active_pg(this);
}

ProcessGroupMCCL::~ProcessGroupMCCL() { shutdown(); }

std::string ProcessGroupMCCL::describe() const {
  std::ostringstream o;
  o << "ProcessGroupMCCL rank " << getRank() << "/" << getSize() << " algo=" << options_->algo
    << " overlap_comm=" << options_->overlap_comm << " arena=" << (options_->arena_bytes >> 20) << "MiB x4"
    << " oneshot_max(ws)=" << tuner_.oneshot_max_bytes(std::min(getSize(), kern::kMaxWorld))
    << " segment=" << (tuner_.segment_bytes() >> 20) << "MiB"
    << " lanes=" << options_->lanes << " comm_ctas=" << options_->comm_ctas << " nvls=" << options_->nvls
    << " wire_dtype=" << options_->wire_dtype
    << " compression=" << (compressor_ ? compressor_->name() : std::string("none"))
    << " topk_ratio=" << options_->topk_ratio << " watchdog_ms=" << options_->watchdog_timeout.count()
    << " heartbeat_ms=" << options_->heartbeat_interval.count()
    << " device_wait_us=" << options_->device_wait_us << " chunk_bytes=" << options_->chunk_bytes
    << " small_msg_threshold=" << options_->small_msg_threshold << " crc=" << options_->transport_crc
    << " (no effect on CUDA: fast_math=" << options_->fast_math << " gpu_threshold=" << options_->gpu_threshold
    << ")";
  return o.str();
}

void ProcessGroupMCCL::shutdown() {
  bool e = false;
  if (!shut_down_.compare_exchange_strong(e, true)) return;
  clear_active_pg(this);
  if (log_enabled(LogLevel::INFO)) metrics_.log_summary();
  if (health_) health_->stop();
  if (watchdog_) watchdog_->stop();
  if (collective_engine_) collective_engine_->shutdown();
  if (p2p_engine_) p2p_engine_->shutdown();
  {
    std::lock_guard<std::mutex> g(transport_init_mu_);
    if (transport_) transport_->shutdown();
  }
  abort_all_inflight("process group shut down");
  {
    std::lock_guard<std::mutex> g(nccl_mu_);
    if (nccl_p2p_) nccl_p2p_->shutdown();
    nccl_p2p_.reset();
  }
  release_nvls();
  arena_quick_.store(nullptr, std::memory_order_release);
  cuda_.reset();
}

void ProcessGroupMCCL::abort() {
  poison("abort() called", /*tell_peers=*/true);
}

std::string ProcessGroupMCCL::poison_reason() const {
  std::lock_guard<std::mutex> g(poison_mu_);
  return poison_reason_;
}

void ProcessGroupMCCL::poison(const std::string& why, bool tell_peers) {
  bool first = false;
  {
    std::lock_guard<std::mutex> g(poison_mu_);
    if (!poisoned_.load()) {
      poison_reason_ = why;
      poisoned_.store(true);
      first = true;
    }
  }
  if (!first) return;
  MCCL_ERROR("rank %d: process group failed: %s", getRank(), why.c_str());
  if (tell_peers) {
    std::lock_guard<std::mutex> g(transport_init_mu_);
    if (transport_) transport_->send_abort(why);
  }
  abort_all_inflight(why);
}

void ProcessGroupMCCL::check_alive(const char* what) {
  if (shut_down_.load()) throw MCCLError(std::string(what) + ": process group is shut down");
  if (poisoned_.load())
    throw MCCLError(std::string(what) + ": process group is in a failed state (" + poison_reason() +
                    "); destroy it and create a new one");
}

void ProcessGroupMCCL::register_work(const c10::intrusive_ptr<WorkMCCL>& w) {
  std::lock_guard<std::mutex> g(works_mu_);
  works_.emplace(w->seq(), c10::weak_intrusive_ptr<WorkMCCL>(w));
}
void ProcessGroupMCCL::unregister_work(uint32_t seq) {
  std::lock_guard<std::mutex> g(works_mu_);
  works_.erase(seq);
}
void ProcessGroupMCCL::abort_all_inflight(const std::string& why) {
  std::vector<c10::intrusive_ptr<WorkMCCL>> live;
  {
    std::lock_guard<std::mutex> g(works_mu_);
    for (auto& kv : works_) {
      auto s = kv.second.lock();
      if (s) live.push_back(std::move(s));
    }
    works_.clear();
  }
  for (auto& w : live)
    if (!w->stream_mode()) w->mark_error(why);
  std::lock_guard<std::mutex> g(transport_init_mu_);
  if (transport_ && !transport_->aborted()) {
    // unblock engine threads waiting in wait_recv
    for (auto& w : live) transport_->cancel_recvs(w->seq());
  }
}

c10::intrusive_ptr<WorkMCCL> ProcessGroupMCCL::completed_work(c10d::OpType op, std::vector<at::Tensor> outs,
                                                              const at::Tensor* like) {
  (void)like;
  // Results on a CUDA device need a CUDA-aware future (a plain future refuses
  // CUDA tensors): complete it on the caller's current stream, no kernel involved.
  for (auto& t : outs) {
    if (t.defined() && t.is_cuda()) {
      const auto dev = t.device().index();
      auto w = c10::make_intrusive<WorkMCCL>(getRank(), op, collective_seq_.load(), "mccl:noop", outs,
                                             /*stream_mode=*/true, dev);
      w->attach_stream(c10::cuda::getCurrentCUDAStream(dev), false);
      return w;
    }
  }
  auto w = c10::make_intrusive<WorkMCCL>(getRank(), op, collective_seq_.load(), "mccl:noop", std::move(outs),
                                         /*stream_mode=*/false, 0);
  w->mark_complete();
  return w;
}

Metrics::Summary ProcessGroupMCCL::get_metrics_summary() {
  poll_device();
  {
    std::lock_guard<std::mutex> g(transport_init_mu_);
    (void)g;
  }
  return metrics_.summarize();
}
void ProcessGroupMCCL::log_metrics() {
  poll_device();
  Metrics::Summary s = metrics_.summarize();
  // Always printed: the caller asked for it explicitly.
  std::lock_guard<std::mutex> g(log_mutex());
  std::fprintf(stderr,
               "[MCCL INFO metrics] ops=%llu sent=%llu recv=%llu errors=%llu avg=%.3fms p50=%.3fms p99=%.3fms "
               "peak=%.2fGbps sync=%.3fms net=%.3fms reduce=%.3fms queue=%.3fms exec=%.3fms\n",
               (unsigned long long)s.total_ops, (unsigned long long)s.total_bytes_sent,
               (unsigned long long)s.total_bytes_recv, (unsigned long long)s.total_errors, s.avg_latency_ms,
               s.p50_latency_ms, s.p99_latency_ms, s.peak_throughput_gbps, s.avg_sync_ms, s.avg_network_ms,
               s.avg_reduce_ms, s.avg_queue_wait_ms, s.avg_execution_ms);
}
void ProcessGroupMCCL::reset_metrics() { metrics_.reset(); }

// ---------------------------------------------------------------------------
// host transport bring-up
// ---------------------------------------------------------------------------
void ProcessGroupMCCL::ensure_transport() {
  std::lock_guard<std::mutex> g(transport_init_mu_);
  if (transport_ || getSize() == 1) return;
  TransportConfig cfg = TransportConfig::from_env();
  cfg.chunk_bytes = static_cast<size_t>(std::max<int64_t>(options_->chunk_bytes, 1));
  cfg.crc = options_->transport_crc;
  if (!options_->listen_addr.empty()) cfg.listen_addr = options_->listen_addr;
  if (!options_->ifname.empty()) cfg.ifname = options_->ifname;
  if (options_->port_base > 0) cfg.port_base = static_cast<int>(options_->port_base);
  if (options_->transport == "rdma")
    MCCL_WARN("transport=rdma: no verbs transport on this platform (GPU data goes over NVLink peer memory); "
              "using tcp for the host plane");
  auto t = std::make_unique<HostTransport>(getRank(), getSize(), cfg);
  t->on_peer_failure = [this](int peer, const std::string& why) {
    if (shut_down_.load()) return;
    metrics_.record_error();
    // Runs on a reader thread: poison without touching transport_init_mu_ re-entrantly.
    bool first = false;
    {
      std::lock_guard<std::mutex> pg(poison_mu_);
      if (!poisoned_.load()) {
        poison_reason_ = "rank " + std::to_string(peer) + ": " + why;
        poisoned_.store(true);
        first = true;
      }
    }
    if (first) {
      MCCL_ERROR("rank %d: peer %d failed: %s", getRank(), peer, why.c_str());
      std::vector<c10::intrusive_ptr<WorkMCCL>> live;
      {
        std::lock_guard<std::mutex> wg(works_mu_);
        for (auto& kv : works_) {
          auto s = kv.second.lock();
          if (s) live.push_back(std::move(s));
        }
      }
      // Receives posted to other (healthy) peers would otherwise wait for their timeout.
      for (auto& w : live)
        if (transport_) transport_->cancel_recvs(w->seq());
    }
  };
  auto timeout = std::chrono::milliseconds(cfg.connect_timeout_ms);
  auto endpoints = rendezvous_->exchange("endpoint", t->listen_endpoint(), timeout);
  t->connect_all(endpoints);
  transport_ = std::move(t);
}

// ---------------------------------------------------------------------------
// host-side submission
// ---------------------------------------------------------------------------
c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::submit_host(c10d::OpType op, const char* name, uint64_t bytes,
                                                             std::vector<at::Tensor> outs,
                                                             std::function<void(uint32_t)> body,
                                                             HostEngine* engine) {
  const bool p2p = engine != nullptr;
  const uint32_t seq = p2p ? (0x80000000u | (++p2p_seq_)) : next_seq();
  // p2p operations do not take a collective sequence number on the wire (ranks
  // issue different p2p calls); the id above is only a local handle.
  auto work = c10::make_intrusive<WorkMCCL>(getRank(), op, seq, name, std::move(outs), false, 0);
  register_work(work);
  watchdog_->watch(seq, name);
  metrics_.op_start(seq, name, bytes);
  HostEngine* eng = engine ? engine : collective_engine_.get();
  eng->submit(
      [this, seq, body] {
        watchdog_->touch(seq);
        metrics_.op_execute_start(seq);
        if (poisoned_.load()) throw MCCLError("process group is in a failed state (" + poison_reason() + ")");
        body(seq);
      },
      [this, seq, work] {
        unregister_work(seq);
        watchdog_->complete(seq);
        metrics_.op_end(seq);
        work->mark_complete();
      },
      [this, seq, work](const std::string& err) {
        unregister_work(seq);
        watchdog_->complete(seq);
        metrics_.record_error();
        metrics_.op_end(seq);
        work->mark_error(err);
      });
  return work;
}

// ---------------------------------------------------------------------------
// CPU algorithms
// ---------------------------------------------------------------------------
namespace {

struct PhaseTimer {
  Metrics& m;
  uint32_t seq;
  Metrics::Phase ph;
  std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
  ~PhaseTimer() {
    m.record_phase(seq, ph, std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count());
  }
};

}  // namespace

void ProcessGroupMCCL::cpu_allreduce(uint32_t seq, at::Tensor& t, c10d::ReduceOp::RedOpType op) {
  const int ws = getSize(), me = getRank();
  const int64_t n = t.numel();
  const size_t esz = t.element_size();
  const size_t nbytes = static_cast<size_t>(n) * esz;
  const auto dtype = t.scalar_type();
  uint8_t* data = static_cast<uint8_t*>(t.data_ptr());
  auto& pool = staging_memory_pool();
  const wire::OpType wop = wire::OpType::ALLREDUCE;

  const bool compressed = compressor_ && (dtype == at::kFloat || (dtype == at::kHalf && compressor_->mode() == CompressionMode::FP16)) &&
                          (op == c10d::ReduceOp::SUM || op == c10d::ReduceOp::AVG);
  if (compressor_ && !compressed && dtype == at::kBFloat16)
    throw TensorError("compression is not supported for bfloat16 CPU tensors");

  if (compressed) {
    // Sparse/half all-exchange: every rank broadcasts its compressed
    // contribution; everyone decompresses all ws contributions (its own
    // included) and sums them in rank order.
    const WireDType wd = to_wire_dtype(dtype);
    const size_t cap = compressor_->max_compressed_size(nbytes, wd);
    const uint64_t stable_id = reinterpret_cast<uint64_t>(t.storage().data()) + t.storage_offset() * esz;
    PooledBuffer mine = pool.acquire(cap);
    size_t csz;
    {
      PhaseTimer pt{metrics_, seq, Metrics::Phase::REDUCE};
      csz = compressor_->compress(data, nbytes, mine.data(), cap, wd, stable_id);
    }
    std::vector<PooledBuffer> bufs(ws);
    std::vector<HostTransport::TicketPtr> tk(ws);
    std::vector<size_t> got(ws, 0);
    {
      PhaseTimer pt{metrics_, seq, Metrics::Phase::NETWORK};
      for (int r = 0; r < ws; ++r) {
        if (r == me) continue;
        bufs[r] = pool.acquire(cap);
        tk[r] = transport_->post_recv(r, HostTransport::collective_key(seq, 0), bufs[r].data(), cap);
      }
      for (int d = 1; d < ws; ++d) {
        int r = (me + d) % ws;
        transport_->send(r, wop, seq, 0, mine.data(), csz, FLAG_COMPRESSED);
      }
      for (int r = 0; r < ws; ++r)
        if (r != me) got[r] = transport_->wait_recv(tk[r]);
    }
    PhaseTimer pt{metrics_, seq, Metrics::Phase::REDUCE};
    PooledBuffer tmp = pool.acquire(nbytes);
    for (int r = 0; r < ws; ++r) {
      const void* src = r == me ? mine.data() : bufs[r].data();
      size_t sz = r == me ? csz : got[r];
      if (r == 0) {
        compressor_->decompress(src, sz, data, nbytes, wd);
      } else {
        compressor_->decompress(src, sz, tmp.data(), nbytes, wd);
        cpu_reduce_into(data, tmp.data(), n, dtype, c10d::ReduceOp::SUM);
      }
    }
    if (op == c10d::ReduceOp::AVG) cpu_scale_inplace(data, n, dtype, 1.0 / ws);
    metrics_.record_transport_bytes(csz * (ws - 1), 0);
    return;
  }

  constexpr size_t kPairSegment = size_t(2) << 20;
  if (ws == 2 && nbytes >= 2 * kPairSegment) {
    // Two ranks, large message: exchange in segments and reduce segment i-1 while segment i is on
    // the wire (both directions run at the same rate, so it has arrived by then).  Same bytes as the
    // plain exchange, but the reduction no longer follows the transfer.
    const int peer = 1 - me;
    const int64_t seg_elems = static_cast<int64_t>(kPairSegment / esz);
    const int nseg = static_cast<int>((n + seg_elems - 1) / seg_elems);
    PooledBuffer theirs = pool.acquire(nbytes);
    std::vector<HostTransport::TicketPtr> tk(nseg);
    auto seg_len = [&](int i) { return std::min<int64_t>(seg_elems, n - static_cast<int64_t>(i) * seg_elems); };
    for (int i = 0; i < nseg; ++i)
      tk[i] = transport_->post_recv(peer, HostTransport::collective_key(seq, 16 + i),
                                    theirs.data() + static_cast<size_t>(i) * seg_elems * esz, seg_len(i) * esz);
    auto finish_seg = [&](int i) {
      {
        PhaseTimer pt{metrics_, seq, Metrics::Phase::NETWORK};
        transport_->wait_recv(tk[i]);
      }
      PhaseTimer pt{metrics_, seq, Metrics::Phase::REDUCE};
      uint8_t* d = data + static_cast<size_t>(i) * seg_elems * esz;
      cpu_reduce_into(d, theirs.data() + static_cast<size_t>(i) * seg_elems * esz, seg_len(i), dtype, op);
      if (op == c10d::ReduceOp::AVG) cpu_scale_inplace(d, seg_len(i), dtype, 0.5);
    };
    for (int i = 0; i < nseg; ++i) {
      {
        PhaseTimer pt{metrics_, seq, Metrics::Phase::NETWORK};
        transport_->send(peer, wop, seq, 16 + i, data + static_cast<size_t>(i) * seg_elems * esz, seg_len(i) * esz);
      }
      if (i >= 1) finish_seg(i - 1);  // segment i-1 of `data` has been sent: safe to overwrite
    }
    finish_seg(nseg - 1);
    metrics_.record_transport_bytes(nbytes, nbytes);
    return;
  }

  if (ws == 2 || nbytes <= static_cast<size_t>(options_->small_msg_threshold)) {
    // All-exchange: (ws-1)*N on the wire per rank, one round.
    std::vector<PooledBuffer> bufs(ws);
    std::vector<HostTransport::TicketPtr> tk(ws);
    {
      PhaseTimer pt{metrics_, seq, Metrics::Phase::NETWORK};
      for (int r = 0; r < ws; ++r) {
        if (r == me) continue;
        bufs[r] = pool.acquire(nbytes);
        tk[r] = transport_->post_recv(r, HostTransport::collective_key(seq, 0), bufs[r].data(), nbytes);
      }
      for (int d = 1; d < ws; ++d) transport_->send((me + d) % ws, wop, seq, 0, data, nbytes);
      for (int r = 0; r < ws; ++r)
        if (r != me) transport_->wait_recv(tk[r]);
    }
    PhaseTimer pt{metrics_, seq, Metrics::Phase::REDUCE};
    // Fixed rank order: acc = x0 op x1 op ... ; `data` holds x_me.  With two ranks the
    // operation is a single elementwise op that gives the same bits for either operand order
    // (IEEE add and mul are commutative; MIN / MAX are made so in cpu/reduce.cpp: NaNs propagate
    // as the canonical NaN and -0 orders below +0), so both ranks reduce in place without the
    // reordering copies.
    if (ws == 2) {
      cpu_reduce_into(data, bufs[1 - me].data(), n, dtype, op);
    } else if (me != 0) {
      PooledBuffer mine = pool.acquire(nbytes);
      std::memcpy(mine.data(), data, nbytes);
      std::memcpy(data, bufs[0].data(), nbytes);
      for (int r = 1; r < ws; ++r)
        cpu_reduce_into(data, r == me ? mine.data() : bufs[r].data(), n, dtype, op);
    } else {
      for (int r = 1; r < ws; ++r) cpu_reduce_into(data, bufs[r].data(), n, dtype, op);
    }
    if (op == c10d::ReduceOp::AVG) cpu_scale_inplace(data, n, dtype, 1.0 / ws);
    metrics_.record_transport_bytes(nbytes * (ws - 1), nbytes * (ws - 1));
    return;
  }

  // Two-shot: chunk c is reduced by rank c, then distributed.
  const int64_t chunk = (n + ws - 1) / ws;
  auto cbeg = [&](int c) { return std::min<int64_t>(n, static_cast<int64_t>(c) * chunk); };
  auto clen = [&](int c) { return cbeg(c + 1) - cbeg(c); };
  const int64_t my_n = clen(me);
  std::vector<PooledBuffer> parts(ws);
  std::vector<HostTransport::TicketPtr> tk(ws);
  {
    PhaseTimer pt{metrics_, seq, Metrics::Phase::NETWORK};
    for (int r = 0; r < ws; ++r) {
      if (r == me || my_n == 0) continue;
      parts[r] = pool.acquire(my_n * esz);
      tk[r] = transport_->post_recv(r, HostTransport::collective_key(seq, 0), parts[r].data(), my_n * esz);
    }
    for (int d = 1; d < ws; ++d) {
      int r = (me + d) % ws;
      if (clen(r) > 0) transport_->send(r, wop, seq, 0, data + cbeg(r) * esz, clen(r) * esz);
    }
    for (int r = 0; r < ws; ++r)
      if (tk[r]) transport_->wait_recv(tk[r]);
  }
  if (my_n > 0) {
    PhaseTimer pt{metrics_, seq, Metrics::Phase::REDUCE};
    uint8_t* mine = data + cbeg(me) * esz;
    if (me != 0) {
      PooledBuffer own = pool.acquire(my_n * esz);
      std::memcpy(own.data(), mine, my_n * esz);
      std::memcpy(mine, parts[0].data(), my_n * esz);
      for (int r = 1; r < ws; ++r) cpu_reduce_into(mine, r == me ? own.data() : parts[r].data(), my_n, dtype, op);
    } else {
      for (int r = 1; r < ws; ++r) cpu_reduce_into(mine, parts[r].data(), my_n, dtype, op);
    }
    if (op == c10d::ReduceOp::AVG) cpu_scale_inplace(mine, my_n, dtype, 1.0 / ws);
  }
  {
    PhaseTimer pt{metrics_, seq, Metrics::Phase::NETWORK};
    std::vector<HostTransport::TicketPtr> tk2(ws);
    for (int r = 0; r < ws; ++r) {
      if (r == me || clen(r) == 0) continue;
      tk2[r] = transport_->post_recv(r, HostTransport::collective_key(seq, 1), data + cbeg(r) * esz, clen(r) * esz);
    }
    if (my_n > 0)
      for (int d = 1; d < ws; ++d) transport_->send((me + d) % ws, wop, seq, 1, data + cbeg(me) * esz, my_n * esz);
    for (int r = 0; r < ws; ++r)
      if (tk2[r]) transport_->wait_recv(tk2[r]);
  }
  metrics_.record_transport_bytes(2 * (nbytes - my_n * esz), 2 * (nbytes - my_n * esz));
}

void ProcessGroupMCCL::cpu_broadcast(uint32_t seq, at::Tensor& t, int root) {
  const int ws = getSize(), me = getRank();
  const size_t nbytes = t.nbytes();
  uint8_t* data = static_cast<uint8_t*>(t.data_ptr());
  const wire::OpType wop = wire::OpType::BROADCAST;
  PhaseTimer pt{metrics_, seq, Metrics::Phase::NETWORK};
  if (ws <= 3 || nbytes <= static_cast<size_t>(options_->small_msg_threshold)) {
    if (me == root) {
      for (int d = 1; d < ws; ++d) transport_->send((me + d) % ws, wop, seq, 0, data, nbytes);
      metrics_.record_transport_bytes(nbytes * (ws - 1), 0);
    } else {
      auto tk = transport_->post_recv(root, HostTransport::collective_key(seq, 0), data, nbytes);
      transport_->wait_recv(tk);
      metrics_.record_transport_bytes(0, nbytes);
    }
    return;
  }
  // Scatter + allgather among the ws-1 non-root ranks: the root sends each byte once.
  const int nr = ws - 1;
  auto idx_of = [&](int r) { return r < root ? r : r - 1; };  // non-root index
  auto rank_of = [&](int i) { return i < root ? i : i + 1; };
  const size_t slice = (nbytes + nr - 1) / nr;
  auto sbeg = [&](int i) { return std::min(nbytes, static_cast<size_t>(i) * slice); };
  auto slen = [&](int i) { return sbeg(i + 1) - sbeg(i); };
  if (me == root) {
    for (int i = 0; i < nr; ++i)
      if (slen(i) > 0) transport_->send(rank_of(i), wop, seq, 0, data + sbeg(i), slen(i));
    metrics_.record_transport_bytes(nbytes, 0);
    return;
  }
  const int mi = idx_of(me);
  std::vector<HostTransport::TicketPtr> tk(nr);
  for (int i = 0; i < nr; ++i) {
    if (i == mi || slen(i) == 0) continue;
    tk[i] = transport_->post_recv(rank_of(i), HostTransport::collective_key(seq, 1), data + sbeg(i), slen(i));
  }
  if (slen(mi) > 0) {
    auto t0 = transport_->post_recv(root, HostTransport::collective_key(seq, 0), data + sbeg(mi), slen(mi));
    transport_->wait_recv(t0);
    for (int d = 1; d < nr; ++d) {
      int i = (mi + d) % nr;
      transport_->send(rank_of(i), wop, seq, 1, data + sbeg(mi), slen(mi));
    }
  }
  for (int i = 0; i < nr; ++i)
    if (tk[i]) transport_->wait_recv(tk[i]);
  metrics_.record_transport_bytes(slen(mi) * (nr - 1), nbytes);
}

void ProcessGroupMCCL::cpu_allgather(uint32_t seq, std::vector<at::Tensor>& outs, const at::Tensor& in) {
  const int ws = getSize(), me = getRank();
  const size_t nbytes = in.nbytes();
  PhaseTimer pt{metrics_, seq, Metrics::Phase::NETWORK};
  std::vector<HostTransport::TicketPtr> tk(ws);
  for (int r = 0; r < ws; ++r) {
    if (r == me) continue;
    tk[r] = transport_->post_recv(r, HostTransport::collective_key(seq, 0), outs[r].data_ptr(), nbytes);
  }
  for (int d = 1; d < ws; ++d) transport_->send((me + d) % ws, wire::OpType::ALLGATHER, seq, 0, in.data_ptr(), nbytes);
  if (outs[me].data_ptr() != in.data_ptr()) std::memcpy(outs[me].data_ptr(), in.data_ptr(), nbytes);
  for (int r = 0; r < ws; ++r)
    if (tk[r]) transport_->wait_recv(tk[r]);
  metrics_.record_transport_bytes(nbytes * (ws - 1), nbytes * (ws - 1));
}

void ProcessGroupMCCL::cpu_reduce_scatter(uint32_t seq, at::Tensor& out, std::vector<at::Tensor>& ins,
                                          c10d::ReduceOp::RedOpType op) {
  const int ws = getSize(), me = getRank();
  const size_t nbytes = out.nbytes();
  const int64_t n = out.numel();
  const auto dtype = out.scalar_type();
  auto& pool = staging_memory_pool();
  std::vector<PooledBuffer> parts(ws);
  std::vector<HostTransport::TicketPtr> tk(ws);
  {
    PhaseTimer pt{metrics_, seq, Metrics::Phase::NETWORK};
    for (int r = 0; r < ws; ++r) {
      if (r == me) continue;
      parts[r] = pool.acquire(nbytes);
      tk[r] = transport_->post_recv(r, HostTransport::collective_key(seq, 0), parts[r].data(), nbytes);
    }
    for (int d = 1; d < ws; ++d) {
      int r = (me + d) % ws;
      transport_->send(r, wire::OpType::REDUCE_SCATTER, seq, 0, ins[r].data_ptr(), nbytes);
    }
    for (int r = 0; r < ws; ++r)
      if (tk[r]) transport_->wait_recv(tk[r]);
  }
  PhaseTimer pt{metrics_, seq, Metrics::Phase::REDUCE};
  // rank order, with ins[me] standing in at position `me`
  PooledBuffer acc = pool.acquire(nbytes);
  std::memcpy(acc.data(), me == 0 ? ins[0].data_ptr() : parts[0].data(), nbytes);
  for (int r = 1; r < ws; ++r)
    cpu_reduce_into(acc.data(), r == me ? ins[me].data_ptr() : parts[r].data(), n, dtype, op);
  if (op == c10d::ReduceOp::AVG) cpu_scale_inplace(acc.data(), n, dtype, 1.0 / ws);
  std::memcpy(out.data_ptr(), acc.data(), nbytes);
  metrics_.record_transport_bytes(nbytes * (ws - 1), nbytes * (ws - 1));
}

void ProcessGroupMCCL::cpu_reduce(uint32_t seq, at::Tensor& t, int root, c10d::ReduceOp::RedOpType op) {
  const int ws = getSize(), me = getRank();
  const size_t nbytes = t.nbytes();
  const int64_t n = t.numel();
  const auto dtype = t.scalar_type();
  auto& pool = staging_memory_pool();
  if (me != root) {
    PhaseTimer pt{metrics_, seq, Metrics::Phase::NETWORK};
    transport_->send(root, wire::OpType::ALLREDUCE, seq, 0, t.data_ptr(), nbytes);
    metrics_.record_transport_bytes(nbytes, 0);
    return;
  }
  std::vector<PooledBuffer> parts(ws);
  std::vector<HostTransport::TicketPtr> tk(ws);
  {
    PhaseTimer pt{metrics_, seq, Metrics::Phase::NETWORK};
    for (int r = 0; r < ws; ++r) {
      if (r == me) continue;
      parts[r] = pool.acquire(nbytes);
      tk[r] = transport_->post_recv(r, HostTransport::collective_key(seq, 0), parts[r].data(), nbytes);
    }
    for (int r = 0; r < ws; ++r)
      if (tk[r]) transport_->wait_recv(tk[r]);
  }
  PhaseTimer pt{metrics_, seq, Metrics::Phase::REDUCE};
  PooledBuffer acc = pool.acquire(nbytes);
  std::memcpy(acc.data(), me == 0 ? t.data_ptr() : parts[0].data(), nbytes);
  for (int r = 1; r < ws; ++r) cpu_reduce_into(acc.data(), r == me ? t.data_ptr() : parts[r].data(), n, dtype, op);
  if (op == c10d::ReduceOp::AVG) cpu_scale_inplace(acc.data(), n, dtype, 1.0 / ws);
  std::memcpy(t.data_ptr(), acc.data(), nbytes);
  metrics_.record_transport_bytes(0, nbytes * (ws - 1));
}

// ---------------------------------------------------------------------------
// public collective entry points
// ---------------------------------------------------------------------------
c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::allreduce(std::vector<at::Tensor>& tensors,
                                                           const c10d::AllreduceOptions& opts) {
  check_alive("allreduce");
  check_single(tensors, "allreduce");
  at::Tensor& t = tensors[0];
  const auto op = static_cast<c10d::ReduceOp::RedOpType>(opts.reduceOp);
  check_reduce_op(op, t.scalar_type());
  if (t.numel() == 0 || getSize() == 1) return completed_work(c10d::OpType::ALLREDUCE, {t}, &t);
  if (t.is_cuda()) return cuda_allreduce(t, op, 1.0f);
  ensure_transport();
  at::Tensor tt = t;
  return submit_host(c10d::OpType::ALLREDUCE, "mccl:all_reduce", t.nbytes(), {t},
                     [this, tt, op](uint32_t seq) mutable { cpu_allreduce(seq, tt, op); });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::allreduce_scaled(std::vector<at::Tensor>& tensors, float scale) {
  check_alive("allreduce_scaled");
  check_single(tensors, "allreduce_scaled");
  at::Tensor& t = tensors[0];
  MCCL_CHECK_TENSOR(t.is_floating_point(), "allreduce_scaled: floating-point tensors only");
  if (t.numel() == 0) return completed_work(c10d::OpType::ALLREDUCE, {t}, &t);
  if (getSize() == 1) {
    if (scale != 1.0f) t.mul_(scale);
    return completed_work(c10d::OpType::ALLREDUCE, {t}, &t);
  }
  // gradient buckets from a DDP hook: they overlap the rest of backward
  if (t.is_cuda()) return cuda_allreduce(t, c10d::ReduceOp::SUM, scale, nullptr, /*overlapped=*/true);
  ensure_transport();
  at::Tensor tt = t;
  return submit_host(c10d::OpType::ALLREDUCE, "mccl:all_reduce_scaled", t.nbytes(), {t},
                     [this, tt, scale](uint32_t seq) mutable {
                       cpu_allreduce(seq, tt, c10d::ReduceOp::SUM);
                       cpu_scale_inplace(tt.data_ptr(), tt.numel(), tt.scalar_type(), scale);
                     });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::allreduce_scaled_then(std::vector<at::Tensor>& tensors, float scale,
                                                                       std::function<void(cudaStream_t)> epilogue,
                                                                       bool overlapped) {
  check_alive("allreduce_scaled_then");
  check_single(tensors, "allreduce_scaled_then");
  at::Tensor& t = tensors[0];
  MCCL_CHECK_TENSOR(t.is_cuda() && t.is_floating_point(), "allreduce_scaled_then: floating-point CUDA tensors only");
  if (getSize() == 1 || t.numel() == 0) {
    if (scale != 1.0f && t.numel() > 0) t.mul_(scale);
    if (epilogue) epilogue(c10::cuda::getCurrentCUDAStream(t.device().index()).stream());
    return completed_work(c10d::OpType::ALLREDUCE, {t}, &t);
  }
  return cuda_allreduce(t, c10d::ReduceOp::SUM, scale, std::move(epilogue), overlapped);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::allreduce_coalesced(
    std::vector<at::Tensor>& tensors, const c10d::AllreduceCoalescedOptions& opts) {
  check_alive("allreduce_coalesced");
  MCCL_CHECK_TENSOR(!tensors.empty(), "allreduce_coalesced: empty tensor list");
  for (auto& t : tensors) {
    check_tensor(t, "allreduce_coalesced");
    MCCL_CHECK_TENSOR(t.scalar_type() == tensors[0].scalar_type() && t.device() == tensors[0].device(),
                      "allreduce_coalesced: tensors must share dtype and device");
  }
  const auto op = static_cast<c10d::ReduceOp::RedOpType>(opts.reduceOp);
  check_reduce_op(op, tensors[0].scalar_type());
  if (getSize() == 1) return completed_work(c10d::OpType::ALLREDUCE_COALESCED, tensors, nullptr);
  // Flatten -> one allreduce -> scatter back.  On CUDA the copies are ordered on
  // the caller's stream and the result is copied back once the collective's
  // event has been waited for.
  std::vector<at::Tensor> flat_parts;
  for (auto& t : tensors) flat_parts.push_back(t.reshape({-1}));
  at::Tensor flat = at::cat(flat_parts);
  std::vector<at::Tensor> one{flat};
  c10d::AllreduceOptions ao;
  ao.reduceOp = opts.reduceOp;
  auto inner = allreduce(one, ao);
  inner->wait();
  int64_t off = 0;
  for (auto& t : tensors) {
    t.reshape({-1}).copy_(flat.narrow(0, off, t.numel()));
    off += t.numel();
  }
  return completed_work(c10d::OpType::ALLREDUCE_COALESCED, tensors, nullptr);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::reduce(std::vector<at::Tensor>& tensors,
                                                        const c10d::ReduceOptions& opts) {
  check_alive("reduce");
  check_single(tensors, "reduce");
  at::Tensor& t = tensors[0];
  const auto op = static_cast<c10d::ReduceOp::RedOpType>(opts.reduceOp);
  check_reduce_op(op, t.scalar_type());
  const int root = static_cast<int>(opts.rootRank);
  MCCL_CHECK_TENSOR(root >= 0 && root < getSize(), "reduce: bad root " << root);
  if (t.numel() == 0 || getSize() == 1) return completed_work(c10d::OpType::REDUCE, {t}, &t);
  if (t.is_cuda()) {
    // Every rank computes the reduction; only the root keeps it.
    if (getRank() == root) return cuda_allreduce(t, op, 1.0f);
    at::Tensor scratch = t.clone();
    auto w = cuda_allreduce(scratch, op, 1.0f);
    return w;
  }
  ensure_transport();
  at::Tensor tt = t;
  return submit_host(c10d::OpType::REDUCE, "mccl:reduce", t.nbytes(), {t},
                     [this, tt, root, op](uint32_t seq) mutable { cpu_reduce(seq, tt, root, op); });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::broadcast(std::vector<at::Tensor>& tensors,
                                                           const c10d::BroadcastOptions& opts) {
  check_alive("broadcast");
  check_single(tensors, "broadcast");
  at::Tensor& t = tensors[0];
  const int root = static_cast<int>(opts.rootRank);
  MCCL_CHECK_TENSOR(root >= 0 && root < getSize(), "broadcast: bad root " << root);
  if (t.numel() == 0 || getSize() == 1) return completed_work(c10d::OpType::BROADCAST, {t}, &t);
  if (t.is_cuda()) return cuda_broadcast(t, root);
  ensure_transport();
  at::Tensor tt = t;
  return submit_host(c10d::OpType::BROADCAST, "mccl:broadcast", t.nbytes(), {t},
                     [this, tt, root](uint32_t seq) mutable { cpu_broadcast(seq, tt, root); });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::allgather(std::vector<std::vector<at::Tensor>>& outputs,
                                                           std::vector<at::Tensor>& inputs,
                                                           const c10d::AllgatherOptions&) {
  check_alive("allgather");
  check_single(inputs, "allgather");
  MCCL_CHECK_TENSOR(outputs.size() == 1, "allgather: expected one output list");
  auto& outs = outputs[0];
  MCCL_CHECK_TENSOR(static_cast<int>(outs.size()) == getSize(),
                    "allgather: output list must hold world_size tensors, got " << outs.size());
  at::Tensor& in = inputs[0];
  for (auto& o : outs) {
    check_tensor(o, "allgather");
    check_same(o, in, "allgather");
  }
  if (getSize() == 1) {
    if (outs[0].data_ptr() != in.data_ptr()) outs[0].copy_(in);
    return completed_work(c10d::OpType::ALLGATHER, outs, &in);
  }
  if (in.numel() == 0) return completed_work(c10d::OpType::ALLGATHER, outs, &in);
  if (in.is_cuda()) {
    // Contiguous output list (views of one flat buffer) gathers in place;
    // otherwise gather into a flat temporary and scatter on the comm stream.
    bool flat_ok = true;
    const char* base = static_cast<const char*>(outs[0].data_ptr());
    for (int r = 0; r < getSize(); ++r)
      if (static_cast<const char*>(outs[r].data_ptr()) != base + static_cast<size_t>(r) * in.nbytes()) flat_ok = false;
    if (flat_ok) {
      at::Tensor flat = at::from_blob(outs[0].data_ptr(), {static_cast<int64_t>(getSize()) * in.numel()},
                                      in.options());
      auto w = cuda_allgather(flat, in, nullptr);
      return w;
    }
    at::Tensor none;
    return cuda_allgather(none, in, &outs);
  }
  ensure_transport();
  std::vector<at::Tensor> o = outs;
  at::Tensor i = in;
  return submit_host(c10d::OpType::ALLGATHER, "mccl:all_gather", in.nbytes() * getSize(), outs,
                     [this, o, i](uint32_t seq) mutable { cpu_allgather(seq, o, i); });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::_allgather_base(at::Tensor& output, at::Tensor& input,
                                                                 const c10d::AllgatherOptions&) {
  check_alive("_allgather_base");
  check_tensor(input, "_allgather_base");
  check_tensor(output, "_allgather_base");
  MCCL_CHECK_TENSOR(output.scalar_type() == input.scalar_type() && output.device() == input.device(),
                    "_allgather_base: dtype/device mismatch");
  MCCL_CHECK_TENSOR(output.numel() == input.numel() * getSize(),
                    "_allgather_base: output must hold world_size * input elements");
  if (getSize() == 1) {
    if (output.data_ptr() != input.data_ptr()) output.reshape({-1}).copy_(input.reshape({-1}));
    return completed_work(c10d::OpType::_ALLGATHER_BASE, {output}, &input);
  }
  if (input.numel() == 0) return completed_work(c10d::OpType::_ALLGATHER_BASE, {output}, &input);
  if (input.is_cuda()) {
    at::Tensor flat = output.reshape({-1});
    return cuda_allgather(flat, input, nullptr);
  }
  ensure_transport();
  std::vector<at::Tensor> outs;
  at::Tensor flat = output.reshape({-1});
  for (int r = 0; r < getSize(); ++r) outs.push_back(flat.narrow(0, r * input.numel(), input.numel()));
  at::Tensor i = input;
  return submit_host(c10d::OpType::_ALLGATHER_BASE, "mccl:_all_gather_base", output.nbytes(), {output},
                     [this, outs, i](uint32_t seq) mutable { cpu_allgather(seq, outs, i); });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::allgather_into_tensor_coalesced(
    std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs, const c10d::AllgatherOptions& opts) {
  MCCL_CHECK_TENSOR(outputs.size() == inputs.size(), "allgather_into_tensor_coalesced: list size mismatch");
  c10::intrusive_ptr<c10d::Work> last;
  for (size_t i = 0; i < inputs.size(); ++i) last = _allgather_base(outputs[i], inputs[i], opts);
  if (!last) return completed_work(c10d::OpType::ALLGATHER_COALESCED, {}, nullptr);
  return last;  // same stream / same engine: the last work completes after all the others
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::reduce_scatter(std::vector<at::Tensor>& outputs,
                                                                std::vector<std::vector<at::Tensor>>& inputs,
                                                                const c10d::ReduceScatterOptions& opts) {
  check_alive("reduce_scatter");
  check_single(outputs, "reduce_scatter");
  MCCL_CHECK_TENSOR(inputs.size() == 1, "reduce_scatter: expected one input list");
  auto& ins = inputs[0];
  MCCL_CHECK_TENSOR(static_cast<int>(ins.size()) == getSize(),
                    "reduce_scatter: input list must hold world_size tensors, got " << ins.size());
  at::Tensor& out = outputs[0];
  for (auto& i : ins) {
    check_tensor(i, "reduce_scatter");
    check_same(i, out, "reduce_scatter");
  }
  const auto op = static_cast<c10d::ReduceOp::RedOpType>(opts.reduceOp);
  check_reduce_op(op, out.scalar_type());
  if (getSize() == 1) {
    if (out.data_ptr() != ins[0].data_ptr()) out.copy_(ins[0]);
    return completed_work(c10d::OpType::REDUCE_SCATTER, {out}, &out);
  }
  if (out.numel() == 0) return completed_work(c10d::OpType::REDUCE_SCATTER, {out}, &out);
  if (out.is_cuda()) {
    std::vector<at::Tensor> parts;
    for (auto& i : ins) parts.push_back(i.reshape({-1}));
    at::Tensor flat = at::cat(parts);
    return cuda_reduce_scatter(out, flat, op);
  }
  ensure_transport();
  at::Tensor o = out;
  std::vector<at::Tensor> iv = ins;
  return submit_host(c10d::OpType::REDUCE_SCATTER, "mccl:reduce_scatter", out.nbytes() * getSize(), {out},
                     [this, o, iv, op](uint32_t seq) mutable { cpu_reduce_scatter(seq, o, iv, op); });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::_reduce_scatter_base(at::Tensor& output, at::Tensor& input,
                                                                      const c10d::ReduceScatterOptions& opts) {
  check_alive("_reduce_scatter_base");
  check_tensor(input, "_reduce_scatter_base");
  check_tensor(output, "_reduce_scatter_base");
  MCCL_CHECK_TENSOR(output.scalar_type() == input.scalar_type() && output.device() == input.device(),
                    "_reduce_scatter_base: dtype/device mismatch");
  MCCL_CHECK_TENSOR(input.numel() == output.numel() * getSize(),
                    "_reduce_scatter_base: input must hold world_size * output elements");
  const auto op = static_cast<c10d::ReduceOp::RedOpType>(opts.reduceOp);
  check_reduce_op(op, output.scalar_type());
  if (getSize() == 1) {
    if (output.data_ptr() != input.data_ptr()) output.reshape({-1}).copy_(input.reshape({-1}));
    return completed_work(c10d::OpType::_REDUCE_SCATTER_BASE, {output}, &output);
  }
  if (output.numel() == 0) return completed_work(c10d::OpType::_REDUCE_SCATTER_BASE, {output}, &output);
  if (output.is_cuda()) {
    at::Tensor flat = input.reshape({-1});
    return cuda_reduce_scatter(output, flat, op);
  }
  ensure_transport();
  std::vector<at::Tensor> ins;
  at::Tensor flat = input.reshape({-1});
  for (int r = 0; r < getSize(); ++r) ins.push_back(flat.narrow(0, r * output.numel(), output.numel()));
  at::Tensor o = output.reshape({-1});
  return submit_host(c10d::OpType::_REDUCE_SCATTER_BASE, "mccl:_reduce_scatter_base", input.nbytes(), {output},
                     [this, o, ins, op](uint32_t seq) mutable {
                       std::vector<at::Tensor> iv = ins;
                       cpu_reduce_scatter(seq, o, iv, op);
                     });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::reduce_scatter_tensor_coalesced(
    std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs, const c10d::ReduceScatterOptions& opts) {
  MCCL_CHECK_TENSOR(outputs.size() == inputs.size(), "reduce_scatter_tensor_coalesced: list size mismatch");
  c10::intrusive_ptr<c10d::Work> last;
  for (size_t i = 0; i < inputs.size(); ++i) last = _reduce_scatter_base(outputs[i], inputs[i], opts);
  if (!last) return completed_work(c10d::OpType::REDUCE_SCATTER, {}, nullptr);
  return last;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::barrier(const c10d::BarrierOptions&) {
  check_alive("barrier");
  if (getSize() == 1) return completed_work(c10d::OpType::BARRIER, {}, nullptr);
  if (data_plane() == "nvlink-p2p") return cuda_barrier();
  // Store barrier, ordered behind earlier CPU collectives on the engine.
  auto timeout = options_->watchdog_timeout;
  return submit_host(c10d::OpType::BARRIER, "mccl:barrier", 0, {},
                     [this, timeout](uint32_t) { rendezvous_->barrier("pg", timeout); });
}

NcclP2P* ProcessGroupMCCL::ensure_nccl_p2p() {
  if (env_str("MCCL_P2P", "nccl") == "host") return nullptr;
  std::lock_guard<std::mutex> g(nccl_mu_);
  if (!nccl_p2p_) {
    try {
      nccl_p2p_ = std::make_shared<NcclP2P>(store_, getRank(), getSize(), options_->timeout);
    } catch (const std::exception& e) {
      MCCL_WARN("NCCL p2p unavailable (%s); CUDA send/recv are staged through host memory", e.what());
      return nullptr;
    }
  }
  return nccl_p2p_.get();
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::send(std::vector<at::Tensor>& tensors, int dst, int tag) {
  check_alive("send");
  check_single(tensors, "send");
  MCCL_CHECK_TENSOR(dst >= 0 && dst < getSize() && dst != getRank(), "send: bad destination rank " << dst);
  at::Tensor t = tensors[0];
  if (t.numel() == 0) return completed_work(c10d::OpType::SEND, {t}, &t);  // zero-size: no wire traffic
  if (t.is_cuda()) {
    if (NcclP2P* p2p = ensure_nccl_p2p()) {
      metrics_.record_transport_bytes(t.nbytes(), 0);
      return p2p->send(tensors, dst, tag);
    }
  }
  ensure_transport();
  at::Tensor host = t;
  if (t.is_cuda()) host = t.to(at::kCPU);  // synchronous device->host copy on the caller's stream
  return submit_host(c10d::OpType::SEND, "mccl:send", t.nbytes(), {t},
                     [this, host, dst, tag](uint32_t) {
                       transport_->send(dst, wire::OpType::SEND, 0, static_cast<uint32_t>(tag), host.data_ptr(),
                                        host.nbytes());
                       metrics_.record_transport_bytes(host.nbytes(), 0);
                     },
                     p2p_engine_.get());
}

c10::intrusive_ptr<c10d::Work> ProcessGroupMCCL::recv(std::vector<at::Tensor>& tensors, int src, int tag) {
  check_alive("recv");
  check_single(tensors, "recv");
  MCCL_CHECK_TENSOR(src >= 0 && src < getSize() && src != getRank(), "recv: bad source rank " << src);
  at::Tensor t = tensors[0];
  if (t.numel() == 0) return completed_work(c10d::OpType::RECV, {t}, &t);
  if (t.is_cuda()) {
    if (NcclP2P* p2p = ensure_nccl_p2p()) {
      metrics_.record_transport_bytes(0, t.nbytes());
      return p2p->recv(tensors, src, tag);
    }
  }
  ensure_transport();
  if (t.is_cuda()) {
    // Host-staged: receive into pinned memory, then copy to the device.
    at::Tensor host = at::empty(t.sizes(), t.options().device(at::kCPU).pinned_memory(true));
    auto tk = transport_->post_recv(src, HostTransport::p2p_key(static_cast<uint32_t>(tag)), host.data_ptr(),
                                    host.nbytes());
    at::Tensor dev = t;
    auto w = submit_host(c10d::OpType::RECV, "mccl:recv", t.nbytes(), {t},
                         [this, host, dev, tk](uint32_t) mutable {
                           size_t got = transport_->wait_recv(tk);
                           MCCL_CHECK(got == host.nbytes(), "recv: size mismatch " << got << " vs " << host.nbytes());
                           dev.copy_(host, /*non_blocking=*/false);
                           metrics_.record_transport_bytes(0, got);
                         },
                         p2p_engine_.get());
    return w;
  }
  // Post now so a message that is already in flight lands in the user buffer.
  auto tk = transport_->post_recv(src, HostTransport::p2p_key(static_cast<uint32_t>(tag)), t.data_ptr(), t.nbytes());
  const size_t want = t.nbytes();
  return submit_host(c10d::OpType::RECV, "mccl:recv", t.nbytes(), {t},
                     [this, tk, want](uint32_t) {
                       size_t got = transport_->wait_recv(tk);
                       MCCL_CHECK(got == want, "recv: size mismatch " << got << " vs " << want);
                       metrics_.record_transport_bytes(0, got);
                     },
                     p2p_engine_.get());
}

}  // namespace mccl
