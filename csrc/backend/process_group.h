// ProcessGroupMCCL: the c10d Backend registered as "mccl".
//
// CUDA tensors: collectives are single fused kernels (csrc/kernels/collectives.cu)
// launched stream-ordered on a high-priority communication stream.  The
// producer stream is fenced with an event before the launch, the Work carries
// an event recorded after it, and a CUDA-aware Future orders DDP's reducer.
// Peers' memory is reached through the SymmetricArena; the variant (one-shot /
// two-shot) comes from the Tuner's size table.  If peer mapping is impossible
// (ranks on different hosts, more than 8 ranks, no P2P) all ranks agree to stage
// through host memory and use the CPU algorithms instead.
//
// CPU tensors: algorithms run on HostEngine workers over the HostTransport
// (framed TCP mesh) with reductions in fixed rank order, so results are
// bit-identical on every rank.  dist.barrier() on a CPU-only group is an
// epoch-keyed Store barrier.
//
// Services: Watchdog (deadlines armed at execution start; also polls the device
// status block written by bounded in-kernel waits), HealthMonitor (peer
// liveness: transport links + heartbeats), Metrics, compression (fp16 wire
// cast, top-k with error feedback), abort propagation (ABORT frames + poisoned
// group: after a failure every later operation fails fast).
//
// Parity: reference csrc/backend/ProcessGroupMCCL.hpp:28-227 and
// ProcessGroupMCCL.cpp:710-3462 (op surface, validation rules, failure
// semantics); the algorithms themselves are new.
#pragma once

#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>

#include <atomic>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "backend/options.h"
#include "backend/work.h"
#include "compression/compressor.h"
#include "kernels/api.h"
#include "runtime/arena.h"
#include "runtime/engine.h"
#include "runtime/health.h"
#include "runtime/metrics.h"
#include "runtime/rendezvous.h"
#include "runtime/tuner.h"
#include "runtime/watchdog.h"
#include "transport/host_transport.h"

namespace mccl { class NcclP2P; }

namespace mccl {

class ProcessGroupMCCL : public c10d::Backend {
 public:
  ProcessGroupMCCL(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                   c10::intrusive_ptr<MCCLOptions> options);
  ~ProcessGroupMCCL() override;

  const std::string getBackendName() const override { return "mccl"; }
  c10::intrusive_ptr<c10d::Backend::Options> getBackendOptions() override {
    return c10::static_intrusive_pointer_cast<c10d::Backend::Options>(options_);
  }

  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors,
                                           const c10d::AllreduceOptions& opts = {}) override;
  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(
      std::vector<at::Tensor>& tensors, const c10d::AllreduceCoalescedOptions& opts = {}) override;
  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors,
                                           const c10d::BroadcastOptions& opts = {}) override;
  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outputs,
                                           std::vector<at::Tensor>& inputs,
                                           const c10d::AllgatherOptions& opts = {}) override;
  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& output, at::Tensor& input,
                                                 const c10d::AllgatherOptions& opts = {}) override;
  c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(
      std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
      const c10d::AllgatherOptions& opts = {}) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor>& outputs,
                                                std::vector<std::vector<at::Tensor>>& inputs,
                                                const c10d::ReduceScatterOptions& opts = {}) override;
  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(
      at::Tensor& output, at::Tensor& input, const c10d::ReduceScatterOptions& opts = {}) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(
      std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
      const c10d::ReduceScatterOptions& opts = {}) override;
  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& tensors,
                                        const c10d::ReduceOptions& opts = {}) override;
  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& opts = {}) override;
  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& tensors, int dst, int tag) override;
  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& tensors, int src, int tag) override;

  void setSequenceNumberForGroup() override {}
  uint64_t getSequenceNumberForGroup() override { return collective_seq_.load(); }
  void abort() override;
  void shutdown() override;

  // ---- introspection / services used by the Python layer -----------------
  Metrics::Summary get_metrics_summary();
  void log_metrics();
  void reset_metrics();
  bool poisoned() const { return poisoned_.load(); }
  // A kernel's bounded wait has given up (read from host-mapped memory: no stream involved).
  bool device_failed_quick() const;
  std::string poison_reason() const;
  std::string describe() const;   // one-line configuration dump
  std::string data_plane() const; // "nvlink-p2p", "nvlink-p2p+nvls", "host-staged", "local", "uninitialised"
  // Fused compressed allreduce (top-k + error feedback) on a CUDA bucket.
  c10::intrusive_ptr<c10d::Work> allreduce_topk(at::Tensor& grad, at::Tensor& residual, double ratio,
                                                float scale);
  // SUM allreduce with a multiplier fused into the reduction epilogue (gradient
  // averaging without DDP's separate pre-division pass).
  c10::intrusive_ptr<c10d::Work> allreduce_scaled(std::vector<at::Tensor>& tensors, float scale);
  // Same, then `epilogue(stream)` is enqueued right behind the reduction on the communication
  // stream and covered by the returned Work (used to chain a bucket's optimizer kernel natively).
  // `overlapped` = false tells the launcher that no compute is left to share the GPU with (the last
  // bucket of a backward pass): the grid may then be larger than the one used under backward.
  c10::intrusive_ptr<c10d::Work> allreduce_scaled_then(std::vector<at::Tensor>& tensors, float scale,
                                                        std::function<void(cudaStream_t)> epilogue,
                                                        bool overlapped = true);
  // Collective: a pool of multicast-bound device memory for user tensors (see runtime/nvls_pool.h).
  bool create_nvls_user_pool(int64_t bytes, c10::DeviceIndex dev);
  // Test hook: next CUDA collective is skipped on this rank (peers must time out).
  void test_skip_next_launch() { skip_next_launch_.store(true); }
  Tuner& tuner() { return tuner_; }
  // globaltimer stamps (ns) of the last arena collective's phases; needs MCCL_PHASE_STAMPS=1.
  std::vector<int64_t> last_phase_stamps();

 private:
  friend struct CudaPath;
  // ---- shared -------------------------------------------------------------
  uint32_t next_seq() { return ++collective_seq_; }
  void check_alive(const char* what);
  void poison(const std::string& why, bool tell_peers);
  c10::intrusive_ptr<WorkMCCL> completed_work(c10d::OpType op, std::vector<at::Tensor> outs,
                                              const at::Tensor* like);
  void register_work(const c10::intrusive_ptr<WorkMCCL>& w);
  void unregister_work(uint32_t seq);
  void abort_all_inflight(const std::string& why);

  // ---- CPU path (process_group_cpu.cpp) ------------------------------------
  void ensure_transport();
  c10::intrusive_ptr<c10d::Work> submit_host(c10d::OpType op, const char* name, uint64_t bytes,
                                             std::vector<at::Tensor> outs,
                                             std::function<void(uint32_t)> body, HostEngine* engine = nullptr);
  void cpu_allreduce(uint32_t seq, at::Tensor& t, c10d::ReduceOp::RedOpType op);
  void cpu_broadcast(uint32_t seq, at::Tensor& t, int root);
  void cpu_allgather(uint32_t seq, std::vector<at::Tensor>& outs, const at::Tensor& in);
  void cpu_reduce_scatter(uint32_t seq, at::Tensor& out, std::vector<at::Tensor>& ins,
                          c10d::ReduceOp::RedOpType op);
  void cpu_reduce(uint32_t seq, at::Tensor& t, int root, c10d::ReduceOp::RedOpType op);

  // ---- CUDA path (process_group_cuda.cpp) ----------------------------------
  void ensure_cuda(c10::DeviceIndex dev);
  c10::intrusive_ptr<c10d::Work> cuda_allreduce(at::Tensor& t, c10d::ReduceOp::RedOpType op, float prescale,
                                                std::function<void(cudaStream_t)> epilogue = nullptr,
                                                bool overlapped = false);
  c10::intrusive_ptr<c10d::Work> cuda_broadcast(at::Tensor& t, int root);
  c10::intrusive_ptr<c10d::Work> cuda_allgather(at::Tensor& out_flat, const at::Tensor& in,
                                                std::vector<at::Tensor>* scatter_to);
  c10::intrusive_ptr<c10d::Work> cuda_reduce_scatter(at::Tensor& out, const at::Tensor& in_flat,
                                                     c10d::ReduceOp::RedOpType op);
  c10::intrusive_ptr<c10d::Work> cuda_barrier();
  c10::intrusive_ptr<c10d::Work> staged_via_host(c10d::OpType op, std::vector<at::Tensor> cuda_tensors,
                                                 std::function<c10::intrusive_ptr<c10d::Work>(std::vector<at::Tensor>&)> fn,
                                                 bool copy_back);
  void release_nvls();  // ordered tear-down of the NVLS region (drain streams, meet the peers, unbind)
  void poll_device(bool must = false);  // watchdog hook: status block + event-timed metrics
  void drain_finished();
  void device_health_check();

  c10::intrusive_ptr<c10d::Store> store_;
  c10::intrusive_ptr<MCCLOptions> options_;
  std::atomic<uint32_t> collective_seq_{0};
  std::atomic<uint32_t> p2p_seq_{0};
  std::atomic<bool> poisoned_{false};
  mutable std::mutex poison_mu_;
  std::string poison_reason_;
  std::atomic<bool> shut_down_{false};
  std::atomic<bool> skip_next_launch_{false};
  uint64_t pool_checks_ = 0;  // Store keys of the pool-offset agreement rounds (same sequence on every rank)
  // MCCL_DEVICE_TIMING: 0 = never, 1 = every CUDA collective, N = every Nth (default 8).  Timed ops carry
  // an event pair and feed the latency statistics; the others are only counted (timing events cost a few
  // microseconds per call, which matters for latency-bound collectives).
  int device_timing_ = 8;
  std::atomic<uint32_t> timing_tick_{0};
  bool profile_titles_ = false; // MCCL_PROFILE_TITLES: name the Work for torch's profiler (RecordFunction per op)

  Metrics metrics_;
  Tuner tuner_;
  std::unique_ptr<Compressor> compressor_;
  std::unique_ptr<Rendezvous> rendezvous_;
  std::unique_ptr<HostTransport> transport_;
  std::mutex transport_init_mu_;
  std::unique_ptr<HostEngine> collective_engine_;  // CPU collectives: one worker, total order
  std::unique_ptr<HostEngine> p2p_engine_;         // send/recv: may overlap collectives
  std::unique_ptr<Watchdog> watchdog_;
  std::unique_ptr<HealthMonitor> health_;
  // CUDA send/recv: NCCL p2p on a side stream (created on first use); MCCL_P2P=host stages through pinned memory instead
  std::shared_ptr<NcclP2P> nccl_p2p_;
  std::mutex nccl_mu_;
  NcclP2P* ensure_nccl_p2p();

  std::mutex works_mu_;
  std::unordered_map<uint32_t, c10::weak_intrusive_ptr<WorkMCCL>> works_;

  // CUDA state
  struct CudaState;
  std::shared_ptr<CudaState> cuda_;  // shared_ptr: destructible where the type is incomplete
  std::atomic<const SymmetricArena*> arena_quick_{nullptr};  // cuda_->arena for lock-free status reads
  std::mutex cuda_mu_;
};

c10::intrusive_ptr<ProcessGroupMCCL> createProcessGroupMCCL(
    const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, std::chrono::milliseconds timeout);

// Process-wide "active" group used by the module-level metrics accessors.
void set_active_pg(ProcessGroupMCCL* pg);
void clear_active_pg(ProcessGroupMCCL* pg);
ProcessGroupMCCL* active_pg_locked(std::unique_lock<std::mutex>& lk);

}  // namespace mccl
