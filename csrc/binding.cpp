// pybind11 module `_C`: backend registration, metrics accessors, kernel test
// hooks, protocol/compression helpers and the single-device emulation harness.
//
// Hooks named `_metal_*` are aliases of the `_ew_*` hooks so that test code
// written against the reference's names keeps working
// (reference csrc/backend/Registration.cpp:84-431).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/chrono.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/utils/pybind.h>
#include <torch/extension.h>

#include <execinfo.h>
#include <signal.h>
#include <unistd.h>

#include <cmath>
#include <optional>

#include "backend/options.h"
#include "backend/process_group.h"
#include "backend/tensor_checks.h"
#include "common/version.h"
#include "compression/compressor.h"
#include "cpu/reduce.h"
#include "kernels/api.h"
#include "kernels/launch_count.h"
#include "kernels/optim_api.h"
#include "kernels/topk_api.h"
#include "optim/adamw_plan.h"
#include "optim/bucket_hook.h"
#include "runtime/arena.h"
#include "runtime/engine.h"
#include "runtime/mempool.h"
#include "runtime/nvls_pool.h"
#include "runtime/watchdog.h"
#ifdef MCCL_WITH_STFT
#include "transforms/stft.h"
#endif
#include "transport/protocol.h"

namespace py = pybind11;
using namespace mccl;

namespace {

#define CK(expr)                                                                  \
  do {                                                                            \
    cudaError_t _e = (expr);                                                      \
    if (_e != cudaSuccess) {                                                      \
      cudaGetLastError();                                                         \
      throw DeviceError(std::string(#expr) + ": " + cudaGetErrorString(_e));      \
    }                                                                             \
  } while (0)

c10d::ReduceOp::RedOpType op_from_kern(kern::RedOp op) {
  switch (op) {
    case kern::SUM: return c10d::ReduceOp::SUM;
    case kern::AVG: return c10d::ReduceOp::AVG;
    case kern::MIN: return c10d::ReduceOp::MIN;
    case kern::MAX: return c10d::ReduceOp::MAX;
    default: return c10d::ReduceOp::PRODUCT;
  }
}

at::Tensor ew_binary(at::Tensor dst, const at::Tensor& src, kern::RedOp op) {
  check_tensor(dst, "elementwise");
  check_tensor(src, "elementwise");
  check_same(dst, src, "elementwise");
  if (dst.is_cuda()) {
    c10::cuda::CUDAGuard g(dst.device());
    CK(kern::launch_ew_reduce(dst.data_ptr(), src.data_ptr(), dst.numel(), to_kern_dtype(dst.scalar_type()), op,
                              at::cuda::getCurrentCUDAStream()));
  } else {
    cpu_reduce_into(dst.data_ptr(), src.data_ptr(), dst.numel(), dst.scalar_type(), op_from_kern(op));
  }
  return dst;
}

at::Tensor ew_scale(at::Tensor buf, double scale) {
  check_tensor(buf, "scale_inplace");
  if (buf.is_cuda()) {
    c10::cuda::CUDAGuard g(buf.device());
    CK(kern::launch_ew_scale(buf.data_ptr(), buf.numel(), to_kern_dtype(buf.scalar_type()), scale,
                             at::cuda::getCurrentCUDAStream()));
  } else {
    cpu_scale_inplace(buf.data_ptr(), buf.numel(), buf.scalar_type(), scale);
  }
  return buf;
}

at::Tensor ew_accscale(at::Tensor dst, const at::Tensor& src, double scale) {
  check_tensor(dst, "accumulate_and_scale");
  check_tensor(src, "accumulate_and_scale");
  check_same(dst, src, "accumulate_and_scale");
  if (dst.is_cuda()) {
    c10::cuda::CUDAGuard g(dst.device());
    CK(kern::launch_ew_accumulate_scale(dst.data_ptr(), src.data_ptr(), dst.numel(),
                                        to_kern_dtype(dst.scalar_type()), scale, at::cuda::getCurrentCUDAStream()));
  } else {
    cpu_accumulate_and_scale(dst.data_ptr(), src.data_ptr(), dst.numel(), dst.scalar_type(), scale);
  }
  return dst;
}

at::Tensor cast_to(const at::Tensor& src, at::ScalarType dt, double scale) {
  check_tensor(src, "cast");
  MCCL_CHECK_TENSOR(src.is_cuda(), "cast: CUDA tensors only");
  at::Tensor dst = at::empty(src.sizes(), src.options().dtype(dt));
  c10::cuda::CUDAGuard g(src.device());
  CK(kern::launch_cast(dst.data_ptr(), to_kern_dtype(dt), src.data_ptr(), to_kern_dtype(src.scalar_type()),
                       src.numel(), static_cast<float>(scale), at::cuda::getCurrentCUDAStream()));
  return dst;
}

// ---- single-device emulation of a multi-rank group ----------------------------
// All "ranks" live on one GPU; each collective is one cooperative launch with
// grid.y = ranks, so the very kernels that run across NVLink are exercised
// (flags, epochs, slots, reductions) on a single-GPU test box.
class EmuGroup {
 public:
  EmuGroup(int ws, int64_t parity_bytes, int64_t device_wait_us)
      : ws_(ws), wait_ns_(static_cast<unsigned long long>(device_wait_us) * 1000ull) {
    arena_.reset(SymmetricArena::make_emulated(ws, static_cast<size_t>(parity_bytes)));
  }
  int world_size() const { return ws_; }

  kern::CollParams params(const std::vector<at::Tensor>& ins, const std::vector<at::Tensor>& outs) {
    MCCL_CHECK(static_cast<int>(ins.size()) == ws_ && static_cast<int>(outs.size()) == ws_,
               "emulation needs one tensor per rank");
    kern::CollParams p;
    std::memset(&p, 0, sizeof(p));
    arena_->fill_params(p, arena_->next_epoch());
    for (int r = 0; r < ws_; ++r) {
      p.ctx[r].in = ins[r].data_ptr();
      p.ctx[r].out = outs[r].data_ptr();
    }
    p.scale = 1.0f;
    p.wait_ns = wait_ns_;
    p.debug_checks = debug_checks_ ? 1 : 0;
    return p;
  }
  // Debug mode: every kernel verifies its buffer ranges and reports ERR_BOUNDS instead of touching
  // memory outside them.
  void set_debug_checks(bool on) { debug_checks_ = on; }
  // Test hook: shrinks the capacity the kernels are told about (not the allocation), so that the
  // range checks can be seen to fire without any out-of-range access.
  void set_claimed_capacity(int64_t bytes) { claimed_capacity_ = bytes; }
  // Fills all data buffers of every emulated rank's arena with a byte pattern (NaNs for 0xFF):
  // a kernel that read a slot nobody wrote in the current epoch would then produce garbage.
  void poison_buffers(int byte) {
    for (int r = 0; r < ws_; ++r)
      CK(cudaMemsetAsync(arena_->base(r) + kern::kSignalBytes, byte, kern::kNumParity * arena_->parity_bytes(),
                         at::cuda::getCurrentCUDAStream()));
  }
  kern::LaunchCfg cfg(int ctas) {
    kern::LaunchCfg c;
    c.ctas = ctas;
    c.emulate_ranks = ws_;
    return c;
  }
  void check_fits(size_t need) {
    MCCL_CHECK(need <= arena_->parity_bytes(), "payload needs " << need << " arena bytes, have " << arena_->parity_bytes());
  }

  void allreduce(std::vector<at::Tensor> ts, const std::string& op, const std::string& algo,
                 const std::string& wire, double scale, int ctas, int tiles, bool push_gather) {
    for (auto& t : ts) check_tensor(t, "emu allreduce");
    c10::cuda::CUDAGuard g(ts[0].device());
    kern::DType dt = to_kern_dtype(ts[0].scalar_type());
    kern::DType wd = wire == "bf16" ? kern::BF16 : wire == "fp16" ? kern::F16 : dt;
    kern::CollParams p = params(ts, ts);
    p.count = ts[0].numel();
    p.op = parse_op(op);
    p.scale = static_cast<float>((p.op == kern::AVG ? 1.0 / ws_ : 1.0) * scale);
    size_t wb = static_cast<size_t>(p.count) * kern::dtype_size(wd);
    p.tiles = tiles;
    p.push_gather = push_gather ? 1 : 0;
    if (algo == "oneshot") {
      check_fits(kern::oneshot_arena_bytes(wb, ws_));
      CK(kern::launch_allreduce_oneshot(p, dt, wd, cfg(ctas), at::cuda::getCurrentCUDAStream()));
    } else {
      check_fits(kern::twoshot_arena_bytes(wb, ws_, push_gather));
      CK(kern::launch_allreduce_twoshot(p, dt, wd, cfg(ctas), at::cuda::getCurrentCUDAStream()));
    }
  }
  // pitch > 0: chunk q of the input starts at element q * pitch (a slice of a larger input)
  void reduce_scatter(std::vector<at::Tensor> outs, std::vector<at::Tensor> ins, const std::string& op, int ctas,
                      int64_t pitch) {
    c10::cuda::CUDAGuard g(ins[0].device());
    kern::DType dt = to_kern_dtype(ins[0].scalar_type());
    kern::CollParams p = params(ins, outs);
    p.count = outs[0].numel();
    p.chunk_pitch = pitch;
    p.op = parse_op(op);
    p.scale = p.op == kern::AVG ? 1.0f / ws_ : 1.0f;
    check_fits(kern::twoshot_arena_bytes(static_cast<size_t>(p.count) * ws_ * kern::dtype_size(dt), ws_) + 128 * ws_);
    CK(kern::launch_reduce_scatter(p, dt, dt, cfg(ctas), at::cuda::getCurrentCUDAStream()));
  }
  // pitch_bytes > 0: rank r's block lands at out + r * pitch_bytes (a slice of a larger gather)
  void allgather(std::vector<at::Tensor> outs, std::vector<at::Tensor> ins, int ctas, int tile_bytes,
                 int64_t pitch_bytes, int64_t slice_bytes, int64_t slice_offset) {
    c10::cuda::CUDAGuard g(ins[0].device());
    kern::CollParams p = params(ins, outs);
    p.count = slice_bytes > 0 ? slice_bytes : static_cast<int64_t>(ins[0].nbytes());
    p.out_pitch = pitch_bytes;
    p.tile_bytes = tile_bytes;
    if (slice_offset > 0)
      for (int r = 0; r < ws_; ++r) {
        p.ctx[r].in = static_cast<const char*>(p.ctx[r].in) + slice_offset;
        p.ctx[r].out = static_cast<char*>(p.ctx[r].out) + slice_offset;
      }
    check_fits(kern::allgather_stage_bytes(static_cast<size_t>(p.count), ws_));
    if (claimed_capacity_ > 0) p.parity_capacity = static_cast<size_t>(claimed_capacity_);
    CK(kern::launch_allgather(p, cfg(ctas), at::cuda::getCurrentCUDAStream()));
  }
  void broadcast(std::vector<at::Tensor> ts, int root, int ctas, int tile_bytes) {
    c10::cuda::CUDAGuard g(ts[0].device());
    kern::CollParams p = params(ts, ts);
    p.count = static_cast<int64_t>(ts[0].nbytes());
    p.root = root;
    p.tile_bytes = tile_bytes;
    check_fits(kern::broadcast_stage_bytes(static_cast<size_t>(p.count)));
    if (claimed_capacity_ > 0) p.parity_capacity = static_cast<size_t>(claimed_capacity_);
    CK(kern::launch_broadcast(p, cfg(ctas), at::cuda::getCurrentCUDAStream()));
  }
  void barrier() {
    std::vector<at::Tensor> none;
    kern::CollParams p;
    std::memset(&p, 0, sizeof(p));
    arena_->fill_params(p, arena_->next_epoch());
    p.wait_ns = wait_ns_;
    CK(kern::launch_barrier(p, cfg(1), at::cuda::getCurrentCUDAStream()));
  }
  // A collective in which `absent` never signals: every other rank's bounded
  // wait must expire and report it.  Implemented as a barrier whose epoch is
  // two ahead of anything `absent` has published (nothing ever sets the flag).
  std::vector<int64_t> barrier_with_absent_rank(int absent) {
    MCCL_CHECK(absent >= 0 && absent < ws_, "bad rank");
    kern::CollParams p;
    std::memset(&p, 0, sizeof(p));
    uint32_t e = arena_->next_epoch();
    arena_->fill_params(p, e);
    p.wait_ns = wait_ns_;
    // Launch only the other ranks: compact their contexts, keep their rank ids.
    kern::CollParams q = p;
    int m = 0;
    for (int r = 0; r < ws_; ++r)
      if (r != absent) q.ctx[m++] = p.ctx[r];
    kern::LaunchCfg c = cfg(1);
    c.emulate_ranks = m;
    CK(kern::launch_barrier(q, c, at::cuda::getCurrentCUDAStream()));
    CK(cudaStreamSynchronize(at::cuda::getCurrentCUDAStream()));
    int probe = absent == 0 ? 1 : 0;
    uint32_t st[kern::kStatusWords];
    arena_->read_status(st, at::cuda::getCurrentCUDAStream(), probe);
    return {st[0], st[1], st[2], st[3]};
  }
  std::vector<int64_t> status(int r) {
    uint32_t st[kern::kStatusWords];
    arena_->read_status(st, at::cuda::getCurrentCUDAStream(), r);
    return {st[0], st[1], st[2], st[3]};
  }
  void clear_status() {
    arena_->clear_status(at::cuda::getCurrentCUDAStream());
    CK(cudaStreamSynchronize(at::cuda::getCurrentCUDAStream()));
  }

  // grads[r], residuals[r] per rank; dense result written into grads.
  void topk_allreduce(std::vector<at::Tensor> grads, std::vector<at::Tensor> residuals, double ratio, double scale,
                      int ctas) {
    c10::cuda::CUDAGuard g(grads[0].device());
    auto stream = at::cuda::getCurrentCUDAStream();
    const int64_t n = grads[0].numel();
    int64_t k = std::max<int64_t>(1, static_cast<int64_t>(std::floor(static_cast<double>(n) * ratio)));
    k = std::min(k, n);
    std::vector<at::Tensor> pairs;
    kern::TopkArgs a0;
    for (int r = 0; r < ws_; ++r) {
      at::Tensor scratch = at::empty({static_cast<int64_t>(kern::topk_scratch_bytes())}, grads[r].options().dtype(at::kByte));
      pairs.push_back(at::empty({k * 2}, grads[r].options().dtype(at::kInt)));
      kern::TopkArgs a;
      a.grad = grads[r].data_ptr();
      a.grad_is_bf16 = grads[r].scalar_type() == at::kBFloat16;
      a.residual = residuals[r].data_ptr<float>();
      a.n = n;
      a.k = k;
      a.scratch = scratch.data_ptr();
      a.pairs = pairs[r].data_ptr();
      a.scale = static_cast<float>(scale);
      CK(kern::launch_topk_select(a, stream));
      if (r == 0) a0 = a;
    }
    kern::CollParams p = params(pairs, grads);
    p.count = k;
    p.scale = static_cast<float>(scale);
    check_fits(kern::topk_pad(static_cast<size_t>(k) * 8) * ws_);
    CK(kern::launch_topk_exchange_scatter(p, a0, cfg(ctas), stream));
  }

 private:
  static kern::RedOp parse_op(const std::string& s) {
    if (s == "sum") return kern::SUM;
    if (s == "avg") return kern::AVG;
    if (s == "min") return kern::MIN;
    if (s == "max") return kern::MAX;
    if (s == "product") return kern::PRODUCT;
    throw TensorError("unknown reduce op '" + s + "'");
  }
  int ws_;
  unsigned long long wait_ns_;
  bool debug_checks_ = false;
  int64_t claimed_capacity_ = 0;
  std::unique_ptr<SymmetricArena> arena_;
};

// (pairs as int32 [k,2], k) of the exact top-k of |grad + residual|; residual updated.
at::Tensor topk_select(const at::Tensor& grad, at::Tensor residual, double ratio) {
  check_tensor(grad, "topk_select");
  MCCL_CHECK_TENSOR(grad.is_cuda(), "topk_select: CUDA tensors only");
  MCCL_CHECK_TENSOR(residual.is_cuda() && residual.scalar_type() == at::kFloat && residual.numel() == grad.numel(),
                    "topk_select: residual must be float32 of the same size");
  c10::cuda::CUDAGuard g(grad.device());
  const int64_t n = grad.numel();
  int64_t k = std::max<int64_t>(1, static_cast<int64_t>(std::floor(static_cast<double>(n) * ratio)));
  k = std::min(k, n);
  at::Tensor scratch = at::empty({static_cast<int64_t>(kern::topk_scratch_bytes())}, grad.options().dtype(at::kByte));
  at::Tensor pairs = at::empty({k, 2}, grad.options().dtype(at::kInt));
  kern::TopkArgs a;
  a.grad = grad.data_ptr();
  a.grad_is_bf16 = grad.scalar_type() == at::kBFloat16;
  a.residual = residual.data_ptr<float>();
  a.n = n;
  a.k = k;
  a.scratch = scratch.data_ptr();
  a.pairs = pairs.data_ptr();
  a.scale = 1.f;
  CK(kern::launch_topk_select(a, at::cuda::getCurrentCUDAStream()));
  return pairs;
}

py::bytes pack_header(int op, uint32_t seq, uint32_t tid, uint32_t chunk_index, uint32_t payload_bytes,
                      int flags, uint32_t crc) {
  MessageHeader h = make_header(static_cast<mccl::OpType>(op), seq, tid, chunk_index, payload_bytes,
                                static_cast<uint8_t>(flags), crc);
  return py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
}

py::bytes pack_handshake(uint32_t rank, uint32_t world_size, const std::string& hostname) {
  HandshakePayload p;
  std::memset(&p, 0, sizeof(p));
  p.version = MCCL_PROTOCOL_VERSION;
  p.rank = rank;
  p.world_size = world_size;
  std::strncpy(p.hostname, hostname.c_str(), sizeof(p.hostname) - 1);
  return py::bytes(reinterpret_cast<const char*>(&p), sizeof(p));
}

// MCCL_CRASH_BACKTRACE=1: print a native backtrace on SIGSEGV/SIGABRT before dying.
void crash_handler(int sig) {
  void* frames[64];
  int n = backtrace(frames, 64);
  const char msg[] = "[MCCL FATAL] fatal signal, native backtrace:\n";
  ssize_t w = write(2, msg, sizeof(msg) - 1);
  (void)w;
  backtrace_symbols_fd(frames, n, 2);
  signal(sig, SIG_DFL);
  raise(sig);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "mccl_b200 native layer: c10d backend 'mccl' for CUDA (NVLink peer kernels) and CPU tensors";
  if (env_bool("MCCL_CRASH_BACKTRACE", false)) {
    signal(SIGSEGV, crash_handler);
    signal(SIGABRT, crash_handler);
  }
  m.attr("__version__") = MCCL_VERSION_STRING;
  m.attr("__protocol_version__") = MCCL_PROTOCOL_VERSION;
  m.attr("MAX_WORLD") = kern::kMaxWorld;
  m.attr("HEADER_BYTES") = sizeof(MessageHeader);
  m.attr("HANDSHAKE_BYTES") = sizeof(HandshakePayload);

  py::register_exception<MCCLError>(m, "MCCLError", PyExc_RuntimeError);

  // ---- backend -----------------------------------------------------------------
  py::enum_<CompressionMode>(m, "CompressionMode")
      .value("NONE", CompressionMode::NONE)
      .value("FP16", CompressionMode::FP16)
      .value("TOPK", CompressionMode::TOPK);

  auto backend_cls = py::module::import("torch._C._distributed_c10d").attr("Backend");
  auto backend_opts_cls = backend_cls.attr("Options");

  py::class_<MCCLOptions, c10::intrusive_ptr<MCCLOptions>>(m, "MCCLOptions", backend_opts_cls)
      .def(py::init([]() { return MCCLOptions::from_env(kBackendDefaultTimeout); }))
      .def(py::init([](std::chrono::milliseconds t) { return MCCLOptions::from_env(t); }), py::arg("timeout"))
      .def_readwrite("transport", &MCCLOptions::transport)
      .def_readwrite("listen_addr", &MCCLOptions::listen_addr)
      .def_readwrite("port_base", &MCCLOptions::port_base)
      .def_readwrite("ifname", &MCCLOptions::ifname)
      .def_readwrite("chunk_bytes", &MCCLOptions::chunk_bytes)
      .def_readwrite("small_msg_threshold", &MCCLOptions::small_msg_threshold)
      .def_readwrite("transport_crc", &MCCLOptions::transport_crc)
      .def_readwrite("fast_math", &MCCLOptions::fast_math)
      .def_readwrite("gpu_threshold", &MCCLOptions::gpu_threshold)
      .def_readwrite("overlap_comm", &MCCLOptions::overlap_comm)
      .def_readwrite("max_queue_depth", &MCCLOptions::max_queue_depth)
      .def_readwrite("compression", &MCCLOptions::compression)
      .def_readwrite("topk_ratio", &MCCLOptions::topk_ratio)
      .def_readwrite("wire_dtype", &MCCLOptions::wire_dtype)
      .def_readwrite("watchdog_timeout", &MCCLOptions::watchdog_timeout)
      .def_readwrite("heartbeat_interval", &MCCLOptions::heartbeat_interval)
      .def_readwrite("algo", &MCCLOptions::algo)
      .def_readwrite("oneshot_max_bytes", &MCCLOptions::oneshot_max_bytes)
      .def_readwrite("comm_ctas", &MCCLOptions::comm_ctas)
      .def_readwrite("tiles", &MCCLOptions::tiles)
      .def_readwrite("gather", &MCCLOptions::gather)
      .def_readwrite("lanes", &MCCLOptions::lanes)
      .def_readwrite("arena_bytes", &MCCLOptions::arena_bytes)
      .def_readwrite("device_wait_us", &MCCLOptions::device_wait_us)
      .def_readwrite("blocking_wait", &MCCLOptions::blocking_wait)
      .def_readwrite("nvls", &MCCLOptions::nvls)
      .def_readwrite("nvls_bytes", &MCCLOptions::nvls_bytes)
      .def_readwrite("nvls_min_bytes", &MCCLOptions::nvls_min_bytes)
      .def_readwrite("nvls_split_min_bytes", &MCCLOptions::nvls_split_min_bytes)
      .def_readwrite("tile_bytes", &MCCLOptions::tile_bytes)
      .def_readwrite("debug_checks", &MCCLOptions::debug_checks);

  py::class_<ProcessGroupMCCL, c10::intrusive_ptr<ProcessGroupMCCL>>(m, "ProcessGroupMCCL", backend_cls)
      .def(py::init([](const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                       c10::intrusive_ptr<MCCLOptions> opts) {
             return c10::make_intrusive<ProcessGroupMCCL>(store, rank, size, std::move(opts));
           }),
           py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("options"),
           py::call_guard<py::gil_scoped_release>())
      .def("describe", &ProcessGroupMCCL::describe)
      .def("data_plane", &ProcessGroupMCCL::data_plane)
      .def_property_readonly("poisoned", &ProcessGroupMCCL::poisoned)
      .def("poison_reason", &ProcessGroupMCCL::poison_reason)
      .def("get_metrics", &ProcessGroupMCCL::get_metrics_summary, py::call_guard<py::gil_scoped_release>())
      .def("reset_metrics", &ProcessGroupMCCL::reset_metrics)
      .def("tuner_dump", [](ProcessGroupMCCL& pg) { return pg.tuner().dump(); })
      .def("allreduce_topk", &ProcessGroupMCCL::allreduce_topk, py::arg("grad"), py::arg("residual"),
           py::arg("ratio"), py::arg("scale") = 1.0f, py::call_guard<py::gil_scoped_release>())
      .def("allreduce_scaled",
           [](ProcessGroupMCCL& pg, at::Tensor t, double scale) {
             // SUM allreduce with a fused multiplier (e.g. 1/world for gradient averaging).
             std::vector<at::Tensor> v{t};
             return pg.allreduce_scaled(v, static_cast<float>(scale));
           },
           py::arg("tensor"), py::arg("scale"), py::call_guard<py::gil_scoped_release>())
      .def("last_phase_stamps", &ProcessGroupMCCL::last_phase_stamps, py::call_guard<py::gil_scoped_release>())
      .def("allreduce_adamw",
           [](ProcessGroupMCCL& pg, at::Tensor bucket, double scale, py::list specs, int64_t step) {
             // bucket = sum(bucket) * scale in one kernel, then the bucket's AdamW update(s) behind it on the
             // same communication stream: no Python between them, one Work covers all.  `specs` holds one
             // (plan, grads, lr, beta1, beta2, eps, weight_decay) tuple per param group present in the bucket.
             struct L {
               AdamWPlan* plan;
               double lr, b1, b2, eps, wd;
             };
             std::vector<L> ls;
             for (auto item : specs) {
               py::tuple t = item.cast<py::tuple>();
               AdamWPlan* plan = t[0].cast<AdamWPlan*>();
               plan->bind_grads(t[1].cast<std::vector<at::Tensor>>());
               ls.push_back({plan, t[2].cast<double>(), t[3].cast<double>(), t[4].cast<double>(), t[5].cast<double>(),
                             t[6].cast<double>()});
             }
             std::vector<at::Tensor> v{bucket};
             py::gil_scoped_release nogil;
             return pg.allreduce_scaled_then(v, static_cast<float>(scale), [ls, step](cudaStream_t s) {
               for (const auto& l : ls) l.plan->launch(s, l.lr, l.b1, l.b2, l.eps, l.wd, step, 1.0);
             });
           },
           py::arg("bucket"), py::arg("scale"), py::arg("specs"), py::arg("step"))
      .def("create_nvls_user_pool",
           [](ProcessGroupMCCL& pg, int64_t bytes, int device) { return pg.create_nvls_user_pool(bytes, static_cast<c10::DeviceIndex>(device)); },
           py::arg("bytes"), py::arg("device"), py::call_guard<py::gil_scoped_release>(),
           "Collective: binds a pool of device memory to an NVLink multicast object for zero-copy allreduce.")
      .def("_test_skip_next_launch", &ProcessGroupMCCL::test_skip_next_launch)
      .def("shutdown", &ProcessGroupMCCL::shutdown, py::call_guard<py::gil_scoped_release>());

  m.def(
      "_create_process_group",
      [](const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, std::chrono::milliseconds timeout) {
        return createProcessGroupMCCL(store, rank, size, timeout);
      },
      py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("timeout"),
      py::call_guard<py::gil_scoped_release>());

  m.def("_register_backend", []() {
    py::object dist = py::module::import("torch.distributed");
    py::object backend = dist.attr("Backend");
    py::object create = py::module::import("mccl_b200._C").attr("_create_process_group");
    py::object wrapper = py::module::import("mccl_b200._registration").attr("make_create_fn")(create);
    backend.attr("register_backend")("mccl", wrapper, py::arg("extended_api") = true,
                                     py::arg("devices") = py::make_tuple("cpu", "cuda"));
  });

  // ---- metrics / pools ----------------------------------------------------------
  py::class_<Metrics::Summary>(m, "MetricsSummary")
      .def_readonly("total_ops", &Metrics::Summary::total_ops)
      .def_readonly("total_bytes_sent", &Metrics::Summary::total_bytes_sent)
      .def_readonly("total_bytes_recv", &Metrics::Summary::total_bytes_recv)
      .def_readonly("total_errors", &Metrics::Summary::total_errors)
      .def_readonly("avg_latency_ms", &Metrics::Summary::avg_latency_ms)
      .def_readonly("p50_latency_ms", &Metrics::Summary::p50_latency_ms)
      .def_readonly("p99_latency_ms", &Metrics::Summary::p99_latency_ms)
      .def_readonly("peak_throughput_gbps", &Metrics::Summary::peak_throughput_gbps)
      .def_readonly("avg_sync_ms", &Metrics::Summary::avg_sync_ms)
      .def_readonly("avg_network_ms", &Metrics::Summary::avg_network_ms)
      .def_readonly("avg_reduce_ms", &Metrics::Summary::avg_reduce_ms)
      .def_readonly("avg_queue_wait_ms", &Metrics::Summary::avg_queue_wait_ms)
      .def_readonly("avg_execution_ms", &Metrics::Summary::avg_execution_ms);

  m.def(
      "_get_metrics_summary",
      []() -> std::optional<Metrics::Summary> {
        std::unique_lock<std::mutex> lk;
        ProcessGroupMCCL* pg = active_pg_locked(lk);
        if (!pg) return std::nullopt;
        return pg->get_metrics_summary();
      },
      py::call_guard<py::gil_scoped_release>());
  m.def(
      "_log_metrics",
      []() {
        std::unique_lock<std::mutex> lk;
        ProcessGroupMCCL* pg = active_pg_locked(lk);
        if (pg) pg->log_metrics();
      },
      py::call_guard<py::gil_scoped_release>());
  m.def(
      "_reset_metrics",
      []() {
        std::unique_lock<std::mutex> lk;
        ProcessGroupMCCL* pg = active_pg_locked(lk);
        if (pg) pg->reset_metrics();
      },
      py::call_guard<py::gil_scoped_release>());
  m.def("_trim_staging_pool", []() { staging_memory_pool().trim(); });
  m.def("_staging_pool_bytes", []() { return staging_memory_pool().total_allocated(); });

  // ---- elementwise kernel hooks ---------------------------------------------------
  m.def("_ew_accumulate_chunk", [](at::Tensor d, const at::Tensor& s) { return ew_binary(d, s, kern::SUM); });
  m.def("_ew_elementwise_min", [](at::Tensor d, const at::Tensor& s) { return ew_binary(d, s, kern::MIN); });
  m.def("_ew_elementwise_max", [](at::Tensor d, const at::Tensor& s) { return ew_binary(d, s, kern::MAX); });
  m.def("_ew_elementwise_product", [](at::Tensor d, const at::Tensor& s) { return ew_binary(d, s, kern::PRODUCT); });
  m.def("_ew_scale_inplace", &ew_scale, py::arg("buf"), py::arg("scale"));
  m.def("_ew_accumulate_and_scale", &ew_accscale, py::arg("dst"), py::arg("src"), py::arg("scale"));
  m.attr("_metal_accumulate_chunk") = m.attr("_ew_accumulate_chunk");
  m.attr("_metal_elementwise_min") = m.attr("_ew_elementwise_min");
  m.attr("_metal_elementwise_max") = m.attr("_ew_elementwise_max");
  m.attr("_metal_elementwise_product") = m.attr("_ew_elementwise_product");
  m.attr("_metal_scale_inplace") = m.attr("_ew_scale_inplace");
  m.attr("_metal_accumulate_and_scale") = m.attr("_ew_accumulate_and_scale");
  m.def("_cast", &cast_to, py::arg("src"), py::arg("dtype"), py::arg("scale") = 1.0);

  // ---- protocol -----------------------------------------------------------------------
  m.def("_crc32", [](py::bytes b) {
    std::string s = b;
    return crc32_compute(s.data(), s.size());
  });
  m.def("_pack_header", &pack_header, py::arg("op"), py::arg("seq"), py::arg("tid"), py::arg("chunk_index"),
        py::arg("payload_bytes"), py::arg("flags") = 0, py::arg("crc") = 0);
  m.def("_pack_handshake", &pack_handshake);
  m.def("_op_codes", []() {
    py::dict d;
    d["ALLREDUCE"] = 1; d["BROADCAST"] = 2; d["BARRIER"] = 3; d["ALLGATHER"] = 4; d["REDUCE_SCATTER"] = 5;
    d["SEND"] = 6; d["RECV"] = 7; d["HANDSHAKE"] = 10; d["HEARTBEAT"] = 11; d["ABORT"] = 255;
    return d;
  });

  // ---- compression (host implementations) ------------------------------------------------
  m.def("_fp16_compress", [](const at::Tensor& t) {
    MCCL_CHECK_TENSOR(t.is_cpu() && t.is_contiguous(), "cpu contiguous tensor expected");
    FP16Compressor c;
    WireDType wd = to_wire_dtype(t.scalar_type());
    std::string out(c.max_compressed_size(t.nbytes(), wd), '\0');
    size_t n = c.compress(t.data_ptr(), t.nbytes(), out.data(), out.size(), wd, 0);
    out.resize(n);
    return py::bytes(out);
  });
  m.def("_fp16_decompress", [](py::bytes b, int64_t numel) {
    std::string s = b;
    at::Tensor t = at::empty({numel}, at::kFloat);
    FP16Compressor c;
    c.decompress(s.data(), s.size(), t.data_ptr(), t.nbytes(), WireDType::F32);
    return t;
  });
  py::class_<TopKCompressor>(m, "TopKCompressor")
      .def(py::init<double>(), py::arg("ratio"))
      .def("k_for", &TopKCompressor::k_for)
      .def("compress",
           [](TopKCompressor& c, const at::Tensor& t, uint64_t stable_id) {
             MCCL_CHECK_TENSOR(t.is_cpu() && t.is_contiguous(), "cpu contiguous tensor expected");
             WireDType wd = to_wire_dtype(t.scalar_type());
             std::string out(c.max_compressed_size(t.nbytes(), wd), '\0');
             size_t n = c.compress(t.data_ptr(), t.nbytes(), out.data(), out.size(), wd, stable_id);
             out.resize(n);
             return py::bytes(out);
           },
           py::arg("tensor"), py::arg("stable_id") = 0)
      .def("decompress",
           [](TopKCompressor& c, py::bytes b, int64_t numel) {
             std::string s = b;
             at::Tensor t = at::empty({numel}, at::kFloat);
             c.decompress(s.data(), s.size(), t.data_ptr(), t.nbytes(), WireDType::F32);
             return t;
           })
      .def("residual",
           [](TopKCompressor& c, uint64_t id) {
             auto v = c.residual(id);
             at::Tensor t = at::empty({static_cast<int64_t>(v.size())}, at::kFloat);
             if (!v.empty()) std::memcpy(t.data_ptr(), v.data(), v.size() * 4);
             return t;
           })
      .def("residual_buffers", &TopKCompressor::residual_buffers)
      .def("reset_error_feedback", [](TopKCompressor& c) { c.reset_error_feedback(); });

  // ---- fused optimizer -------------------------------------------------------------------
  py::class_<AdamWPlan>(m, "AdamWPlan")
      .def(py::init<std::vector<at::Tensor>, std::vector<at::Tensor>, std::vector<at::Tensor>>(), py::arg("params"),
           py::arg("exp_avg"), py::arg("exp_avg_sq"))
      .def("step", &AdamWPlan::step, py::arg("grads"), py::arg("lr"), py::arg("beta1"), py::arg("beta2"),
           py::arg("eps"), py::arg("weight_decay"), py::arg("step"), py::arg("grad_scale") = 1.0)
      .def_property_readonly("num_chunks", &AdamWPlan::num_chunks);
  // ---- native DDP hook: allreduce + AdamW per bucket, registered on the C++ reducer ----
  py::class_<BucketOptimizerState, std::shared_ptr<BucketOptimizerState>>(m, "BucketOptimizerState")
      .def(py::init([](c10::intrusive_ptr<ProcessGroupMCCL> pg, double scale) {
             return std::make_shared<BucketOptimizerState>(std::move(pg), scale);
           }),
           py::arg("backend"), py::arg("scale"))
      .def("add_param", &BucketOptimizerState::add_param, py::arg("param"), py::arg("exp_avg"), py::arg("exp_avg_sq"),
           py::arg("group"))
      .def("set_hyper", &BucketOptimizerState::set_hyper, py::arg("group"), py::arg("lr"), py::arg("beta1"),
           py::arg("beta2"), py::arg("eps"), py::arg("weight_decay"))
      .def("set_step", &BucketOptimizerState::set_step)
      .def("take_stepped", &BucketOptimizerState::take_stepped);
  m.def(
      "_register_bucket_optimizer_hook",
      [](py::object reducer, std::shared_ptr<BucketOptimizerState> st) {
        auto r = reducer.cast<std::shared_ptr<c10d::Reducer>>();
        r->register_comm_hook(std::make_unique<BucketOptimizerHook>(std::move(st)));
      },
      py::arg("reducer"), py::arg("state"),
      "Installs the native allreduce+AdamW bucket hook on a DistributedDataParallel reducer (ddp.reducer).");

  // Drives the pool's range allocator with a script of (+bytes | -index) steps: +n allocates n bytes,
  // -i releases the block returned by step i.  Returns (offsets, bytes in use, free blocks).
  m.def("_test_range_allocator", [](int64_t size, std::vector<int64_t> steps) {
    RangeAllocator ra;
    ra.reset(static_cast<size_t>(size));
    std::vector<int64_t> offs;
    for (int64_t st : steps) {
      if (st > 0) offs.push_back(ra.alloc(static_cast<size_t>(st)));
      else offs.push_back(ra.release(static_cast<size_t>(offs.at(static_cast<size_t>(-st - 1)))) ? 0 : -2);
    }
    return std::make_tuple(offs, static_cast<int64_t>(ra.bytes_in_use()), static_cast<int64_t>(ra.free_blocks()));
  });
  m.def("_nvls_pool_bytes_in_use", [](int device) { return NvlsUserPool::get(device).bytes_in_use(); });
  m.def("_nvls_pool_contains", [](const at::Tensor& t) {
    return t.is_cuda() && NvlsUserPool::get(t.device().index()).contains(t.data_ptr(), t.nbytes());
  });
  m.def("_kernel_launches", []() { return kern::launch_counter().load(); });
  // (tile_units, ntiles) the pipelined kernels derive for a 16-byte-unit index space and a grid
  m.def("_tile_plan", [](int64_t units, int nctas, int nthreads, int64_t tile_bytes) {
    int64_t tu = 0, nt = 0;
    kern::tile_plan_host(units, nctas, nthreads, tile_bytes, &tu, &nt);
    return std::make_pair(tu, nt);
  }, py::arg("units"), py::arg("nctas"), py::arg("nthreads") = 512, py::arg("tile_bytes") = 0);
  m.def("_mover_tile_bytes", &kern::mover_tile_bytes_host, py::arg("units"), py::arg("nctas"), py::arg("tile_bytes") = 0,
        py::arg("ws") = 2);
  m.attr("MAX_CTAS_PER_LANE") = kern::kMaxCtasPerLane;

  // ---- top-k kernels ------------------------------------------------------------------------
  m.def("_topk_select", &topk_select, py::arg("grad"), py::arg("residual"), py::arg("ratio"));

  // ---- emulation harness ----------------------------------------------------------------------
  py::class_<EmuGroup>(m, "EmuGroup")
      .def(py::init<int, int64_t, int64_t>(), py::arg("world_size"), py::arg("parity_bytes") = (32 << 20),
           py::arg("device_wait_us") = 2000000)
      .def_property_readonly("world_size", &EmuGroup::world_size)
      .def("allreduce", &EmuGroup::allreduce, py::arg("tensors"), py::arg("op") = "sum",
           py::arg("algo") = "oneshot", py::arg("wire") = "none", py::arg("scale") = 1.0, py::arg("ctas") = 0,
           py::arg("tiles") = 1, py::arg("push_gather") = false)
      .def("reduce_scatter", &EmuGroup::reduce_scatter, py::arg("outputs"), py::arg("inputs"),
           py::arg("op") = "sum", py::arg("ctas") = 0, py::arg("pitch") = 0)
      .def("allgather", &EmuGroup::allgather, py::arg("outputs"), py::arg("inputs"), py::arg("ctas") = 0,
           py::arg("tile_bytes") = 0, py::arg("pitch_bytes") = 0, py::arg("slice_bytes") = 0, py::arg("slice_offset") = 0)
      .def("broadcast", &EmuGroup::broadcast, py::arg("tensors"), py::arg("root"), py::arg("ctas") = 0,
           py::arg("tile_bytes") = 0)
      .def("set_debug_checks", &EmuGroup::set_debug_checks)
      .def("set_claimed_capacity", &EmuGroup::set_claimed_capacity)
      .def("poison_buffers", &EmuGroup::poison_buffers, py::arg("byte") = 0xFF)
      .def("barrier", &EmuGroup::barrier)
      .def("barrier_with_absent_rank", &EmuGroup::barrier_with_absent_rank)
      .def("status", &EmuGroup::status)
      .def("clear_status", &EmuGroup::clear_status)
      .def("topk_allreduce", &EmuGroup::topk_allreduce, py::arg("grads"), py::arg("residuals"), py::arg("ratio"),
           py::arg("scale") = 1.0, py::arg("ctas") = 0);

  // ---- host runtime unit hooks -----------------------------------------------------------------
  m.def(
      "_test_watchdog",
      [](int timeout_ms, bool arm, int wait_ms) {
        std::atomic<int> fired{0};
        Watchdog wd(std::chrono::milliseconds(timeout_ms), [&](uint32_t, const std::string&) { fired++; },
                    std::chrono::milliseconds(20));
        wd.start();
        wd.watch(1, "probe");
        if (arm) wd.touch(1);
        std::this_thread::sleep_for(std::chrono::milliseconds(wait_ms));
        wd.stop();
        return fired.load();
      },
      py::call_guard<py::gil_scoped_release>());
  m.def(
      "_test_engine",
      [](int workers, int depth, int n_ops, int fail_every) {
        // Returns (start order, completed, errors).
        std::vector<int> order;
        std::mutex mu;
        std::atomic<int> done{0}, errs{0};
        {
          HostEngine eng("probe", workers, static_cast<size_t>(depth));
          for (int i = 0; i < n_ops; ++i) {
            eng.submit(
                [&, i] {
                  {
                    std::lock_guard<std::mutex> g(mu);
                    order.push_back(i);
                  }
                  if (fail_every > 0 && i % fail_every == fail_every - 1) throw std::runtime_error("injected");
                },
                [&] { done++; }, [&](const std::string&) { errs++; });
          }
          eng.drain();
        }
        py::gil_scoped_acquire gil;
        return py::make_tuple(order, done.load(), errs.load());
      },
      py::call_guard<py::gil_scoped_release>());
  m.def("_test_mempool", []() {
    MemoryPool pool(4096);
    size_t first_cap, second_cap;
    void* first_ptr;
    {
      PooledBuffer a = pool.acquire(1000000);
      first_cap = a.capacity();
      first_ptr = a.data();
    }
    PooledBuffer b = pool.acquire(1100000);  // fits the 25 % head-room of the first buffer
    second_cap = b.capacity();
    bool reused = b.data() == first_ptr;
    size_t total = pool.total_allocated();
    b.release();
    pool.trim();
    return py::make_tuple(first_cap, second_cap, reused, total, pool.total_allocated());
  });

#ifdef MCCL_WITH_STFT
  // ---- STFT / iSTFT ---------------------------------------------------------------------------------
  m.def("_stft_forward", &stft_forward, py::arg("waveform"), py::arg("window"), py::arg("n_fft"),
        py::arg("hop_length"), py::arg("win_length"), py::arg("center") = true, py::arg("normalized") = false,
        py::arg("backend") = "auto");
  m.def("_stft_backward", &stft_backward, py::arg("grad_spec"), py::arg("window"), py::arg("n_fft"),
        py::arg("hop_length"), py::arg("win_length"), py::arg("center") = true, py::arg("normalized") = false,
        py::arg("length"), py::arg("backend") = "auto");
  m.def("_istft_forward", &istft_forward, py::arg("spec"), py::arg("window"), py::arg("n_fft"),
        py::arg("hop_length"), py::arg("win_length"), py::arg("center") = true, py::arg("normalized") = false,
        py::arg("length"), py::arg("backend") = "auto");
  m.def("_istft_backward", &istft_backward, py::arg("grad_waveform"), py::arg("window"), py::arg("n_fft"),
        py::arg("hop_length"), py::arg("win_length"), py::arg("center") = true, py::arg("normalized") = false,
        py::arg("n_frames"), py::arg("backend") = "auto");
#endif
}
