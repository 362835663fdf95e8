// MCCLOptions: every knob of a process group, resolved once at construction.
//
// `from_env()` reads the MCCL_* variables (which the Python MCCLConfig mirrors
// into os.environ).  Unlike the reference, where the options class was exposed
// to Python but never consumed (reference csrc/backend/Options.hpp:12-45,
// csrc/backend/Registration.cpp:54-61), an MCCLOptions instance passed through
// init_process_group(pg_options=...) is honoured: the create function copies
// it instead of reading the environment.
//
// Knobs that only meant something on Apple hardware (fast_math, shader_path,
// gpu_threshold, unified_collective, fp32_cpu_reduce, cpu_write_sync,
// event_sync, ring_algo, ring_pipeline, pipeline_depth, credit_min_chunk) are
// accepted and reported but change nothing on CUDA.
#pragma once

#include <torch/csrc/distributed/c10d/Backend.hpp>

#include <chrono>
#include <string>

#include "common/env.h"
#include "compression/compressor.h"

namespace mccl {

struct MCCLOptions : c10d::Backend::Options {
  explicit MCCLOptions(std::chrono::milliseconds timeout = kBackendDefaultTimeout)
      : c10d::Backend::Options("mccl", timeout) {}

  static c10::intrusive_ptr<MCCLOptions> create(
      std::chrono::milliseconds timeout = kBackendDefaultTimeout) {
    return c10::make_intrusive<MCCLOptions>(timeout);
  }

  // transport (host control/data plane)
  std::string transport = "auto";
  std::string listen_addr = "auto";
  int64_t port_base = 0;
  std::string ifname;
  int64_t chunk_bytes = 16 << 20;
  int64_t small_msg_threshold = 262144;  // CPU path: all-exchange below, two-shot above
  bool transport_crc = false;

  // compute / overlap
  bool fast_math = true;
  int64_t gpu_threshold = 4096;
  bool overlap_comm = true;
  int64_t max_queue_depth = 1024;

  // compression
  CompressionMode compression = CompressionMode::NONE;
  double topk_ratio = 0.01;
  std::string wire_dtype = "none";  // none | bf16 | fp16 : fused wire cast for fp32 CUDA allreduce

  // runtime
  std::chrono::milliseconds watchdog_timeout{300000};
  std::chrono::milliseconds heartbeat_interval{5000};

  // B200 data plane
  std::string algo = "auto";            // auto | oneshot | twoshot | nvls | staged
  std::string nvls = "auto";            // auto | 0 | 1 : NVLS (multimem) region and kernels; auto = use when the
                                        // devices support NVLink multicast, 0 = never create it, 1 = warn if unavailable
  int64_t nvls_bytes = 64ll << 20;      // one NVLS buffer (4 per rank)
  int64_t nvls_min_bytes = -2;          // allreduce: smallest payload for the NVLS kernel (-2: tuner table, -1: never)
  int64_t nvls_split_min_bytes = -2;    // NVLS allreduce: staging as separate kernels from this size (-2: tuner, -1: never)
  int64_t tile_bytes = 0;               // pipeline tile of the byte movers / NVLS kernels (0: tuner table)
  bool debug_checks = false;            // kernels verify their buffer ranges and report ERR_BOUNDS
  int64_t oneshot_max_bytes = -1;       // -1: tuner table
  int64_t comm_ctas = 0;                // 0: from message size
  int64_t tiles = 1;                    // two-shot pipeline tiles per CTA (1: bulk phases)
  std::string gather = "auto";          // two-shot allreduce second half: auto (tuner) | pull | push
  int64_t lanes = 2;                    // collectives in flight at once on the arena (1 or 2)
  int64_t arena_bytes = 128ll << 20;    // one parity buffer
  int64_t device_wait_us = 60ll * 1000 * 1000;
  bool blocking_wait = false;

  static c10::intrusive_ptr<MCCLOptions> from_env(std::chrono::milliseconds timeout) {
    auto o = create(timeout);
    o->transport = env_str("MCCL_TRANSPORT", "auto");
    o->listen_addr = env_str("MCCL_LISTEN_ADDR", "auto");
    o->port_base = env_int("MCCL_PORT_BASE", 0);
    o->ifname = env_str("MCCL_IFNAME", "");
    o->chunk_bytes = env_int("MCCL_CHUNK_BYTES", 16 << 20);
    o->small_msg_threshold = env_int("MCCL_SMALL_MSG_THRESHOLD", 262144);
    o->transport_crc = env_bool("MCCL_TRANSPORT_CRC", false);
    o->fast_math = env_bool("MCCL_FAST_MATH", true);
    o->gpu_threshold = env_int("MCCL_GPU_THRESHOLD", 4096);
    o->overlap_comm = env_bool("MCCL_OVERLAP_COMM", true);
    o->max_queue_depth = env_int("MCCL_MAX_QUEUE_DEPTH", 1024);
    o->compression = parse_compression_mode(env_str("MCCL_COMPRESSION", "none"));
    o->topk_ratio = env_double("MCCL_TOPK_RATIO", 0.01);
    o->wire_dtype = env_str("MCCL_WIRE_DTYPE", "none");
    o->watchdog_timeout = std::chrono::milliseconds(env_int("MCCL_WATCHDOG_TIMEOUT_MS", 300000));
    o->heartbeat_interval = std::chrono::milliseconds(env_int("MCCL_HEARTBEAT_INTERVAL_MS", 5000));
    o->algo = env_str("MCCL_ALGO", "auto");
    o->oneshot_max_bytes = env_int("MCCL_ONESHOT_MAX_BYTES", -1);
    o->comm_ctas = env_int("MCCL_COMM_CTAS", 0);
    o->nvls = env_str("MCCL_NVLS", "auto");
    o->nvls_bytes = env_int("MCCL_NVLS_BYTES", 64ll << 20);
    o->nvls_min_bytes = env_int("MCCL_NVLS_MIN_BYTES", -2);
    o->nvls_split_min_bytes = env_int("MCCL_NVLS_SPLIT_MIN_BYTES", -2);
    o->tile_bytes = env_int("MCCL_TILE_BYTES", 0);
    o->debug_checks = env_bool("MCCL_DEBUG_CHECKS", false);
    o->tiles = env_int("MCCL_TILES", 1);
    o->gather = env_str("MCCL_GATHER", "auto");
    // MCCL_COLLECTIVE_CONCURRENCY, when set, caps the lanes (1 = strictly one collective at a time)
    o->lanes = std::getenv("MCCL_COLLECTIVE_CONCURRENCY") ? std::min<int64_t>(2, collective_concurrency_requested()) : 2;
    o->arena_bytes = env_int("MCCL_ARENA_BYTES", 128ll << 20);
    int64_t wd_us = o->watchdog_timeout.count() * 1000;
    o->device_wait_us = env_int("MCCL_DEVICE_WAIT_US", std::min<int64_t>(60ll * 1000 * 1000, wd_us));
    o->blocking_wait = env_bool("MCCL_BLOCKING_WAIT", false);
    return o;
  }
};

}  // namespace mccl
