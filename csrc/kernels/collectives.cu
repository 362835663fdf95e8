// Fused collective kernels for NVLink 5 / NVSwitch peer memory (sm_100a).
//
// Every kernel here is ONE launch that moves the data over NVLink with plain
// 16-byte peer stores/loads, synchronises with release/acquire epoch flags in
// the peers' signal pads and performs the adjacent compute (reduction in fixed
// rank order, 1/world or user scale, fp32<->fp16/bf16 wire cast) in the same
// pass.  There is no ring: through NVSwitch every peer is one hop away at full
// bandwidth, so small messages use a one-shot exchange (latency optimal) and
// large ones a two-shot push-reduce-scatter + pull-allgather (bandwidth
// optimal: 2*(ws-1)/ws * N bytes per direction per GPU).
//
// Work split.  CTA b of every rank owns the same interleaved set of 16-byte
// units of every chunk, so CTA b only ever waits for CTA b of its peers and
// CTAs of one kernel never wait for each other.
//
// Determinism.  Contributions are combined in rank order 0..ws-1 with the
// accumulator type of vec.cuh, by exactly one reducer per element (two-shot,
// reduce_scatter) or by the same instruction sequence on every rank
// (one-shot), so all ranks end with bit-identical results.
//
// Replaces the reference's host-staged TCP algorithms A1-A8, B1-B3, C1-C2,
// D1-D2 (reference csrc/backend/ProcessGroupMCCL.cpp:1218-3307) and its Metal
// reduction shaders K1-K4 (reference csrc/metal/shaders.metal:196-731).
#include <cooperative_groups.h>
#include "kernels/coll_common.cuh"

namespace mccl {
namespace kern {

// Reducing kernels (one-shot, two-shot, reduce_scatter): one translation unit per world-size class.
enum ReduceKind : int { kOneShot = 0, kTwoShot = 1, kReduceScatter = 2 };
cudaError_t launch_reduce_ws2(int kind, const CollParams& p, DType dtype, DType wire, int ctas,
                              const LaunchCfg& cfg, cudaStream_t s);
cudaError_t launch_reduce_ws4(int kind, const CollParams& p, DType dtype, DType wire, int ctas,
                              const LaunchCfg& cfg, cudaStream_t s);
cudaError_t launch_reduce_ws8(int kind, const CollParams& p, DType dtype, DType wire, int ctas,
                              const LaunchCfg& cfg, cudaStream_t s);

namespace {

cudaError_t launch_reduce(int kind, const CollParams& p, DType dtype, DType wire, int ctas,
                          const LaunchCfg& cfg, cudaStream_t s) {
  const int ws = p.ctx[0].ws;
  if (ws == 2) return launch_reduce_ws2(kind, p, dtype, wire, ctas, cfg, s);
  if (ws <= 4) return launch_reduce_ws4(kind, p, dtype, wire, ctas, cfg, s);
  return launch_reduce_ws8(kind, p, dtype, wire, ctas, cfg, s);
}

// ---------------------------------------------------------------------------
// Byte movers: allgather (publish + pull), broadcast (root publishes, others
// pull), barrier (flag exchange only).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void copy_bytes(const CtaCtx& k, char* dst, const char* src, int64_t nbytes) {
  const bool al = is_aligned16(dst) && is_aligned16(src);
  const int64_t units = (nbytes + 15) / 16;
  const int64_t stride = static_cast<int64_t>(k.nctas) * k.nthreads;
  const int64_t first = static_cast<int64_t>(k.cta) * k.nthreads + k.tid;
  for (int64_t u0 = first; u0 < units; u0 += stride * kUnroll) {
    uint4 v[kUnroll];
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      int64_t u = u0 + i * stride;
      if (u < units)
        v[i] = ld_vec_guarded<uint8_t>(reinterpret_cast<const uint8_t*>(src), u, nbytes, al);
    }
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      int64_t u = u0 + i * stride;
      if (u < units) st_vec_guarded<uint8_t>(reinterpret_cast<uint8_t*>(dst), u, nbytes, al, v[i]);
    }
  }
}

__global__ void __launch_bounds__(512) allgather_kernel(const __grid_constant__ CollParams p) {
  CtaCtx k = make_ctx(p);
  const RankCtx& c = *k.c;
  if (!enter_collective(k)) return;
  const int64_t nbytes = p.count;
  const char* in = static_cast<const char*>(c.in);
  char* out = static_cast<char*>(c.out);
  // publish my block in my own arena (the arena side is padded: whole units)
  {
    char* pub = c.arena[c.rank] + p.parity_offset;
    const bool al = is_aligned16(in);
    const int64_t units = (nbytes + 15) / 16;
    const int64_t stride = static_cast<int64_t>(k.nctas) * k.nthreads;
    for (int64_t u = static_cast<int64_t>(k.cta) * k.nthreads + k.tid; u < units; u += stride)
      stg16(pub + u * 16, ld_vec_guarded<uint8_t>(reinterpret_cast<const uint8_t*>(in), u, nbytes, al));
  }
  signal_all(k, 0);
  // own block needs no peer: copy it while the flags travel
  if (out + static_cast<int64_t>(c.rank) * nbytes != in)
    copy_bytes(k, out + static_cast<int64_t>(c.rank) * nbytes, in, nbytes);
  if (!wait_all(k, 0)) return;
  for (int d = 1; d < c.ws; ++d) {
    int q = c.rank + d;
    if (q >= c.ws) q -= c.ws;
    copy_bytes(k, out + static_cast<int64_t>(q) * nbytes, c.arena[q] + p.parity_offset, nbytes);
  }
}

// Broadcast in two hops so the root's egress is N, not (ws-1)*N: the root
// publishes the payload; non-root rank r pulls slice r from the root, stores it
// and republishes it in its own arena; every non-root then pulls the remaining
// slices from the other non-roots (the root's own slice comes from the root).
__global__ void __launch_bounds__(512) broadcast_kernel(const __grid_constant__ CollParams p) {
  CtaCtx k = make_ctx(p);
  const RankCtx& c = *k.c;
  if (!enter_collective(k)) return;
  const int64_t nbytes = p.count;
  char* buf = static_cast<char*>(c.out);  // in-place tensor
  const int root = p.root;
  const int64_t units = (nbytes + 15) / 16;
  const int64_t slice_units = (units + c.ws - 1) / c.ws;
  const int64_t slice_bytes = slice_units * 16;
  auto slice_len = [&](int s) -> int64_t {
    int64_t b = static_cast<int64_t>(s) * slice_bytes, e = b + slice_bytes;
    if (e > nbytes) e = nbytes;
    return e > b ? e - b : 0;
  };
  if (c.rank == root) {
    char* pub = c.arena[root] + p.parity_offset;
    const bool al = is_aligned16(buf);
    const int64_t stride = static_cast<int64_t>(k.nctas) * k.nthreads;
    for (int64_t u = static_cast<int64_t>(k.cta) * k.nthreads + k.tid; u < units; u += stride)
      stg16(pub + u * 16, ld_vec_guarded<uint8_t>(reinterpret_cast<const uint8_t*>(buf), u, nbytes, al));
    signal_all(k, 0);
    return;
  }
  if (!wait_all(k, 0, root)) return;
  if (nbytes <= kBroadcastDirectBytes) {  // latency-bound: one hop straight from the root
    copy_bytes(k, buf, c.arena[root] + p.parity_offset, nbytes);
    return;
  }
  // hop 1: my slice, plus the root's slice, straight from the root
  {
    const char* rsrc = c.arena[root] + p.parity_offset;
    char* mine = c.arena[c.rank] + p.parity_offset;
    int64_t off = static_cast<int64_t>(c.rank) * slice_bytes;
    int64_t len = slice_len(c.rank);
    if (len > 0) {
      copy_bytes(k, mine + off, rsrc + off, (len + 15) / 16 * 16);  // arena copy: whole units
      copy_bytes(k, buf + off, rsrc + off, len);
    }
    int64_t roff = static_cast<int64_t>(root) * slice_bytes;
    int64_t rlen = slice_len(root);
    if (rlen > 0) copy_bytes(k, buf + roff, rsrc + roff, rlen);
  }
  signal_all(k, 1);
  // hop 2: the other non-roots' slices from their arenas
  for (int d = 1; d < c.ws; ++d) {
    int q = c.rank + d;
    if (q >= c.ws) q -= c.ws;
    if (q == root) continue;
    if (!wait_all(k, 1, q)) return;
    int64_t off = static_cast<int64_t>(q) * slice_bytes;
    int64_t len = slice_len(q);
    if (len > 0) copy_bytes(k, buf + off, c.arena[q] + p.parity_offset + off, len);
  }
}

__global__ void __launch_bounds__(128) barrier_kernel(const __grid_constant__ CollParams p) {
  CtaCtx k = make_ctx(p);
  if (!enter_collective(k)) return;
  signal_all(k, 0);
  wait_all(k, 0);
}

}  // namespace

int pick_ctas(size_t bytes, int ws, int requested) {
  // `bytes` is what one rank pushes over the links; one CTA per 16 KiB of it
  // (2 vectors per thread), up to the cap.  Small grids keep latency-bound
  // messages cheap, large ones are needed to fill NVLink.
  (void)ws;
  int cap = requested > 0 ? requested : 128;
  if (cap > kMaxCtas) cap = kMaxCtas;
  size_t want = (bytes + (16u << 10) - 1) / (16u << 10);
  if (want < 1) want = 1;
  if (want > static_cast<size_t>(cap)) want = cap;
  return static_cast<int>(want);
}

size_t oneshot_arena_bytes(size_t nbytes_wire, int ws) {
  return round_up(round_up(nbytes_wire, 16), 128) * ws;
}
size_t twoshot_arena_bytes(size_t nbytes_wire, int ws, bool push_gather) {
  size_t units = (nbytes_wire + 15) / 16;
  size_t chunk_units = (units + ws - 1) / ws;
  return round_up(chunk_units * 16, 128) * ws * (push_gather ? 2 : 1);
}

cudaError_t launch_allreduce_oneshot(const CollParams& p, DType dtype, DType wire, LaunchCfg cfg,
                                     cudaStream_t s) {
  int ctas = clamp_ctas(cfg.ctas > 0 ? cfg.ctas : pick_ctas(p.count * dtype_size(wire) * (p.ctx[0].ws - 1), p.ctx[0].ws, 0), cfg);
  return launch_reduce(kOneShot, p, dtype, wire, ctas, cfg, s);
}
cudaError_t launch_allreduce_twoshot(const CollParams& p, DType dtype, DType wire, LaunchCfg cfg,
                                     cudaStream_t s) {
  int ctas = clamp_ctas(cfg.ctas > 0 ? cfg.ctas : pick_ctas(p.count * dtype_size(wire), p.ctx[0].ws, 0), cfg);
  return launch_reduce(kTwoShot, p, dtype, wire, ctas, cfg, s);
}
cudaError_t launch_reduce_scatter(const CollParams& p, DType dtype, DType wire, LaunchCfg cfg,
                                  cudaStream_t s) {
  int ctas = clamp_ctas(
      cfg.ctas > 0 ? cfg.ctas : pick_ctas(p.count * dtype_size(wire) * p.ctx[0].ws, p.ctx[0].ws, 0), cfg);
  return launch_reduce(kReduceScatter, p, dtype, wire, ctas, cfg, s);
}
cudaError_t launch_allgather(const CollParams& p, LaunchCfg cfg, cudaStream_t s) {
  int ctas = clamp_ctas(cfg.ctas > 0 ? cfg.ctas : pick_ctas(p.count * p.ctx[0].ws, p.ctx[0].ws, 0), cfg);
  return do_launch(allgather_kernel, p, ctas, cfg.threads, cfg.emulate_ranks, s);
}
cudaError_t launch_broadcast(const CollParams& p, LaunchCfg cfg, cudaStream_t s) {
  int ctas = clamp_ctas(cfg.ctas > 0 ? cfg.ctas : pick_ctas(p.count, p.ctx[0].ws, 0), cfg);
  return do_launch(broadcast_kernel, p, ctas, cfg.threads, cfg.emulate_ranks, s);
}
cudaError_t launch_barrier(const CollParams& p, LaunchCfg cfg, cudaStream_t s) {
  return do_launch(barrier_kernel, p, 1, 128, cfg.emulate_ranks, s);
}

}  // namespace kern
}  // namespace mccl
