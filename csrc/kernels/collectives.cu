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
// Byte movers: allgather and broadcast.  Both PUSH: the sender loads each 16-byte unit of the
// user tensor once and stores it into the staging buffer of every receiver (one plain store per
// peer over NVLink, or ONE multimem.st through the NVSwitch multicast mapping when the group has
// an NVLS region), publishes a running tile count, and the receiver copies finished tiles from
// its own staging buffer into its output.  Stores are fire-and-forget, so the links run at their
// store rate, and because the work is cut into tiles (TilePlan) the receiver's copy-out of tile
// i overlaps the sender's push of tile i+1.  No rank ever stages its payload locally first.
// ---------------------------------------------------------------------------
constexpr int kDeep = 8;  // 16-byte loads in flight per thread in the local copy-out loops

template <bool kMC>
__device__ __forceinline__ char* stage_local(const CtaCtx& k) {
  return kMC ? k.c->nvls_uc + k.p->nvls_offset : k.c->arena[k.c->rank] + k.p->parity_offset;
}
template <bool kMC>
__device__ __forceinline__ size_t stage_capacity(const CtaCtx& k) {
  return kMC ? k.p->nvls_capacity : k.p->parity_capacity;
}
// Stores one unit at byte `off` of the staging buffer of every rank in `mask` (never this rank's
// own on the unicast path; the multicast store reaches all ranks, which is harmless).
template <bool kMC>
__device__ __forceinline__ void push16(const CtaCtx& k, size_t off, uint4 v, uint32_t mask) {
  const RankCtx& c = *k.c;
  if (kMC) {
    multimem_st16(c.nvls_mc + k.p->nvls_offset + off, v);
  } else {
    for (int d = 1; d < c.ws; ++d) {
      int q = c.rank + d;
      if (q >= c.ws) q -= c.ws;
      if ((mask >> q) & 1u) stg16(c.arena[q] + k.p->parity_offset + off, v);
    }
  }
}
// dst[u*16 ...] = staged units [u0, u1); `src` is unit-indexed from 0, dst holds nbytes bytes.
__device__ __forceinline__ void copy_units_out(const CtaCtx& k, char* dst, const char* src, int64_t u0, int64_t u1,
                                               int64_t nbytes) {
  const bool al = is_aligned16(dst);
  for (int64_t ub = u0; ub < u1; ub += static_cast<int64_t>(k.nthreads) * kDeep) {
    uint4 v[kDeep];
#pragma unroll
    for (int i = 0; i < kDeep; ++i) {
      const int64_t u = ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
      if (u < u1) v[i] = ldg16(src + u * 16);
    }
#pragma unroll
    for (int i = 0; i < kDeep; ++i) {
      const int64_t u = ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
      if (u < u1) st_vec_guarded<uint8_t>(reinterpret_cast<uint8_t*>(dst), u, nbytes, al, v[i]);
    }
  }
}

// allgather: staging slot r of every rank receives rank r's block.
template <bool kMC>
__global__ void __launch_bounds__(512) allgather_kernel(const __grid_constant__ CollParams p) {
  CtaCtx k = make_ctx(p);
  const RankCtx& c = *k.c;
  if (!enter_collective(k)) return;
  const int64_t nbytes = p.count;
  const int64_t pitch = p.out_pitch > 0 ? p.out_pitch : nbytes;
  const char* in = static_cast<const char*>(c.in);
  char* out = static_cast<char*>(c.out);
  const int64_t units = (nbytes + 15) / 16;
  const size_t slot_bytes = round_up(static_cast<size_t>(units) * 16, 128);
  if (!range_ok(k, 0, slot_bytes * c.ws, stage_capacity<kMC>(k), 10)) return;
  const TilePlan tp = TilePlan::make(units, k.nctas, k.nthreads, mover_tile_bytes(units, k.nctas, p.tile_bytes, c.ws));
  const int64_t my_tiles = tp.count_for(k.cta, k.nctas);
  const char* stage = stage_local<kMC>(k);
  const bool in_al = is_aligned16(in);
  char* own_out = out + static_cast<int64_t>(c.rank) * pitch;
  const bool own_copy = own_out != in;  // in-place allgather: the own block is already there
  const bool own_al = is_aligned16(own_out);
  const uint32_t peers = ((1u << c.ws) - 1u) & ~(1u << c.rank);
  for (int64_t it = 0; it <= my_tiles; ++it) {
    if (it < my_tiles) {  // push tile `it` of my block
      const int64_t u0 = tp.begin(k.cta, k.nctas, it), u1 = tp.end(k.cta, k.nctas, it);
      for (int64_t ub = u0; ub < u1; ub += static_cast<int64_t>(k.nthreads) * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int i = 0; i < kUnroll; ++i) {
          const int64_t u = ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
          if (u < u1) v[i] = ld_vec_guarded<uint8_t>(reinterpret_cast<const uint8_t*>(in), u, nbytes, in_al);
        }
#pragma unroll
        for (int i = 0; i < kUnroll; ++i) {
          const int64_t u = ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
          if (u < u1) {
            push16<kMC>(k, c.rank * slot_bytes + static_cast<size_t>(u) * 16, v[i], peers);
            if (own_copy) st_vec_guarded<uint8_t>(reinterpret_cast<uint8_t*>(own_out), u, nbytes, own_al, v[i]);
          }
        }
      }
      signal_all(k, 0, static_cast<uint32_t>(it + 1));
    }
    if (it >= 1) {  // copy tile it-1 of every peer's block out of my staging buffer
      if (!wait_mask(k, 0, peers, static_cast<uint32_t>(it))) return;
      const int64_t u0 = tp.begin(k.cta, k.nctas, it - 1), u1 = tp.end(k.cta, k.nctas, it - 1);
      for (int d = 1; d < c.ws; ++d) {
        int q = c.rank + d;
        if (q >= c.ws) q -= c.ws;
        copy_units_out(k, out + static_cast<int64_t>(q) * pitch, stage + q * slot_bytes, u0, u1, nbytes);
      }
    }
  }
}

// broadcast.  Direct form (two ranks, small messages, or the NVLS path where one multimem.st
// reaches everybody): the root pushes every tile to all receivers.  Two-hop form (unicast, large):
// the message is cut into ws-1 slices, one per non-root; the root pushes slice s only to its
// owner, which copies it out and forwards it to the other non-roots, so the root sends every byte
// once and every link carries about N bytes in each direction.  The staging buffer is an image of
// the message (unit U of the message at byte 16*U), tiles are cut in slice-local unit space and
// belong to the same CTA index on every rank.
template <bool kMC>
__global__ void __launch_bounds__(512) broadcast_kernel(const __grid_constant__ CollParams p) {
  CtaCtx k = make_ctx(p);
  const RankCtx& c = *k.c;
  if (!enter_collective(k)) return;
  const int64_t nbytes = p.count;
  char* buf = static_cast<char*>(c.out);  // in-place tensor
  const int root = p.root;
  const int64_t units = (nbytes + 15) / 16;
  if (!range_ok(k, 0, static_cast<size_t>(units) * 16, stage_capacity<kMC>(k), 20)) return;
  const char* stage = stage_local<kMC>(k);
  const uint32_t nonroot = ((1u << c.ws) - 1u) & ~(1u << root);
  const bool buf_al = is_aligned16(buf);
  const bool direct = kMC || c.ws == 2 || nbytes <= kBroadcastDirectBytes;
  if (direct) {
    const TilePlan tp = TilePlan::make(units, k.nctas, k.nthreads, p.tile_bytes);
    const int64_t my_tiles = tp.count_for(k.cta, k.nctas);
    for (int64_t it = 0; it < my_tiles; ++it) {
      const int64_t u0 = tp.begin(k.cta, k.nctas, it), u1 = tp.end(k.cta, k.nctas, it);
      if (c.rank == root) {
        for (int64_t ub = u0; ub < u1; ub += static_cast<int64_t>(k.nthreads) * kUnroll) {
          uint4 v[kUnroll];
#pragma unroll
          for (int i = 0; i < kUnroll; ++i) {
            const int64_t u = ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
            if (u < u1) v[i] = ld_vec_guarded<uint8_t>(reinterpret_cast<const uint8_t*>(buf), u, nbytes, buf_al);
          }
#pragma unroll
          for (int i = 0; i < kUnroll; ++i) {
            const int64_t u = ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
            if (u < u1) push16<kMC>(k, static_cast<size_t>(u) * 16, v[i], nonroot);
          }
        }
        signal_all(k, 0, static_cast<uint32_t>(it + 1));
      } else {
        if (!wait_mask(k, 0, 1u << root, static_cast<uint32_t>(it + 1))) return;
        copy_units_out(k, buf, stage, u0, u1, nbytes);
      }
    }
    return;
  }
  // ---- two hops ------------------------------------------------------------------------------
  const int ns = c.ws - 1;
  const int64_t slice_units = (units + ns - 1) / ns;
  const TilePlan tp = TilePlan::make(slice_units, k.nctas, k.nthreads,
                                     mover_tile_bytes(slice_units, k.nctas, p.tile_bytes, c.ws));
  const int64_t my_tiles = tp.count_for(k.cta, k.nctas);
  auto slice_base = [&](int q) -> int64_t { return static_cast<int64_t>(q < root ? q : q - 1) * slice_units; };
  if (c.rank == root) {
    for (int64_t it = 0; it < my_tiles; ++it) {
      const int64_t u0 = tp.begin(k.cta, k.nctas, it), u1 = tp.end(k.cta, k.nctas, it);
      for (int d = 1; d < c.ws; ++d) {
        int q = root + d;
        if (q >= c.ws) q -= c.ws;
        const int64_t base = slice_base(q);
        char* dst = c.arena[q] + p.parity_offset;
        for (int64_t ub = u0; ub < u1; ub += static_cast<int64_t>(k.nthreads) * kUnroll) {
          uint4 v[kUnroll];
#pragma unroll
          for (int i = 0; i < kUnroll; ++i) {
            const int64_t U = base + ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
            if (U < base + u1 && U < units)
              v[i] = ld_vec_guarded<uint8_t>(reinterpret_cast<const uint8_t*>(buf), U, nbytes, buf_al);
          }
#pragma unroll
          for (int i = 0; i < kUnroll; ++i) {
            const int64_t U = base + ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
            if (U < base + u1 && U < units) stg16(dst + U * 16, v[i]);
          }
        }
      }
      signal_all(k, 0, static_cast<uint32_t>(it + 1));
    }
    return;
  }
  const int64_t my_base = slice_base(c.rank);
  const uint32_t others = nonroot & ~(1u << c.rank);
  for (int64_t it = 0; it <= my_tiles; ++it) {
    if (it < my_tiles) {  // hop 1 arrived: keep tile `it` of my slice and forward it
      if (!wait_mask(k, 0, 1u << root, static_cast<uint32_t>(it + 1))) return;
      const int64_t u0 = tp.begin(k.cta, k.nctas, it), u1 = tp.end(k.cta, k.nctas, it);
      for (int64_t ub = u0; ub < u1; ub += static_cast<int64_t>(k.nthreads) * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int i = 0; i < kUnroll; ++i) {
          const int64_t U = my_base + ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
          if (U < my_base + u1 && U < units) v[i] = ldg16(stage + U * 16);
        }
#pragma unroll
        for (int i = 0; i < kUnroll; ++i) {
          const int64_t U = my_base + ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
          if (U < my_base + u1 && U < units) {
            push16<false>(k, static_cast<size_t>(U) * 16, v[i], others);
            st_vec_guarded<uint8_t>(reinterpret_cast<uint8_t*>(buf), U, nbytes, buf_al, v[i]);
          }
        }
      }
      signal_all(k, 1, static_cast<uint32_t>(it + 1));
    }
    if (it >= 1 && others != 0u) {  // hop 2 arrived: tile it-1 of the other non-roots' slices
      if (!wait_mask(k, 1, others, static_cast<uint32_t>(it))) return;
      const int64_t u0 = tp.begin(k.cta, k.nctas, it - 1), u1 = tp.end(k.cta, k.nctas, it - 1);
      for (int d = 1; d < c.ws; ++d) {
        int q = c.rank + d;
        if (q >= c.ws) q -= c.ws;
        if (q == root) continue;
        const int64_t base = slice_base(q);
        const int64_t e = base + u1 < units ? base + u1 : units;
        if (base + u0 < e) copy_units_out(k, buf, stage, base + u0, e, nbytes);
      }
    }
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
  int cap = requested > 0 ? requested : kMaxCtasPerLane;
  if (cap > kMaxCtasPerLane) cap = kMaxCtasPerLane;
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
size_t allgather_stage_bytes(size_t nbytes_per_rank, int ws) {
  return round_up(round_up(nbytes_per_rank, 16), 128) * ws;
}
size_t broadcast_stage_bytes(size_t nbytes) { return round_up(nbytes, 16); }

cudaError_t launch_allgather(const CollParams& p, LaunchCfg cfg, cudaStream_t s) {
  int ctas = clamp_ctas(cfg.ctas > 0 ? cfg.ctas : pick_ctas(p.count * p.ctx[0].ws, p.ctx[0].ws, 0), cfg);
  if (p.use_nvls) {
    if (cfg.emulate_ranks > 0 || p.ctx[0].nvls_mc == nullptr) return cudaErrorInvalidValue;
    return do_launch(allgather_kernel<true>, p, ctas, cfg.threads, 0, s);
  }
  return do_launch(allgather_kernel<false>, p, ctas, cfg.threads, cfg.emulate_ranks, s);
}
cudaError_t launch_broadcast(const CollParams& p, LaunchCfg cfg, cudaStream_t s) {
  int ctas = clamp_ctas(cfg.ctas > 0 ? cfg.ctas : pick_ctas(p.count, p.ctx[0].ws, 0), cfg);
  if (p.use_nvls) {
    if (cfg.emulate_ranks > 0 || p.ctx[0].nvls_mc == nullptr) return cudaErrorInvalidValue;
    return do_launch(broadcast_kernel<true>, p, ctas, cfg.threads, 0, s);
  }
  return do_launch(broadcast_kernel<false>, p, ctas, cfg.threads, cfg.emulate_ranks, s);
}

int64_t mover_tile_bytes_host(int64_t units, int nctas, int64_t tile_bytes, int ws) {
  return mover_tile_bytes(units, nctas, tile_bytes, ws);
}

void tile_plan_host(int64_t units, int nctas, int nthreads, int64_t tile_bytes, int64_t* tile_units, int64_t* ntiles) {
  const TilePlan t = TilePlan::make(units, nctas, nthreads, tile_bytes);
  *tile_units = t.tile_units;
  *ntiles = t.ntiles;
}
cudaError_t launch_barrier(const CollParams& p, LaunchCfg cfg, cudaStream_t s) {
  return do_launch(barrier_kernel, p, 1, 128, cfg.emulate_ranks, s);
}

}  // namespace kern
}  // namespace mccl
