// Reducing collective kernels (one-shot allreduce, two-shot allreduce, reduce_scatter) as
// templates over the world-size class, and their per-class launcher.
#pragma once

#include "kernels/coll_common.cuh"

namespace mccl {
namespace kern {
namespace {

// ---------------------------------------------------------------------------
// Two-shot allreduce and reduce_scatter.
//   phase 0  push: rank r stores its part of chunk q into slot[r] of peer q
//   phase 1  owner reduces chunk (own input + ws-1 slots, rank order), applies
//            scale, keeps the wire-rounded result in slot[owner] and writes
//            its own output
//   phase 2  (allreduce only) pull: every rank loads the reduced chunks from
//            the owners' arenas straight into its output tensor
// With CollParams::push_gather the owner instead stores each reduced unit into
// slot[ws + owner] of every peer from inside the reduction loop (link traffic
// overlaps the HBM-bound reduction) and phase 2 is a local copy out of the arena;
// that needs twice the arena space.
// For reduce_scatter the "chunks" are the ws equal parts of the input list.
// ---------------------------------------------------------------------------
// Stores one reduced unit: wire-rounded copy for the peers (pushed to them, or kept in
// slot[owner] for them to pull) and the owner's own output.
template <typename T, typename W>
__device__ __forceinline__ void finish_unit(const CtaCtx& k, typename Unit<T, W>::Acc* acc, int64_t u, T* out_chunk,
                                            int64_t own_n, size_t slot_bytes, char* local_buf, bool keep_wire,
                                            bool out_al) {
  using U = Unit<T, W>;
  const RankCtx& c = *k.c;
  if (k.p->op == AVG || k.p->scale != 1.0f) {
#pragma unroll
    for (int j = 0; j < U::N; ++j) acc[j] = Traits<T>::scale(acc[j], k.p->scale);
  }
  if (keep_wire) {
    uint4 w = U::pack_W(acc);
    if (k.p->push_gather) {
      // hand the reduced unit to every peer now: the stores ride the links while the
      // next loads of this loop are in flight
      for (int d = 1; d < c.ws; ++d) {
        int q = c.rank + d;
        if (q >= c.ws) q -= c.ws;
        stg16(c.arena[q] + k.p->parity_offset + (c.ws + c.rank) * slot_bytes + u * 16, w);
      }
    } else {
      stg16(local_buf + c.rank * slot_bytes + u * 16, w);
    }
    U::unpack_W(w, acc);  // the owner outputs exactly what the peers will receive
  }
  U::store_T(out_chunk, u * U::N, own_n, out_al, acc);
}

// This rank's own contribution to unit u, rounded through the wire type like the peers' were.
template <typename T, typename W, int TV>
__device__ __forceinline__ void own_unit(const uint4* own, bool fast, const T* in_chunk, int64_t u, int64_t own_n,
                                         bool in_al, typename Unit<T, W>::Acc* x) {
  using U = Unit<T, W>;
  constexpr int PER = 16 / sizeof(T);
  if (fast) {
#pragma unroll
    for (int v = 0; v < TV; ++v) {
      typename VecOf<T>::U uu;
      uu.raw = own[v];
#pragma unroll
      for (int j = 0; j < PER; ++j) x[v * PER + j] = Traits<T>::load(uu.e[j]);
    }
  } else {
    U::load_T(in_chunk, u * U::N, own_n, in_al, x);
  }
  U::round_through_wire(x);
}

// Reduces units [u0, u1) of the chunk this rank owns.  The reduction is bound by HBM
// latency, not bandwidth, unless enough loads are outstanding: 64 CTAs x 512 threads need
// about a dozen 16-byte loads in flight per thread.  G units are therefore processed per
// thread and iteration, all their loads (G x (peers + own input)) issued before any math.
// MAXR is the largest world size the variant supports (register array bound).
template <typename T, typename W, int OP, int G, int MAXR>
__device__ __forceinline__ void reduce_tile_g(const CtaCtx& k, const T* in_chunk, int64_t own_n, T* out_chunk,
                                              int64_t u0, int64_t u1, size_t slot_bytes, char* local_buf,
                                              bool keep_wire, bool in_al, bool out_al) {
  using U = Unit<T, W>;
  using Acc = typename U::Acc;
  const RankCtx& c = *k.c;
  constexpr int TV = sizeof(T) * U::N / 16;  // 16-byte vectors of T per unit
  constexpr int PER = 16 / sizeof(T);
  for (int64_t ub = u0 + k.tid; ub < u1; ub += static_cast<int64_t>(k.nthreads) * G) {
    uint4 raw[G][MAXR];
    uint4 own[G][TV];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int64_t u = ub + static_cast<int64_t>(g) * k.nthreads;
#pragma unroll
      for (int r = 0; r < MAXR; ++r)
        if (u < u1 && r < c.ws && r != c.rank) raw[g][r] = ldg16(local_buf + r * slot_bytes + u * 16);
      if (u < u1 && in_al && (u + 1) * U::N <= own_n) {
#pragma unroll
        for (int v = 0; v < TV; ++v) own[g][v] = ldg16(in_chunk + u * U::N + v * PER);
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int64_t u = ub + static_cast<int64_t>(g) * k.nthreads;
      if (u >= u1) break;
      Acc acc[U::N], x[U::N];
#pragma unroll
      for (int r = 0; r < MAXR; ++r) {
        if (r >= c.ws) break;
        if (r == c.rank) own_unit<T, W, TV>(own[g], in_al && (u + 1) * U::N <= own_n, in_chunk, u, own_n, in_al, x);
        else U::unpack_W(raw[g][r], x);
        if (r == 0) {
#pragma unroll
          for (int j = 0; j < U::N; ++j) acc[j] = x[j];
        } else {
          combine<T, OP>(acc, x, U::N, k.p->op);
        }
      }
      finish_unit<T, W>(k, acc, u, out_chunk, own_n, slot_bytes, local_buf, keep_wire, out_al);
    }
  }
}

// Two ranks: one peer slot per unit, so the register array holds exactly the loads that are
// issued and G can be large.  Operand order stays rank order.
template <typename T, typename W, int OP, int G>
__device__ __forceinline__ void reduce_tile_pair(const CtaCtx& k, const T* in_chunk, int64_t own_n, T* out_chunk,
                                                 int64_t u0, int64_t u1, size_t slot_bytes, char* local_buf,
                                                 bool keep_wire, bool in_al, bool out_al) {
  using U = Unit<T, W>;
  using Acc = typename U::Acc;
  const RankCtx& c = *k.c;
  constexpr int TV = sizeof(T) * U::N / 16;
  constexpr int PER = 16 / sizeof(T);
  const char* peer_slot = local_buf + (1 - c.rank) * slot_bytes;
  for (int64_t ub = u0 + k.tid; ub < u1; ub += static_cast<int64_t>(k.nthreads) * G) {
    uint4 raw[G];
    uint4 own[G][TV];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int64_t u = ub + static_cast<int64_t>(g) * k.nthreads;
      if (u < u1) raw[g] = ldg16(peer_slot + u * 16);
      if (u < u1 && in_al && (u + 1) * U::N <= own_n) {
#pragma unroll
        for (int v = 0; v < TV; ++v) own[g][v] = ldg16(in_chunk + u * U::N + v * PER);
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int64_t u = ub + static_cast<int64_t>(g) * k.nthreads;
      if (u >= u1) break;
      Acc mine[U::N], theirs[U::N];
      own_unit<T, W, TV>(own[g], in_al && (u + 1) * U::N <= own_n, in_chunk, u, own_n, in_al, mine);
      U::unpack_W(raw[g], theirs);
      if (c.rank == 0) {
        combine<T, OP>(mine, theirs, U::N, k.p->op);
        finish_unit<T, W>(k, mine, u, out_chunk, own_n, slot_bytes, local_buf, keep_wire, out_al);
      } else {
        combine<T, OP>(theirs, mine, U::N, k.p->op);
        finish_unit<T, W>(k, theirs, u, out_chunk, own_n, slot_bytes, local_buf, keep_wire, out_al);
      }
    }
  }
}

template <typename T, typename W, int OP, int CLS>
__device__ __forceinline__ void reduce_tile(const CtaCtx& k, const T* in_chunk, int64_t own_n, T* out_chunk,
                                            int64_t u0, int64_t u1, size_t slot_bytes, char* local_buf,
                                            bool keep_wire) {
  const bool in_al = is_aligned16(in_chunk), out_al = is_aligned16(out_chunk);
  // units whose own input spans two 16-byte vectors (fp32 over a 16-bit wire) get half the depth
  constexpr int kWide = sizeof(T) * Unit<T, W>::N / 16 > 1 ? 2 : 1;
  if (CLS == 2) reduce_tile_pair<T, W, OP, 8 / kWide>(k, in_chunk, own_n, out_chunk, u0, u1, slot_bytes, local_buf, keep_wire, in_al, out_al);
  else if (CLS == 4) reduce_tile_g<T, W, OP, 4 / kWide, 4>(k, in_chunk, own_n, out_chunk, u0, u1, slot_bytes, local_buf, keep_wire, in_al, out_al);
  else reduce_tile_g<T, W, OP, 2 / kWide, kMaxWorld>(k, in_chunk, own_n, out_chunk, u0, u1, slot_bytes, local_buf, keep_wire, in_al, out_al);
}

// Tile-pipelined two-shot.  A CTA's share of the chunk index space is cut into
// tiles of nthreads * kTileUnroll 16-byte units; in iteration `it` the CTA
// pushes tile it, reduces tile it-1 (whose peer pushes were signalled one
// iteration ago) and pulls tile it-2, so link traffic, the HBM-bound reduction
// and the flag round trips overlap instead of forming three bulk-synchronous
// phases.
constexpr int kTileUnroll = 4;
constexpr int kPullUnroll = 8;  // remote loads are round trips: keep more of them in flight

// kSum: SUM/AVG (AVG differs only by the scale); otherwise MIN/MAX/PRODUCT at run time.
// CLS: world-size class (2: exactly two ranks, 4: three or four, 8: five to eight); it fixes the
// depth of the reduction loop, and each class is compiled in its own translation unit so that
// the register allocation of one does not spill the others.
template <typename T, typename W, bool kAllGather, bool kSum, int CLS>
__global__ void __launch_bounds__(512) twoshot_kernel(const __grid_constant__ CollParams p) {
  using U = Unit<T, W>;
  using Acc = typename U::Acc;
  CtaCtx k = make_ctx(p);
  const RankCtx& c = *k.c;
  stamp(k, 0);
  if (!enter_collective(k)) return;
  stamp(k, 1);

  const T* in = static_cast<const T*>(c.in);
  T* out = static_cast<T*>(c.out);
  // allreduce: count = total elements, chunks are unit-aligned slices of it.
  // reduce_scatter: count = elements per chunk, chunk q starts at q * count.
  int64_t chunk_units, chunk_elems;
  if (kAllGather) {
    const int64_t units = (p.count + U::N - 1) / U::N;
    chunk_units = (units + c.ws - 1) / c.ws;
    chunk_elems = chunk_units * U::N;
  } else {
    chunk_units = (p.count + U::N - 1) / U::N;
    chunk_elems = p.count;
  }
  const int64_t total = kAllGather ? p.count : p.count * c.ws;
  const size_t slot_bytes = round_up(static_cast<size_t>(chunk_units) * 16, 128);
  if (!range_ok(k, 0, slot_bytes * c.ws * (p.push_gather ? 2 : 1), p.parity_capacity, 50)) return;
  auto chunk_len = [&](int q) -> int64_t {  // valid elements of chunk q
    int64_t b = static_cast<int64_t>(q) * chunk_elems;
    int64_t e = b + chunk_elems;
    if (e > total) e = total;
    return e > b ? e - b : 0;
  };

  // A tile is a whole number of batches (nthreads * kTileUnroll units); the
  // requested tiles per CTA fix its size.  One tile per CTA = bulk phases.
  const int64_t batch_units = static_cast<int64_t>(k.nthreads) * kTileUnroll;
  const int64_t want_tiles = p.tiles > 1 ? p.tiles : 1;
  const int64_t per_cta_units = (chunk_units + k.nctas - 1) / k.nctas;
  int64_t tile_units = ((per_cta_units + want_tiles - 1) / want_tiles + batch_units - 1) / batch_units * batch_units;
  if (tile_units < batch_units) tile_units = batch_units;
  const int64_t ntiles_total = (chunk_units + tile_units - 1) / tile_units;
  // tiles g = cta, cta + nctas, ... belong to this CTA
  const int64_t my_tiles = ntiles_total > k.cta ? (ntiles_total - k.cta + k.nctas - 1) / k.nctas : 0;
  auto tile_begin = [&](int64_t j) { return (static_cast<int64_t>(k.cta) + j * k.nctas) * tile_units; };
  auto tile_end = [&](int64_t j) {
    int64_t e = tile_begin(j) + tile_units;
    return e < chunk_units ? e : chunk_units;
  };
  char* local_buf = c.arena[c.rank] + p.parity_offset;
  // distance between the starts of consecutive input chunks (reduce_scatter may read a slice of
  // every chunk of a larger input: pitch > count)
  const int64_t in_pitch = (!kAllGather && p.chunk_pitch > 0) ? p.chunk_pitch : chunk_elems;
  const T* in_chunk = in + static_cast<int64_t>(c.rank) * in_pitch;
  const int64_t own_n = chunk_len(c.rank);
  T* out_chunk = kAllGather ? out + static_cast<int64_t>(c.rank) * chunk_elems : out;
  const int last_stage = kAllGather ? 2 : 1;

  for (int64_t it = 0; it < my_tiles + last_stage; ++it) {
    // ---- stage 0: push my part of tile `it` of every peer's chunk ------------
    if (it < my_tiles) {
      const int64_t u0 = tile_begin(it), u1 = tile_end(it);
      for (int d = 1; d < c.ws; ++d) {
        int q = c.rank + d;
        if (q >= c.ws) q -= c.ws;
        const T* src = in + static_cast<int64_t>(q) * in_pitch;
        const int64_t src_n = chunk_len(q);
        const bool al = is_aligned16(src);
        char* dst = c.arena[q] + p.parity_offset + c.rank * slot_bytes;
        for (int64_t ub = u0; ub < u1; ub += batch_units) {
          uint4 v[kTileUnroll];
#pragma unroll
          for (int i = 0; i < kTileUnroll; ++i) {
            const int64_t u = ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
            if (u < u1) {
              if (U::kSame && al && (u + 1) * U::N <= src_n) {
                v[i] = ldg16(src + u * U::N);
              } else {
                Acc a[U::N];
                U::load_T(src, u * U::N, src_n, al, a);
                v[i] = U::pack_W(a);
              }
            }
          }
#pragma unroll
          for (int i = 0; i < kTileUnroll; ++i) {
            const int64_t u = ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
            if (u < u1) stg16(dst + u * 16, v[i]);
          }
        }
      }
      if (it == my_tiles - 1) stamp(k, 2);
      signal_all(k, 0, static_cast<uint32_t>(it + 1));
    }
    // ---- stage 1: reduce tile it-1 of the chunk this rank owns ---------------
    if (it >= 1 && it - 1 < my_tiles) {
      if (!wait_all(k, 0, -1, static_cast<uint32_t>(it))) return;
      if (it == my_tiles) stamp(k, 3);
      const int64_t u0 = tile_begin(it - 1), u1 = tile_end(it - 1);
      reduce_tile<T, W, kSum ? SUM : kRuntimeOp, CLS>(k, in_chunk, own_n, out_chunk, u0, u1, slot_bytes, local_buf, kAllGather);
      if (it == my_tiles) stamp(k, 4);
      if (kAllGather) signal_all(k, 1, static_cast<uint32_t>(it));
    }
    // ---- stage 2: pull reduced tile it-2 from its owners ----------------------
    if (kAllGather && it >= 2 && it - 2 < my_tiles) {
      if (!wait_all(k, 1, -1, static_cast<uint32_t>(it - 1))) return;
      if (it == my_tiles + 1) stamp(k, 5);
      const int64_t u0 = tile_begin(it - 2), u1 = tile_end(it - 2);
      for (int d = 1; d < c.ws; ++d) {
        int q = c.rank + d;
        if (q >= c.ws) q -= c.ws;
        // pull mode: the owner's arena over the link; push mode: the copy the owner left here
        const char* src = p.push_gather ? local_buf + (c.ws + q) * slot_bytes
                                        : c.arena[q] + p.parity_offset + q * slot_bytes;
        T* dst = out + static_cast<int64_t>(q) * chunk_elems;
        const int64_t dst_n = chunk_len(q);
        const bool al = is_aligned16(dst);
        for (int64_t ub = u0; ub < u1; ub += static_cast<int64_t>(k.nthreads) * kPullUnroll) {
          uint4 v[kPullUnroll];
#pragma unroll
          for (int i = 0; i < kPullUnroll; ++i) {
            const int64_t u = ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
            if (u < u1) v[i] = ldg16(src + u * 16);
          }
#pragma unroll
          for (int i = 0; i < kPullUnroll; ++i) {
            const int64_t u = ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
            if (u < u1 && u * U::N < dst_n) {
              if (U::kSame && al && (u + 1) * U::N <= dst_n) {
                stg16(dst + u * U::N, v[i]);
              } else {
                Acc a[U::N];
                U::unpack_W(v[i], a);
                U::store_T(dst, u * U::N, dst_n, al, a);
              }
            }
          }
        }
      }
    }
  }
  stamp(k, 6);
}


// ---------------------------------------------------------------------------
// One-shot allreduce: every rank pushes its whole vector into slot[rank] of
// every peer, then reduces the ws slots locally (same rank order, same
// instruction sequence on every rank: bit-identical results).  CTA b owns the
// contiguous unit range [b * per, (b + 1) * per) in both phases, so it only
// waits for CTA b of its peers.
// ---------------------------------------------------------------------------
template <typename T, typename W, bool kSum, int CLS>
__global__ void __launch_bounds__(512) allreduce_oneshot_kernel(const __grid_constant__ CollParams p) {
  using U = Unit<T, W>;
  using Acc = typename U::Acc;
  CtaCtx k = make_ctx(p);
  const RankCtx& c = *k.c;
  stamp(k, 0);
  if (!enter_collective(k)) return;
  stamp(k, 1);

  const int64_t n = p.count;
  const int64_t units = (n + U::N - 1) / U::N;
  const size_t slot_bytes = round_up(static_cast<size_t>(units) * 16, 128);
  if (!range_ok(k, 0, slot_bytes * c.ws, p.parity_capacity, 40)) return;
  const T* in = static_cast<const T*>(c.in);
  const bool in_al = is_aligned16(in);
  const int64_t per = (units + k.nctas - 1) / k.nctas;
  const int64_t u0 = static_cast<int64_t>(k.cta) * per;
  const int64_t u1 = u0 + per < units ? u0 + per : units;

  // push
  for (int64_t ub = u0; ub < u1; ub += static_cast<int64_t>(k.nthreads) * kUnroll) {
    uint4 v[kUnroll];
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      const int64_t u = ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
      if (u < u1) {
        if (U::kSame && in_al && (u + 1) * U::N <= n) {
          v[i] = ldg16(in + u * U::N);
        } else {
          Acc a[U::N];
          U::load_T(in, u * U::N, n, in_al, a);
          v[i] = U::pack_W(a);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      const int64_t u = ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
      if (u < u1) {
        for (int d = 1; d < c.ws; ++d) {
          int q = c.rank + d;
          if (q >= c.ws) q -= c.ws;
          stg16(c.arena[q] + p.parity_offset + c.rank * slot_bytes + u * 16, v[i]);
        }
      }
    }
  }
  stamp(k, 2);
  signal_all(k, 0);
  if (!wait_all(k, 0)) return;
  stamp(k, 3);

  char* local_buf = c.arena[c.rank] + p.parity_offset;
  if (u0 < u1)
    reduce_tile<T, W, kSum ? SUM : kRuntimeOp, CLS>(k, in, n, static_cast<T*>(c.out), u0, u1, slot_bytes, local_buf, false);
  stamp(k, 4);
  stamp(k, 6);
}

template <int CLS> struct ReduceClass {
  template <typename T, typename W> struct AllReduce {
    static cudaError_t go(const CollParams& p, int ctas, const LaunchCfg& cfg, cudaStream_t s) {
      if (p.op == SUM || p.op == AVG)
        return do_launch(twoshot_kernel<T, W, true, true, CLS>, p, ctas, cfg.threads, cfg.emulate_ranks, s);
      if (!std::is_same<T, W>::value) return cudaErrorInvalidValue;  // wire cast is defined for sums only
      return do_launch(twoshot_kernel<T, T, true, false, CLS>, p, ctas, cfg.threads, cfg.emulate_ranks, s);
    }
  };
  template <typename T, typename W> struct ReduceScatter {
    static cudaError_t go(const CollParams& p, int ctas, const LaunchCfg& cfg, cudaStream_t s) {
      if (p.op == SUM || p.op == AVG)
        return do_launch(twoshot_kernel<T, W, false, true, CLS>, p, ctas, cfg.threads, cfg.emulate_ranks, s);
      if (!std::is_same<T, W>::value) return cudaErrorInvalidValue;
      return do_launch(twoshot_kernel<T, T, false, false, CLS>, p, ctas, cfg.threads, cfg.emulate_ranks, s);
    }
  };
  template <typename T, typename W> struct OneShot {
    static cudaError_t go(const CollParams& p, int ctas, const LaunchCfg& cfg, cudaStream_t s) {
      if (p.op == SUM || p.op == AVG)
        return do_launch(allreduce_oneshot_kernel<T, W, true, CLS>, p, ctas, cfg.threads, cfg.emulate_ranks, s);
      if (!std::is_same<T, W>::value) return cudaErrorInvalidValue;
      return do_launch(allreduce_oneshot_kernel<T, T, false, CLS>, p, ctas, cfg.threads, cfg.emulate_ranks, s);
    }
  };
  // kind: 0 one-shot allreduce, 1 two-shot allreduce, 2 reduce_scatter
  static cudaError_t launch(int kind, const CollParams& p, DType dtype, DType wire, int ctas,
                            const LaunchCfg& cfg, cudaStream_t s) {
    if (kind == 0) return dispatch_types<OneShot>(dtype, wire, p, ctas, cfg, s);
    if (kind == 1) return dispatch_types<AllReduce>(dtype, wire, p, ctas, cfg, s);
    return dispatch_types<ReduceScatter>(dtype, wire, p, ctas, cfg, s);
  }
};

}  // namespace
}  // namespace kern
}  // namespace mccl
