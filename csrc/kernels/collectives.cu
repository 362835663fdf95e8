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

#include <type_traits>

#include "kernels/api.h"
#include "kernels/flags.cuh"
#include "kernels/launch_count.h"
#include "kernels/vec.cuh"

namespace mccl {
namespace kern {

namespace {

constexpr int kUnroll = 4;
constexpr int64_t kBroadcastDirectBytes = 256 << 10;

__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void stg16(void* p, uint4 v) { __stcg(reinterpret_cast<uint4*>(p), v); }

__host__ __device__ inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// One 16-byte wire unit = N elements of W; the same N elements of T span
// sizeof(T)/sizeof(W) 16-byte vectors on the tensor side.
template <typename T, typename W>
struct Unit {
  static constexpr int N = 16 / sizeof(W);
  using Acc = typename Traits<T>::Acc;
  static_assert(std::is_same<typename Traits<T>::Acc, typename Traits<W>::Acc>::value,
                "tensor and wire types must share an accumulator type");
  static constexpr bool kSame = std::is_same<T, W>::value;

  static __device__ __forceinline__ void load_T(const T* base, int64_t e0, int64_t n, bool aligned,
                                                Acc* a) {
    if (aligned && e0 + N <= n) {
      constexpr int TV = sizeof(T) * N / 16;
      constexpr int PER = 16 / sizeof(T);
#pragma unroll
      for (int v = 0; v < TV; ++v) {
        typename VecOf<T>::U u;
        u.raw = ldg16(base + e0 + v * PER);
#pragma unroll
        for (int j = 0; j < PER; ++j) a[v * PER + j] = Traits<T>::load(u.e[j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < N; ++j) a[j] = (e0 + j < n) ? Traits<T>::load(base[e0 + j]) : Acc(0);
    }
  }
  static __device__ __forceinline__ void store_T(T* base, int64_t e0, int64_t n, bool aligned,
                                                 const Acc* a) {
    if (aligned && e0 + N <= n) {
      constexpr int TV = sizeof(T) * N / 16;
      constexpr int PER = 16 / sizeof(T);
#pragma unroll
      for (int v = 0; v < TV; ++v) {
        typename VecOf<T>::U u;
#pragma unroll
        for (int j = 0; j < PER; ++j) u.e[j] = Traits<T>::store(a[v * PER + j]);
        stg16(base + e0 + v * PER, u.raw);
      }
    } else {
#pragma unroll
      for (int j = 0; j < N; ++j)
        if (e0 + j < n) base[e0 + j] = Traits<T>::store(a[j]);
    }
  }
  static __device__ __forceinline__ uint4 pack_W(const Acc* a) {
    typename VecOf<W>::U u;
#pragma unroll
    for (int j = 0; j < N; ++j) u.e[j] = Traits<W>::store(a[j]);
    return u.raw;
  }
  static __device__ __forceinline__ void unpack_W(uint4 v, Acc* a) {
    typename VecOf<W>::U u;
    u.raw = v;
#pragma unroll
    for (int j = 0; j < N; ++j) a[j] = Traits<W>::load(u.e[j]);
  }
  // The value a rank contributes is what travels on the wire: round-trip the
  // local contribution through W as well, or ranks would disagree bitwise.
  static __device__ __forceinline__ void round_through_wire(Acc* a) {
    if (!kSame) {
#pragma unroll
      for (int j = 0; j < N; ++j) a[j] = Traits<W>::load(Traits<W>::store(a[j]));
    }
  }
};

struct CtaCtx {
  const RankCtx* c;
  const CollParams* p;
  int cta, nctas, tid, nthreads;
};

// Announces "this rank has started epoch seq" (in the epoch's lane) to every
// peer and waits until every peer has started epoch seq-2 of the same lane.  A
// lane is one stream, so a peer that has started seq-2 has finished seq-4, the
// previous user of this epoch's data buffer (seq % 4): nothing of it is still
// being read or written.  In steady state the wait is already satisfied.
__device__ __forceinline__ bool enter_collective(const CtaCtx& k) {
  const RankCtx& c = *k.c;
  bool ok = true;
  if (k.tid < c.ws && k.tid != c.rank) {
    const int lane = lane_of(k.p->seq);
    if (k.cta == 0) st_release_sys(entered_flag(c.arena[k.tid], lane, c.rank), k.p->seq);
    ok = wait_epoch(entered_flag(c.arena[c.rank], lane, k.tid), k.p->seq - 2, k.p->wait_ns, c.status, 100, k.tid);
  }
  if (k.tid == 0 && c.status != nullptr && *reinterpret_cast<volatile uint32_t*>(c.status) != 0u) ok = false;
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// Publishes "my CTA finished `phase`" to every rank (self included).
__device__ __forceinline__ void signal_all(const CtaCtx& k, int phase, uint32_t count = kSigDone) {
  const RankCtx& c = *k.c;
  __syncthreads();
  if (k.tid < c.ws) {
    fence_sys();
    st_release_sys(sig_flag(c.arena[k.tid], lane_of(k.p->seq), phase, k.cta, c.rank), sig_value(k.p->seq, count));
  }
}
// Waits for the same CTA index of every rank (or of `only`, if >= 0).
__device__ __forceinline__ bool wait_all(const CtaCtx& k, int phase, int only = -1, uint32_t count = kSigDone) {
  const RankCtx& c = *k.c;
  bool ok = true;
  if (k.tid < c.ws && (only < 0 || k.tid == only))
    ok = wait_epoch(sig_flag(c.arena[c.rank], lane_of(k.p->seq), phase, k.cta, k.tid), sig_value(k.p->seq, count), k.p->wait_ns, c.status,
                    static_cast<uint32_t>(phase), static_cast<uint32_t>(k.tid));
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

__device__ __forceinline__ void stamp(const CtaCtx& k, int slot) {
  if (k.c->stamps != nullptr && k.cta == 0 && k.tid == 0) k.c->stamps[slot] = globaltimer_ns();
}

__device__ __forceinline__ CtaCtx make_ctx(const CollParams& p) {
  CtaCtx k;
  k.c = &p.ctx[blockIdx.y];
  k.p = &p;
  k.cta = blockIdx.x;
  k.nctas = gridDim.x;
  k.tid = threadIdx.x;
  k.nthreads = blockDim.x;
  return k;
}

template <typename T, int OP>
__device__ __forceinline__ void combine(typename Traits<T>::Acc* acc, const typename Traits<T>::Acc* x, int n,
                                        int rt_op = 0) {
#pragma unroll
  for (int j = 0; j < 16; ++j)
    if (j < n) acc[j] = OP == kRuntimeOp ? Reduce<T, OP>::apply_rt(rt_op, acc[j], x[j]) : Reduce<T, OP>::apply(acc[j], x[j]);
}

// ---------------------------------------------------------------------------
// One-shot allreduce: every rank pushes its whole vector into slot[rank] of
// every peer, then reduces the ws slots locally.
// ---------------------------------------------------------------------------
template <typename T, typename W, int OP>
__device__ __forceinline__ void oneshot_reduce_phase(const CtaCtx& k, int64_t units, size_t slot_bytes,
                                                     char* local_buf) {
  using U = Unit<T, W>;
  using Acc = typename U::Acc;
  const RankCtx& c = *k.c;
  const T* in = static_cast<const T*>(c.in);
  T* out = static_cast<T*>(c.out);
  const int64_t n = k.p->count;
  const bool in_al = is_aligned16(in), out_al = is_aligned16(out);
  const int64_t stride = static_cast<int64_t>(k.nctas) * k.nthreads;
  for (int64_t u = static_cast<int64_t>(k.cta) * k.nthreads + k.tid; u < units; u += stride) {
    Acc acc[U::N], x[U::N];
    uint4 raw[kMaxWorld];
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      if (r < c.ws && r != c.rank) raw[r] = ldg16(local_buf + r * slot_bytes + u * 16);
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r) {
      if (r >= c.ws) break;
      if (r == c.rank) {
        U::load_T(in, u * U::N, n, in_al, x);
        U::round_through_wire(x);
      } else {
        U::unpack_W(raw[r], x);
      }
      if (r == 0) {
#pragma unroll
        for (int j = 0; j < U::N; ++j) acc[j] = x[j];
      } else {
        combine<T, OP>(acc, x, U::N);
      }
    }
    if (OP == AVG || k.p->scale != 1.0f) {
#pragma unroll
      for (int j = 0; j < U::N; ++j) acc[j] = Traits<T>::scale(acc[j], k.p->scale);
    }
    U::store_T(out, u * U::N, n, out_al, acc);
  }
}

template <typename T, typename W>
__global__ void __launch_bounds__(512) allreduce_oneshot_kernel(const __grid_constant__ CollParams p) {
  using U = Unit<T, W>;
  using Acc = typename U::Acc;
  CtaCtx k = make_ctx(p);
  const RankCtx& c = *k.c;
  if (!enter_collective(k)) return;

  const int64_t n = p.count;
  const int64_t units = (n + U::N - 1) / U::N;
  const size_t slot_bytes = round_up(static_cast<size_t>(units) * 16, 128);
  const T* in = static_cast<const T*>(c.in);
  const bool in_al = is_aligned16(in);
  const int64_t stride = static_cast<int64_t>(k.nctas) * k.nthreads;
  const int64_t first = static_cast<int64_t>(k.cta) * k.nthreads + k.tid;

  // push
  for (int64_t u0 = first; u0 < units; u0 += stride * kUnroll) {
    uint4 v[kUnroll];
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      int64_t u = u0 + i * stride;
      if (u < units) {
        Acc a[U::N];
        U::load_T(in, u * U::N, n, in_al, a);
        v[i] = U::pack_W(a);
      }
    }
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      int64_t u = u0 + i * stride;
      if (u < units) {
        for (int d = 1; d < c.ws; ++d) {
          int q = c.rank + d;
          if (q >= c.ws) q -= c.ws;
          stg16(c.arena[q] + p.parity_offset + c.rank * slot_bytes + u * 16, v[i]);
        }
      }
    }
  }
  signal_all(k, 0);
  if (!wait_all(k, 0)) return;

  char* local_buf = c.arena[c.rank] + p.parity_offset;
  switch (p.op) {
    case SUM: oneshot_reduce_phase<T, W, SUM>(k, units, slot_bytes, local_buf); break;
    case AVG: oneshot_reduce_phase<T, W, AVG>(k, units, slot_bytes, local_buf); break;
    case MIN: oneshot_reduce_phase<T, W, MIN>(k, units, slot_bytes, local_buf); break;
    case MAX: oneshot_reduce_phase<T, W, MAX>(k, units, slot_bytes, local_buf); break;
    default: oneshot_reduce_phase<T, W, PRODUCT>(k, units, slot_bytes, local_buf); break;
  }
}

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
// Reduces units [u0, u1) of the chunk this rank owns.  G units are in flight per
// thread so that G * ws independent 16-byte loads are outstanding: with few
// ranks one unit per thread would leave HBM idle.
template <typename T, typename W, int OP, int G>
__device__ __forceinline__ void reduce_tile_g(const CtaCtx& k, const T* in_chunk, int64_t own_n, T* out_chunk,
                                              int64_t u0, int64_t u1, size_t slot_bytes, char* local_buf,
                                              bool keep_wire, bool in_al, bool out_al) {
  using U = Unit<T, W>;
  using Acc = typename U::Acc;
  const RankCtx& c = *k.c;
  constexpr int MAXR = kMaxWorld / G;  // ranks this variant supports
  constexpr int TV = sizeof(T) * U::N / 16;  // 16-byte vectors of T per unit
  constexpr int PER = 16 / sizeof(T);
  for (int64_t ub = u0 + k.tid; ub < u1; ub += static_cast<int64_t>(k.nthreads) * G) {
    uint4 raw[G][MAXR];
    uint4 own[G][TV];
    // all loads of the group first (peers' slots and this rank's own input), then the math
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
        if (r == c.rank) {
          if (in_al && (u + 1) * U::N <= own_n) {
#pragma unroll
            for (int v = 0; v < TV; ++v) {
              typename VecOf<T>::U uu;
              uu.raw = own[g][v];
#pragma unroll
              for (int j = 0; j < PER; ++j) x[v * PER + j] = Traits<T>::load(uu.e[j]);
            }
          } else {
            U::load_T(in_chunk, u * U::N, own_n, in_al, x);
          }
          U::round_through_wire(x);
        } else {
          U::unpack_W(raw[g][r], x);
        }
        if (r == 0) {
#pragma unroll
          for (int j = 0; j < U::N; ++j) acc[j] = x[j];
        } else {
          combine<T, OP>(acc, x, U::N, k.p->op);
        }
      }
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
  }
}

template <typename T, typename W, int OP>
__device__ __forceinline__ void reduce_tile(const CtaCtx& k, const T* in_chunk, int64_t own_n, T* out_chunk,
                                            int64_t u0, int64_t u1, size_t slot_bytes, char* local_buf,
                                            bool keep_wire) {
  const bool in_al = is_aligned16(in_chunk), out_al = is_aligned16(out_chunk);
  const int ws = k.c->ws;
  if (ws <= 4) reduce_tile_g<T, W, OP, 2>(k, in_chunk, own_n, out_chunk, u0, u1, slot_bytes, local_buf, keep_wire, in_al, out_al);
  else reduce_tile_g<T, W, OP, 1>(k, in_chunk, own_n, out_chunk, u0, u1, slot_bytes, local_buf, keep_wire, in_al, out_al);
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
template <typename T, typename W, bool kAllGather, bool kSum>
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
  const T* in_chunk = in + static_cast<int64_t>(c.rank) * chunk_elems;
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
        const T* src = in + static_cast<int64_t>(q) * chunk_elems;
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
      reduce_tile<T, W, kSum ? SUM : kRuntimeOp>(k, in_chunk, own_n, out_chunk, u0, u1, slot_bytes, local_buf, kAllGather);
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

template <typename K>
cudaError_t do_launch(K kernel, const CollParams& p, int ctas, int threads, int emulate_ranks,
                      cudaStream_t s) {
  note_launch();
  if (emulate_ranks > 0) {
    void* args[] = {const_cast<CollParams*>(&p)};
    return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3(ctas, emulate_ranks),
                                       dim3(threads), args, 0, s);
  }
  kernel<<<dim3(ctas, 1), dim3(threads), 0, s>>>(p);
  return cudaGetLastError();
}

template <template <typename, typename> class Launcher>
cudaError_t dispatch_types(DType dtype, DType wire, const CollParams& p, int ctas, const LaunchCfg& cfg,
                           cudaStream_t s) {
  if (dtype == F32 && wire == BF16) return Launcher<float, __nv_bfloat16>::go(p, ctas, cfg, s);
  if (dtype == F32 && wire == F16) return Launcher<float, __half>::go(p, ctas, cfg, s);
  if (wire != dtype) return cudaErrorInvalidValue;
  switch (dtype) {
    case F32: return Launcher<float, float>::go(p, ctas, cfg, s);
    case F64: return Launcher<double, double>::go(p, ctas, cfg, s);
    case F16: return Launcher<__half, __half>::go(p, ctas, cfg, s);
    case BF16: return Launcher<__nv_bfloat16, __nv_bfloat16>::go(p, ctas, cfg, s);
    case I32: return Launcher<int32_t, int32_t>::go(p, ctas, cfg, s);
    case I64: return Launcher<int64_t, int64_t>::go(p, ctas, cfg, s);
    case U8: return Launcher<uint8_t, uint8_t>::go(p, ctas, cfg, s);
    case BOOL: return Launcher<bool8, bool8>::go(p, ctas, cfg, s);
    default: return cudaErrorInvalidValue;
  }
}

template <typename T, typename W> struct OneShotL {
  static cudaError_t go(const CollParams& p, int ctas, const LaunchCfg& cfg, cudaStream_t s) {
    return do_launch(allreduce_oneshot_kernel<T, W>, p, ctas, cfg.threads, cfg.emulate_ranks, s);
  }
};
template <typename T, typename W> struct TwoShotL {
  static cudaError_t go(const CollParams& p, int ctas, const LaunchCfg& cfg, cudaStream_t s) {
    if (p.op == SUM || p.op == AVG)
      return do_launch(twoshot_kernel<T, W, true, true>, p, ctas, cfg.threads, cfg.emulate_ranks, s);
    if (!std::is_same<T, W>::value) return cudaErrorInvalidValue;  // wire cast is defined for sums only
    return do_launch(twoshot_kernel<T, T, true, false>, p, ctas, cfg.threads, cfg.emulate_ranks, s);
  }
};
template <typename T, typename W> struct ReduceScatterL {
  static cudaError_t go(const CollParams& p, int ctas, const LaunchCfg& cfg, cudaStream_t s) {
    if (p.op == SUM || p.op == AVG)
      return do_launch(twoshot_kernel<T, W, false, true>, p, ctas, cfg.threads, cfg.emulate_ranks, s);
    if (!std::is_same<T, W>::value) return cudaErrorInvalidValue;
    return do_launch(twoshot_kernel<T, T, false, false>, p, ctas, cfg.threads, cfg.emulate_ranks, s);
  }
};

int clamp_ctas(int ctas, const LaunchCfg& cfg) {
  if (ctas < 1) ctas = 1;
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  // Emulated ranks share one device and must all be co-resident.
  if (cfg.emulate_ranks > 0 && ctas > 16) ctas = 16;
  return ctas;
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
  return dispatch_types<OneShotL>(dtype, wire, p, ctas, cfg, s);
}
cudaError_t launch_allreduce_twoshot(const CollParams& p, DType dtype, DType wire, LaunchCfg cfg,
                                     cudaStream_t s) {
  int ctas = clamp_ctas(cfg.ctas > 0 ? cfg.ctas : pick_ctas(p.count * dtype_size(wire), p.ctx[0].ws, 0), cfg);
  return dispatch_types<TwoShotL>(dtype, wire, p, ctas, cfg, s);
}
cudaError_t launch_reduce_scatter(const CollParams& p, DType dtype, DType wire, LaunchCfg cfg,
                                  cudaStream_t s) {
  int ctas = clamp_ctas(
      cfg.ctas > 0 ? cfg.ctas : pick_ctas(p.count * dtype_size(wire) * p.ctx[0].ws, p.ctx[0].ws, 0), cfg);
  return dispatch_types<ReduceScatterL>(dtype, wire, p, ctas, cfg, s);
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
