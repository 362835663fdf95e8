// Shared device helpers of the collective kernels: 16-byte unit packing with the wire type,
// the per-CTA context, epoch entry and phase signalling, and the launch / dtype dispatch
// helpers.  Included by collectives.cu and by the per-world-size two-shot translation units.
#pragma once

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

// Waits for the same CTA index of every rank whose bit is set in `mask`.
__device__ __forceinline__ bool wait_mask(const CtaCtx& k, int phase, uint32_t mask, uint32_t count) {
  const RankCtx& c = *k.c;
  bool ok = true;
  if (k.tid < c.ws && ((mask >> k.tid) & 1u))
    ok = wait_epoch(sig_flag(c.arena[c.rank], lane_of(k.p->seq), phase, k.cta, k.tid), sig_value(k.p->seq, count), k.p->wait_ns, c.status,
                    static_cast<uint32_t>(phase), static_cast<uint32_t>(k.tid));
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// Debug-mode range check (CollParams::debug_checks): is [off, off + len) inside a buffer of `cap`
// bytes?  A violation is recorded as ERR_BOUNDS {seq, site, rank} and the caller skips the kernel
// body; nothing is accessed out of range and nothing traps.
__device__ __forceinline__ bool range_ok(const CtaCtx& k, size_t off, size_t len, size_t cap, uint32_t site) {
  if (!k.p->debug_checks) return true;
  if (off <= cap && len <= cap - off) return true;
  report_failure(k.c->status, ERR_BOUNDS, k.p->seq, site, static_cast<uint32_t>(k.c->rank));
  return false;
}

// ---- NVSwitch multicast (NVLS) accesses --------------------------------------------------------
// `multimem.st` stores 16 bytes to the same offset of every rank's buffer bound to the multicast
// object; `multimem.ld_reduce` returns the element-wise sum over all ranks' copies, added up inside
// the switch (16-bit floats are accumulated in fp32).  These are NVLS instructions on a multicast
// *address*; they have nothing to do with TMA cluster multicast, which this library never uses.
// The store is a weak one (ordered, like the plain peer stores, by the fence + release flag that
// follows it); a strong sys-scope store per 16 bytes measured markedly slower.
__device__ __forceinline__ void multimem_st16(void* mc, uint4 v) {
  asm volatile("multimem.st.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
template <typename W> struct MultimemSum;
template <> struct MultimemSum<float> {
  static __device__ __forceinline__ uint4 ld(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
  }
};
template <> struct MultimemSum<__half> {
  static __device__ __forceinline__ uint4 ld(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
  }
};
template <> struct MultimemSum<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
  }
};

// Tile geometry of the pipelined kernels.  The 16-byte-unit index space [0, units) is cut into
// tiles of `tile_units` (a whole number of nthreads * kUnroll batches); tile g belongs to CTA
// g % nctas on EVERY rank, so the CTA that wrote a tile on one rank is the CTA that reads it on
// another and a CTA only ever waits for its own index on its peers.
struct TilePlan {
  int64_t units, tile_units, ntiles;
  __host__ __device__ static TilePlan make(int64_t units, int nctas, int nthreads, int64_t tile_bytes) {
    TilePlan t;
    t.units = units;
    const int64_t batch = static_cast<int64_t>(nthreads) * kUnroll;
    const int64_t per_cta = (units + nctas - 1) / nctas;
    int64_t want = (tile_bytes > 0 ? tile_bytes : (128 << 10)) / 16;
    if (want > per_cta) want = per_cta;
    int64_t tu = (want + batch - 1) / batch * batch;
    const int64_t floor_tu = ((per_cta + kMaxTilesPerCta - 1) / kMaxTilesPerCta + batch - 1) / batch * batch;
    if (tu < floor_tu) tu = floor_tu;
    if (tu < batch) tu = batch;
    t.tile_units = tu;
    t.ntiles = (units + tu - 1) / tu;
    return t;
  }
  __host__ __device__ int64_t count_for(int cta, int nctas) const {
    return ntiles > cta ? (ntiles - cta + nctas - 1) / nctas : 0;
  }
  __host__ __device__ int64_t begin(int cta, int nctas, int64_t j) const {
    return (static_cast<int64_t>(cta) + j * nctas) * tile_units;
  }
  __host__ __device__ int64_t end(int cta, int nctas, int64_t j) const {
    const int64_t e = begin(cta, nctas, j) + tile_units;
    return e < units ? e : units;
  }
};

// Tile size of a byte mover.  With more than four ranks a rank's share per CTA is small, and one
// tile per CTA would serialise the two stages of the mover (push, then copy out or forward); such a
// share is cut into about four tiles of at least 64 KiB.  Measured on 8 ranks: a 128 MiB two-hop
// broadcast took 325 us with one 290 KB tile per CTA and slice (hop 1 then hop 2: no overlap).
// Depends only on (units, grid, tile_bytes, ws), so it is the same on every rank.
__host__ __device__ inline int64_t mover_tile_bytes(int64_t units, int nctas, int64_t tile_bytes, int ws) {
  int64_t tb = tile_bytes > 0 ? tile_bytes : (128 << 10);
  if (ws <= 4) return tb;
  const int64_t per_cta_bytes = (units + nctas - 1) / nctas * 16;
  if (per_cta_bytes >= 2 * tb) return tb;
  int64_t quarter = per_cta_bytes / 4;
  if (quarter < (64 << 10)) quarter = 64 << 10;
  return quarter < tb ? quarter : tb;
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

int clamp_ctas(int ctas, const LaunchCfg& cfg) {
  if (ctas < 1) ctas = 1;
  // Two lanes may run at once and every CTA that waits on a peer must be resident: a request above
  // the per-lane limit is clamped, not left to turn into a device-side wait timeout.
  if (ctas > kMaxCtasPerLane) ctas = kMaxCtasPerLane;
  // Emulated ranks share one device and must all be co-resident.
  if (cfg.emulate_ranks > 0 && ctas > 16) ctas = 16;
  return ctas;
}


}  // namespace
}  // namespace kern
}  // namespace mccl
