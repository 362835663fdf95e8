// Top-k gradient compression kernels (sm_100a): exact radix select with error
// feedback, and the fused sparse exchange + deterministic scatter-add.
// See topk_api.h for the pipeline.  Semantics follow the host TopKCompressor
// (csrc/compression/compressor.cpp), which is the oracle in the tests:
// k = max(1, floor(n*ratio)), adjusted = g + residual, ties towards the lower
// index, pairs sorted by index, residual = adjusted with sent entries zeroed
// (reference csrc/compression/TopKCompression.cpp:42-152).
#include <cuda_bf16.h>

#include <algorithm>

#include "kernels/api.h"
#include "kernels/flags.cuh"
#include "kernels/launch_count.h"
#include "kernels/topk_api.h"

namespace mccl {
namespace kern {

namespace {

// ---- scratch layout ---------------------------------------------------------
struct TopkState {
  uint32_t prefix;    // magnitude bits fixed so far (aligned to the low end)
  uint32_t need;      // how many more elements must come from the current bin
  uint32_t threshold; // final: 31-bit magnitude key of the k-th element
  uint32_t need_eq;   // final: number of ties (key == threshold) to take
  uint32_t ncand;     // candidates appended by the collect pass (may exceed the capacity)
  uint32_t overflow;  // 1: the candidate list did not fit -> the full-vector refinement runs
  uint32_t ticket[5]; // "last block done" counters: adjust, collect, level 1, level 2, count
  uint32_t pad[1];
};
struct TopkScratch {
  uint32_t hist0[kTopkBins0];
  uint32_t hist1[kTopkBins12];
  uint32_t hist2[kTopkBins12];
  TopkState st;
  uint32_t blk_gt[kTopkMaxBlocks];
  uint32_t blk_eq[kTopkMaxBlocks];
  uint32_t off_gt[kTopkMaxBlocks];
  uint32_t off_eq[kTopkMaxBlocks];
};

__device__ __forceinline__ uint32_t mag_key(float a) { return __float_as_uint(a) & 0x7FFFFFFFu; }

// level 0: bits 30..18 (13), level 1: bits 17..9 (9), level 2: bits 8..0 (9)
__device__ __forceinline__ uint32_t digit_of(uint32_t key, int level) {
  return level == 0 ? (key >> 18) : level == 1 ? ((key >> 9) & 0x1FFu) : (key & 0x1FFu);
}
__device__ __forceinline__ bool prefix_matches(uint32_t key, int level, uint32_t prefix) {
  return level == 0 ? true : level == 1 ? ((key >> 18) == prefix) : ((key >> 9) == prefix);
}
__device__ __forceinline__ uint32_t* hist_of(TopkScratch* sc, int level) {
  return level == 0 ? sc->hist0 : level == 1 ? sc->hist1 : sc->hist2;
}

__global__ void topk_clear_kernel(TopkScratch* sc) {
  uint32_t* h = sc->hist0;  // hist0, hist1, hist2 are contiguous
  for (int i = threadIdx.x + blockIdx.x * blockDim.x; i < kTopkBins0 + 2 * kTopkBins12; i += blockDim.x * gridDim.x) h[i] = 0;
  if (blockIdx.x == 0 && threadIdx.x < sizeof(TopkState) / 4) reinterpret_cast<uint32_t*>(&sc->st)[threadIdx.x] = 0;
}

// Exclusive scan of one value per thread over a block of up to 1024 threads.
__device__ __forceinline__ uint32_t block_excl_scan(uint32_t v, uint32_t* warp_sums, uint32_t& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = lane < (blockDim.x >> 5) ? warp_sums[lane] : 0;
    uint32_t winc = w;
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t t = __shfl_up_sync(0xFFFFFFFFu, winc, o);
      if (lane >= o) winc += t;
    }
    warp_sums[lane] = winc - w;            // exclusive prefix of warp sums
    if (lane == 31) warp_sums[32] = winc;  // block total
  }
  __syncthreads();
  uint32_t excl = warp_sums[warp] + inc - v;
  total = warp_sums[32];
  __syncthreads();
  return excl;
}

// Walks a histogram from the top bin down (as a parallel suffix scan: every thread owns a run of
// consecutive bins) and fixes the next digit: the first bin, from the top, at which the running
// count reaches `need`.  Called by every thread of one block; `hist` may be global or shared.
__device__ void pick_bin_block(TopkScratch* sc, const uint32_t* hist, int nbins, int level, uint32_t k) {
  __shared__ uint32_t wsum[33];
  __shared__ uint32_t s_digit, s_cum;
  const uint32_t need = level == 0 ? k : sc->st.need;
  const uint32_t old_prefix = sc->st.prefix;
  if (threadIdx.x == 0) {
    s_digit = 0;
    s_cum = 0xFFFFFFFFu;
  }
  const int per = (nbins + static_cast<int>(blockDim.x) - 1) / static_cast<int>(blockDim.x);
  const int top = nbins - 1 - static_cast<int>(threadIdx.x) * per;  // my bins: top, top-1, ..., top-per+1
  uint32_t mine = 0;
  for (int j = 0; j < per; ++j)
    if (top - j >= 0) mine += hist[top - j];
  uint32_t total;
  uint32_t above = block_excl_scan(mine, wsum, total);  // count in bins above my run
  for (int j = 0; j < per; ++j) {
    const int bin = top - j;
    if (bin < 0) break;
    const uint32_t c = hist[bin];
    if (above < need && above + c >= need) {
      s_digit = static_cast<uint32_t>(bin);
      s_cum = above;
    }
    above += c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t digit = s_digit, cum = s_cum;
    if (cum == 0xFFFFFFFFu) {  // fewer than `need` elements in total: take everything
      digit = 0;
      cum = total - hist[0];
    }
    const uint32_t prefix = level == 0 ? digit : ((old_prefix << 9) | digit);
    sc->st.prefix = prefix;
    sc->st.need = need - cum;  // elements still to take from inside the chosen bin
    if (level == 2) {
      sc->st.threshold = prefix;
      sc->st.need_eq = need - cum;
    }
    __threadfence();
  }
  __syncthreads();
}

// True in exactly one block of the grid: the one that finishes last.  All blocks' global writes
// made before the call are visible to that block afterwards.
__device__ __forceinline__ bool last_block_done(uint32_t* ticket) {
  __shared__ bool s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last) __threadfence();
  return s_last;
}

// Pass 1.  a = g + e, e = a, histogram of the top digit; the last block picks the digit.
// kVec: 16-byte accesses (all three arrays 16-byte aligned); otherwise element-wise.
template <bool kBf16, bool kVec>
__global__ void __launch_bounds__(512) topk_adjust_hist_kernel(const void* __restrict__ grad,
                                                               float* __restrict__ res, int64_t n,
                                                               TopkScratch* sc, uint32_t k) {
  extern __shared__ uint32_t sh[];  // kTopkBins0 counters
  for (int i = threadIdx.x; i < kTopkBins0; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (kVec) {
    const int64_t nv = n / 4;
    for (int64_t v = tid0; v < nv; v += stride) {
      float4 r = reinterpret_cast<const float4*>(res)[v];
      float g0, g1, g2, g3;
      if (kBf16) {
        const uint2 raw = reinterpret_cast<const uint2*>(grad)[v];
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        g0 = __low2float(lo); g1 = __high2float(lo); g2 = __low2float(hi); g3 = __high2float(hi);
      } else {
        const float4 g = reinterpret_cast<const float4*>(grad)[v];
        g0 = g.x; g1 = g.y; g2 = g.z; g3 = g.w;
      }
      r.x += g0; r.y += g1; r.z += g2; r.w += g3;
      reinterpret_cast<float4*>(res)[v] = r;
      atomicAdd(&sh[digit_of(mag_key(r.x), 0)], 1u);
      atomicAdd(&sh[digit_of(mag_key(r.y), 0)], 1u);
      atomicAdd(&sh[digit_of(mag_key(r.z), 0)], 1u);
      atomicAdd(&sh[digit_of(mag_key(r.w), 0)], 1u);
    }
  }
  for (int64_t i = (kVec ? n / 4 * 4 : 0) + tid0; i < n; i += stride) {
    float g = kBf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(grad)[i])
                    : static_cast<const float*>(grad)[i];
    float a = g + res[i];
    res[i] = a;
    atomicAdd(&sh[digit_of(mag_key(a), 0)], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kTopkBins0; i += blockDim.x)
    if (sh[i]) atomicAdd(&sc->hist0[i], sh[i]);
  if (last_block_done(&sc->st.ticket[0])) pick_bin_block(sc, sc->hist0, kTopkBins0, 0, k);
}

// Blocks own contiguous ranges (multiples of 4096 elements) so that compaction preserves index order.
__host__ __device__ __forceinline__ int64_t block_span(int64_t n, int nblocks) {
  int64_t per = (n + nblocks - 1) / nblocks;
  return (per + 4095) / 4096 * 4096;
}
__device__ __forceinline__ void block_range(int64_t n, int nblocks, int b, int64_t& lo, int64_t& hi) {
  const int64_t per = block_span(n, nblocks);
  lo = static_cast<int64_t>(b) * per;
  hi = lo + per;
  if (lo > n) lo = n;
  if (hi > n) hi = n;
}

// Pass 2.  One read of the residual: counts, per block, the elements above the chosen top-digit bin
// (selected for sure) and appends the elements INSIDE the bin, as (index, key) pairs, to a
// candidate list; the remaining 18 bits of the threshold are then found on that short list instead
// of on two more passes over the whole vector.  The last block does that refinement, turns the
// candidates into exact per-block counts of selected and tied elements and scans them.  If the bin
// holds more elements than the list can take (heavily tied data), `overflow` is set and the
// full-vector refinement kernels below take over.
constexpr int kStageCap = 2048;  // candidates a block collects in shared memory before one global append

__global__ void __launch_bounds__(1024) topk_collect_refine_kernel(const float* __restrict__ res, int64_t n,
                                                                   TopkScratch* sc, uint2* __restrict__ cand,
                                                                   uint32_t cap, uint32_t k) {
  __shared__ uint32_t s_gt, s_cnt, s_base;
  __shared__ uint2 stage[kStageCap];
  __shared__ uint32_t sh_hist[kTopkBins12];
  __shared__ uint32_t sh_gt[kTopkMaxBlocks], sh_eq[kTopkMaxBlocks];
  __shared__ uint32_t wsum[33];
  if (threadIdx.x == 0) s_gt = s_cnt = 0;
  for (int i = threadIdx.x; i < kTopkBins12; i += blockDim.x) sh_hist[i] = 0;
  __syncthreads();
  const uint32_t b0 = sc->st.prefix;
  int64_t lo, hi;
  block_range(n, gridDim.x, blockIdx.x, lo, hi);
  uint32_t gt = 0;
  const int lane = threadIdx.x & 31;
  const bool vec = (reinterpret_cast<uintptr_t>(res) & 15) == 0;
  // Candidates go to the shared staging list first (one shared atomic per warp and element slot) and
  // from there to the global list in bulk (one global atomic per flush), so the global counter is
  // touched a few times per block instead of once per warp and iteration.
  auto flush = [&]() {
    __syncthreads();
    const uint32_t cnt = s_cnt < kStageCap ? s_cnt : kStageCap;
    if (threadIdx.x == 0 && cnt) s_base = atomicAdd(&sc->st.ncand, cnt);
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < cnt; i += blockDim.x) {
      const uint32_t pos = s_base + i;
      if (pos < cap) cand[pos] = stage[i];
      else sc->st.overflow = 1u;
    }
    __syncthreads();
    if (threadIdx.x == 0) s_cnt = 0;
    __syncthreads();
  };
  // the next tile's elements are loaded before this tile's barriers, so the load latency hides
  // behind the ballots and the block synchronisation
  auto load_tile = [&](int64_t t0, float* a) {
    const int64_t i0 = t0 + static_cast<int64_t>(threadIdx.x) * 4;
    a[0] = a[1] = a[2] = a[3] = 0.f;
    if (vec && i0 + 4 <= hi) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(res + i0));
      a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (i0 + j < hi) a[j] = res[i0 + j];
    }
  };
  float nxt[4];
  if (lo < hi) load_tile(lo, nxt);
  for (int64_t t0 = lo; t0 < hi; t0 += 4096) {
    const int64_t i0 = t0 + static_cast<int64_t>(threadIdx.x) * 4;
    float a[4] = {nxt[0], nxt[1], nxt[2], nxt[3]};
    if (t0 + 4096 < hi) load_tile(t0 + 4096, nxt);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t key = mag_key(a[j]);
      const uint32_t d = key >> 18;
      const bool in = i0 + j < hi;
      gt += in && d > b0;
      const bool inbin = in && d == b0;
      const uint32_t m = __ballot_sync(0xFFFFFFFFu, inbin);
      if (m != 0u) {
        const int leader = __ffs(m) - 1;
        uint32_t base = 0;
        if (lane == leader) base = atomicAdd(&s_cnt, __popc(m));
        base = __shfl_sync(0xFFFFFFFFu, base, leader);
        if (inbin) {
          atomicAdd(&sh_hist[digit_of(key, 1)], 1u);  // second-level histogram of the bin, for free
          const uint32_t pos = base + __popc(m & ((1u << lane) - 1u));
          const uint2 e = make_uint2(static_cast<uint32_t>(i0 + j), key);
          if (pos < kStageCap) {
            stage[pos] = e;
          } else {  // more than the staging list holds within one tile: append directly (rare)
            const uint32_t gp = atomicAdd(&sc->st.ncand, 1u);
            if (gp < cap) cand[gp] = e;
            else sc->st.overflow = 1u;
          }
        }
      }
    }
    __syncthreads();
    if (s_cnt > kStageCap / 2) flush();  // uniform across the block: s_cnt is read after the barrier
  }
  flush();
  for (int o = 16; o > 0; o >>= 1) gt += __shfl_down_sync(0xFFFFFFFFu, gt, o);
  if (lane == 0 && gt) atomicAdd(&s_gt, gt);
  __syncthreads();
  if (threadIdx.x == 0) sc->blk_gt[blockIdx.x] = s_gt;
  for (int i = threadIdx.x; i < kTopkBins12; i += blockDim.x)
    if (sh_hist[i]) atomicAdd(&sc->hist1[i], sh_hist[i]);
  if (!last_block_done(&sc->st.ticket[1])) return;

  // ---- refinement on the candidate list (one block) ----------------------------------------------
  // Level 1 comes from the histogram the blocks have just merged; level 2 and the per-block counts
  // are two passes over the list, eight independent loads per thread in flight.
  if (*reinterpret_cast<volatile uint32_t*>(&sc->st.overflow) != 0u) return;
  const uint32_t nc = *reinterpret_cast<volatile uint32_t*>(&sc->st.ncand);
  constexpr int kRef = 8;
  pick_bin_block(sc, sc->hist1, kTopkBins12, 1, k);
  for (int i = threadIdx.x; i < kTopkBins12; i += blockDim.x) sh_hist[i] = 0;
  __syncthreads();
  {
    const uint32_t prefix = sc->st.prefix;
    for (uint32_t c0 = threadIdx.x; c0 < nc; c0 += blockDim.x * kRef) {
      uint32_t key[kRef];
#pragma unroll
      for (int i = 0; i < kRef; ++i) {
        const uint32_t c = c0 + i * blockDim.x;
        key[i] = c < nc ? __ldcg(&cand[c].y) : 0xFFFFFFFFu;  // the sentinel matches no prefix
      }
#pragma unroll
      for (int i = 0; i < kRef; ++i)
        if (key[i] != 0xFFFFFFFFu && prefix_matches(key[i], 2, prefix)) atomicAdd(&sh_hist[digit_of(key[i], 2)], 1u);
    }
  }
  __syncthreads();
  pick_bin_block(sc, sh_hist, kTopkBins12, 2, k);
  const uint32_t T = sc->st.threshold;
  for (int i = threadIdx.x; i < kTopkMaxBlocks; i += blockDim.x) sh_gt[i] = sh_eq[i] = 0;
  __syncthreads();
  const int64_t span = block_span(n, gridDim.x);
  for (uint32_t c0 = threadIdx.x; c0 < nc; c0 += blockDim.x * kRef) {
    uint2 e[kRef];
#pragma unroll
    for (int i = 0; i < kRef; ++i) {
      const uint32_t c = c0 + i * blockDim.x;
      e[i] = c < nc ? __ldcg(&cand[c]) : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int i = 0; i < kRef; ++i) {
      if (c0 + i * blockDim.x >= nc) continue;
      const int b = static_cast<int>(e[i].x / span);
      if (e[i].y > T) atomicAdd(&sh_gt[b], 1u);
      else if (e[i].y == T) atomicAdd(&sh_eq[b], 1u);
    }
  }
  __syncthreads();
  // one block per thread: totals and exclusive offsets (gridDim.x <= kTopkMaxBlocks == blockDim.x)
  const int b = threadIdx.x;
  const bool live = b < static_cast<int>(gridDim.x);
  const uint32_t g = live ? __ldcg(&sc->blk_gt[b]) + sh_gt[b] : 0u;
  const uint32_t e = live ? sh_eq[b] : 0u;
  uint32_t tot;
  const uint32_t og = block_excl_scan(g, wsum, tot);
  const uint32_t oe = block_excl_scan(e, wsum, tot);
  if (live) {
    sc->blk_gt[b] = g;
    sc->blk_eq[b] = e;
    sc->off_gt[b] = og;
    sc->off_eq[b] = oe;
  }
}

// ---- full-vector refinement: only does work when the candidate list overflowed -------------------
__global__ void __launch_bounds__(512) topk_hist_level_kernel(const float* __restrict__ res, int64_t n,
                                                              TopkScratch* sc, int level, uint32_t k) {
  if (sc->st.overflow == 0u) return;
  if (level == 1) {
    // the collect pass has already merged the complete second-level histogram of the chosen bin
    // (every element of the bin is counted there, whether or not its candidate entry fitted)
    if (blockIdx.x == 0) pick_bin_block(sc, sc->hist1, kTopkBins12, 1, k);
    return;
  }
  __shared__ uint32_t sh[kTopkBins12];
  for (int i = threadIdx.x; i < kTopkBins12; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const uint32_t prefix = sc->st.prefix;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    uint32_t key = mag_key(res[i]);
    if (prefix_matches(key, level, prefix)) atomicAdd(&sh[digit_of(key, level)], 1u);
  }
  __syncthreads();
  uint32_t* h = hist_of(sc, level);
  for (int i = threadIdx.x; i < kTopkBins12; i += blockDim.x)
    if (sh[i]) atomicAdd(&h[i], sh[i]);
  if (last_block_done(&sc->st.ticket[1 + level])) pick_bin_block(sc, h, kTopkBins12, level, k);
}

__global__ void __launch_bounds__(1024) topk_count_scan_kernel(const float* __restrict__ res, int64_t n,
                                                               TopkScratch* sc) {
  if (sc->st.overflow == 0u) return;
  __shared__ uint32_t s_gt, s_eq;
  __shared__ uint32_t wsum[33];
  if (threadIdx.x == 0) s_gt = s_eq = 0;
  __syncthreads();
  const uint32_t T = sc->st.threshold;
  int64_t lo, hi;
  block_range(n, gridDim.x, blockIdx.x, lo, hi);
  uint32_t gt = 0, eq = 0;
  for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    uint32_t key = mag_key(res[i]);
    gt += key > T;
    eq += key == T;
  }
  for (int o = 16; o > 0; o >>= 1) {
    gt += __shfl_down_sync(0xFFFFFFFFu, gt, o);
    eq += __shfl_down_sync(0xFFFFFFFFu, eq, o);
  }
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(&s_gt, gt);
    atomicAdd(&s_eq, eq);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    sc->blk_gt[blockIdx.x] = s_gt;
    sc->blk_eq[blockIdx.x] = s_eq;
  }
  if (!last_block_done(&sc->st.ticket[4])) return;
  const int b = threadIdx.x;
  const bool live = b < static_cast<int>(gridDim.x);
  const uint32_t g = live ? __ldcg(&sc->blk_gt[b]) : 0u;
  const uint32_t e = live ? __ldcg(&sc->blk_eq[b]) : 0u;
  uint32_t tot;
  const uint32_t og = block_excl_scan(g, wsum, tot);
  const uint32_t oe = block_excl_scan(e, wsum, tot);
  if (live) {
    sc->off_gt[b] = og;
    sc->off_eq[b] = oe;
  }
}

// Pass 3.  Ordered compaction: every thread owns 4 consecutive elements, one block-wide scan per
// 4096 elements gives each selected element its position in the index-sorted output.
__global__ void __launch_bounds__(1024) topk_compact_kernel(float* __restrict__ res, int64_t n, TopkScratch* sc,
                                                            uint2* __restrict__ pairs, uint32_t k) {
  __shared__ uint32_t ws_a[33];
  const uint32_t T = sc->st.threshold;
  const uint32_t need_eq = sc->st.need_eq;
  int64_t lo, hi;
  block_range(n, gridDim.x, blockIdx.x, lo, hi);
  uint32_t eq_base = sc->off_eq[blockIdx.x];
  // selected elements that precede this block
  uint32_t out_base = sc->off_gt[blockIdx.x] + (eq_base < need_eq ? eq_base : need_eq);
  const bool vec = (reinterpret_cast<uintptr_t>(res) & 15) == 0;
  auto load_tile = [&](int64_t t0, float* a) {
    const int64_t i0 = t0 + static_cast<int64_t>(threadIdx.x) * 4;
    a[0] = a[1] = a[2] = a[3] = 0.f;
    if (vec && i0 + 4 <= hi) {
      const float4 v = *reinterpret_cast<const float4*>(res + i0);
      a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (i0 + j < hi) a[j] = res[i0 + j];
    }
  };
  float nxt[4];
  if (lo < hi) load_tile(lo, nxt);
  for (int64_t t0 = lo; t0 < hi; t0 += 4096) {
    const int64_t i0 = t0 + static_cast<int64_t>(threadIdx.x) * 4;
    float a[4] = {nxt[0], nxt[1], nxt[2], nxt[3]};
    if (t0 + 4096 < hi) load_tile(t0 + 4096, nxt);  // in flight during this tile's scan
    uint32_t gt[4], eq[4], ngt = 0, neq = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t key = mag_key(a[j]);
      const bool in = i0 + j < hi;
      gt[j] = in && key > T;
      eq[j] = in && key == T;
      ngt += gt[j];
      neq += eq[j];
    }
    // one scan of both counts: at most 4096 of each per tile, so 16 bits apiece are enough
    uint32_t total;
    const uint32_t ex = block_excl_scan((ngt << 16) | neq, ws_a, total);
    uint32_t my_gt = ex >> 16, my_eq = eq_base + (ex & 0xFFFFu);
    const uint32_t eq_taken_before_tile = eq_base < need_eq ? eq_base : need_eq;
    bool wrote = false;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool sel = gt[j] || (eq[j] && my_eq < need_eq);
      if (sel) {
        const uint32_t eq_taken = my_eq < need_eq ? my_eq : need_eq;
        const uint32_t pos = out_base + my_gt + (eq_taken - eq_taken_before_tile);
        if (pos < k) {
          pairs[pos] = make_uint2(static_cast<uint32_t>(i0 + j), __float_as_uint(a[j]));
          a[j] = 0.f;  // sent: nothing left to feed back for this entry
          wrote = true;
        }
      }
      my_gt += gt[j];
      my_eq += eq[j];
    }
    if (wrote) {
      if (vec && i0 + 4 <= hi) {
        *reinterpret_cast<float4*>(res + i0) = make_float4(a[0], a[1], a[2], a[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (i0 + j < hi) res[i0 + j] = a[j];
      }
    }
    const uint32_t t_gt = total >> 16, t_eq = total & 0xFFFFu;
    const uint32_t eq_after = eq_base + t_eq;
    out_base += t_gt + ((eq_after < need_eq ? eq_after : need_eq) - eq_taken_before_tile);
    eq_base = eq_after;
  }
}

// ---- scatter ------------------------------------------------------------------
__device__ __forceinline__ int64_t lower_bound_idx(const uint2* list, int64_t k, uint32_t target) {
  int64_t lo = 0, hi = k;
  while (lo < hi) {
    int64_t mid = (lo + hi) >> 1;
    if (list[mid].x < target) lo = mid + 1;
    else hi = mid;
  }
  return lo;
}

// dense[range of this CTA] = scale * sum over lists (in order) of their entries.
template <bool kBf16>
__device__ __forceinline__ void scatter_lists(void* dense, int64_t n, const uint2* const* lists, int nlists,
                                              int64_t k, float scale, int cta, int nctas) {
  int64_t per = (n + nctas - 1) / nctas;
  per = (per + 7) / 8 * 8;  // keeps 16-byte alignment of each range for both dtypes
  int64_t lo = static_cast<int64_t>(cta) * per, hi = lo + per;
  if (lo > n) lo = n;
  if (hi > n) hi = n;
  // zero-fill
  if (kBf16) {
    __nv_bfloat16* d = static_cast<__nv_bfloat16*>(dense);
    for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) d[i] = __float2bfloat16_rn(0.f);
  } else {
    float* d = static_cast<float*>(dense);
    for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) d[i] = 0.f;
  }
  __syncthreads();
  for (int r = 0; r < nlists; ++r) {
    const uint2* list = lists[r];
    const int64_t b = lower_bound_idx(list, k, static_cast<uint32_t>(lo));
    const int64_t e = hi >= n ? k : lower_bound_idx(list, k, static_cast<uint32_t>(hi));
    for (int64_t j = b + threadIdx.x; j < e; j += blockDim.x) {
      uint2 pr = list[j];
      if (pr.x >= static_cast<uint32_t>(lo) && pr.x < static_cast<uint32_t>(hi)) {  // bounds: skip corrupt indices
        float v = __uint_as_float(pr.y) * scale;
        if (kBf16) {
          __nv_bfloat16* d = static_cast<__nv_bfloat16*>(dense);
          d[pr.x] = __float2bfloat16_rn(__bfloat162float(d[pr.x]) + v);
        } else {
          float* d = static_cast<float*>(dense);
          d[pr.x] += v;
        }
      }
    }
    __syncthreads();  // list r fully applied to this range before list r+1 touches it
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(512) topk_exchange_scatter_kernel(const __grid_constant__ CollParams p, int64_t n,
                                                                    int64_t k, float scale) {
  const RankCtx& c = p.ctx[blockIdx.y];
  const int cta = blockIdx.x, nctas = gridDim.x, tid = threadIdx.x;
  // enter: credit protocol of the arena (same as every collective kernel)
  {
    bool ok = true;
    if (tid < c.ws && tid != c.rank) {
      if (cta == 0) st_release_sys(entered_flag(c.arena[tid], lane_of(p.seq), c.rank), p.seq);
      ok = wait_epoch(entered_flag(c.arena[c.rank], lane_of(p.seq), tid), p.seq - 2, p.wait_ns, c.status, 100, tid);
    }
    if (tid == 0 && c.status != nullptr && *reinterpret_cast<volatile uint32_t*>(c.status) != 0u) ok = false;
    if (!__syncthreads_and(ok ? 1 : 0)) return;
  }
  const size_t slot_bytes = topk_pad(static_cast<size_t>(k) * 8);
  const uint4* src = static_cast<const uint4*>(c.in);
  const int64_t units = (k * 8 + 15) / 16;
  const bool tail_half = (k & 1) != 0;  // last unit holds one pair only
  const int64_t stride = static_cast<int64_t>(nctas) * blockDim.x;
  for (int64_t u = static_cast<int64_t>(cta) * blockDim.x + tid; u < units; u += stride) {
    uint4 v;
    if (tail_half && u == units - 1) {
      const uint2 last = static_cast<const uint2*>(c.in)[k - 1];
      v = make_uint4(last.x, last.y, 0xFFFFFFFFu, 0u);
    } else {
      v = __ldcg(src + u);
    }
    for (int d = 0; d < c.ws; ++d) {
      int q = c.rank + d;
      if (q >= c.ws) q -= c.ws;
      __stcg(reinterpret_cast<uint4*>(c.arena[q] + p.parity_offset + c.rank * slot_bytes) + u, v);
    }
  }
  __syncthreads();
  if (tid < c.ws) {
    fence_sys();
    st_release_sys(sig_flag(c.arena[tid], lane_of(p.seq), 0, cta, c.rank), sig_value(p.seq, kSigDone));
  }
  // Scatter needs every CTA's share of every list: wait for all (cta, rank) flags.
  {
    bool ok = true;
    for (int f = tid; f < nctas * c.ws; f += blockDim.x)
      ok = ok && wait_epoch(sig_flag(c.arena[c.rank], lane_of(p.seq), 0, f / c.ws, f % c.ws), sig_value(p.seq, kSigDone), p.wait_ns, c.status, 0, f % c.ws);
    if (!__syncthreads_and(ok ? 1 : 0)) return;
  }
  const uint2* lists[kMaxWorld];
  for (int r = 0; r < c.ws; ++r)
    lists[r] = reinterpret_cast<const uint2*>(c.arena[c.rank] + p.parity_offset + r * slot_bytes);
  scatter_lists<kBf16>(c.out, n, lists, c.ws, k, scale, cta, nctas);
}

template <bool kBf16>
__global__ void __launch_bounds__(512) topk_local_scatter_kernel(void* dense, int64_t n, const uint2* pairs, int64_t k,
                                                                 float scale) {
  const uint2* lists[1] = {pairs};
  scatter_lists<kBf16>(dense, n, lists, 1, k, scale, blockIdx.x, gridDim.x);
}

// Blocks of the collect and compaction passes.  Every block pays a fixed price (staging flush, block
// reduction, histogram merge, ticket), so a block gets at least 32 Ki elements: with 8 Ki per block the
// collect pass measured 54-67 us on 8 Mi elements, almost all of it that per-block overhead.
int select_blocks(int64_t n) {
  int64_t b = (n + 32767) / 32768;
  if (b < 1) b = 1;
  if (b > kTopkMaxBlocks) b = kTopkMaxBlocks;
  return static_cast<int>(b);
}

}  // namespace

size_t topk_scratch_bytes() { return sizeof(TopkScratch); }

cudaError_t launch_topk_select(const TopkArgs& a, cudaStream_t s) {
  if (a.n <= 0 || a.k <= 0 || a.k > a.n) return cudaErrorInvalidValue;
  TopkScratch* sc = static_cast<TopkScratch*>(a.scratch);
  const uint32_t k = static_cast<uint32_t>(a.k);
  note_launch(7);
  const int grid = static_cast<int>(std::min<int64_t>((a.n + 4095) / 4096, 148 * 4));
  const bool vec = ((reinterpret_cast<uintptr_t>(a.grad) | reinterpret_cast<uintptr_t>(a.residual)) & 15) == 0;
  const size_t smem = kTopkBins0 * sizeof(uint32_t);
  topk_clear_kernel<<<8, 256, 0, s>>>(sc);
  if (a.grad_is_bf16) {
    if (vec) topk_adjust_hist_kernel<true, true><<<grid, 512, smem, s>>>(a.grad, a.residual, a.n, sc, k);
    else topk_adjust_hist_kernel<true, false><<<grid, 512, smem, s>>>(a.grad, a.residual, a.n, sc, k);
  } else {
    if (vec) topk_adjust_hist_kernel<false, true><<<grid, 512, smem, s>>>(a.grad, a.residual, a.n, sc, k);
    else topk_adjust_hist_kernel<false, false><<<grid, 512, smem, s>>>(a.grad, a.residual, a.n, sc, k);
  }
  const int nb = select_blocks(a.n);
  // The output buffer doubles as the candidate list: it is only written for good by the last pass.
  topk_collect_refine_kernel<<<nb, 1024, 0, s>>>(a.residual, a.n, sc, static_cast<uint2*>(a.pairs), k, k);
  // heavily tied data only (these return at once otherwise; one CTA per SM keeps the idle launch cheap)
  const int fgrid = grid < 148 ? grid : 148;
  topk_hist_level_kernel<<<1, 512, 0, s>>>(a.residual, a.n, sc, 1, k);
  topk_hist_level_kernel<<<fgrid, 512, 0, s>>>(a.residual, a.n, sc, 2, k);
  topk_count_scan_kernel<<<nb, 1024, 0, s>>>(a.residual, a.n, sc);
  topk_compact_kernel<<<nb, 1024, 0, s>>>(a.residual, a.n, sc, static_cast<uint2*>(a.pairs), k);
  return cudaGetLastError();
}

cudaError_t launch_topk_exchange_scatter(const CollParams& p, const TopkArgs& a, LaunchCfg cfg, cudaStream_t s) {
  note_launch();
  int ctas = cfg.ctas > 0 ? cfg.ctas : 32;
  if (ctas > 64) ctas = 64;            // ctas * ws flags are polled by one CTA
  if (cfg.emulate_ranks > 0 && ctas > 16) ctas = 16;
  // more CTAs than index ranges of 8 elements would leave empty ranges: harmless but wasteful
  int64_t max_useful = (a.n + 7) / 8;
  if (ctas > max_useful) ctas = static_cast<int>(max_useful);
  if (ctas < 1) ctas = 1;
  void* args[] = {const_cast<CollParams*>(&p), const_cast<int64_t*>(&a.n), const_cast<int64_t*>(&a.k),
                  const_cast<float*>(&a.scale)};
  if (cfg.emulate_ranks > 0) {
    void* fn = a.grad_is_bf16 ? reinterpret_cast<void*>(topk_exchange_scatter_kernel<true>)
                              : reinterpret_cast<void*>(topk_exchange_scatter_kernel<false>);
    return cudaLaunchCooperativeKernel(fn, dim3(ctas, cfg.emulate_ranks), dim3(512), args, 0, s);
  }
  if (a.grad_is_bf16)
    topk_exchange_scatter_kernel<true><<<dim3(ctas, 1), 512, 0, s>>>(p, a.n, a.k, a.scale);
  else
    topk_exchange_scatter_kernel<false><<<dim3(ctas, 1), 512, 0, s>>>(p, a.n, a.k, a.scale);
  return cudaGetLastError();
}

cudaError_t launch_topk_local_scatter(const TopkArgs& a, cudaStream_t s) {
  note_launch();
  int ctas = static_cast<int>(std::min<int64_t>(148, (a.n + 4095) / 4096));
  if (ctas < 1) ctas = 1;
  if (a.grad_is_bf16)
    topk_local_scatter_kernel<true><<<ctas, 512, 0, s>>>(const_cast<void*>(a.grad), a.n,
                                                         static_cast<const uint2*>(a.pairs), a.k, a.scale);
  else
    topk_local_scatter_kernel<false><<<ctas, 512, 0, s>>>(const_cast<void*>(a.grad), a.n,
                                                          static_cast<const uint2*>(a.pairs), a.k, a.scale);
  return cudaGetLastError();
}

}  // namespace kern
}  // namespace mccl
