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
  uint32_t nblocks;
  uint32_t pad[3];
};
struct TopkScratch {
  uint32_t hist[3][kTopkBins];
  TopkState st;
  uint32_t blk_gt[kTopkMaxBlocks];
  uint32_t blk_eq[kTopkMaxBlocks];
  uint32_t off_gt[kTopkMaxBlocks];
  uint32_t off_eq[kTopkMaxBlocks];
};

__device__ __forceinline__ uint32_t mag_key(float a) { return __float_as_uint(a) & 0x7FFFFFFFu; }

// level 0: bits 30..20 (11), level 1: bits 19..9 (11), level 2: bits 8..0 (9)
__device__ __forceinline__ uint32_t digit_of(uint32_t key, int level) {
  return level == 0 ? (key >> 20) : level == 1 ? ((key >> 9) & 0x7FFu) : (key & 0x1FFu);
}
__device__ __forceinline__ bool prefix_matches(uint32_t key, int level, uint32_t prefix) {
  return level == 0 ? true : level == 1 ? ((key >> 20) == prefix) : ((key >> 9) == prefix);
}

__global__ void topk_clear_kernel(TopkScratch* sc) {
  uint32_t* h = &sc->hist[0][0];
  for (int i = threadIdx.x + blockIdx.x * blockDim.x; i < 3 * kTopkBins; i += blockDim.x * gridDim.x) h[i] = 0;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    sc->st.prefix = 0;
    sc->st.need = 0;
    sc->st.threshold = 0;
    sc->st.need_eq = 0;
  }
}

// a = g + e, e = a, histogram of the top digit.
template <bool kBf16>
__global__ void __launch_bounds__(512) topk_adjust_hist_kernel(const void* __restrict__ grad,
                                                               float* __restrict__ res, int64_t n,
                                                               TopkScratch* sc) {
  __shared__ uint32_t sh[kTopkBins];
  for (int i = threadIdx.x; i < kTopkBins; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float g = kBf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(grad)[i])
                    : static_cast<const float*>(grad)[i];
    float a = g + res[i];
    res[i] = a;
    atomicAdd(&sh[digit_of(mag_key(a), 0)], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kTopkBins; i += blockDim.x)
    if (sh[i]) atomicAdd(&sc->hist[0][i], sh[i]);
}

__global__ void __launch_bounds__(512) topk_hist_level_kernel(const float* __restrict__ res, int64_t n,
                                                              TopkScratch* sc, int level) {
  __shared__ uint32_t sh[kTopkBins];
  for (int i = threadIdx.x; i < kTopkBins; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const uint32_t prefix = sc->st.prefix;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    uint32_t key = mag_key(res[i]);
    if (prefix_matches(key, level, prefix)) atomicAdd(&sh[digit_of(key, level)], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kTopkBins; i += blockDim.x)
    if (sh[i]) atomicAdd(&sc->hist[level][i], sh[i]);
}

// Exclusive scan of one value per thread over a 1024-thread block.
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

// Walks the histogram of `level` from the top bin down (as a parallel suffix
// scan: thread t owns bins 2047-2t and 2046-2t) and fixes the next digit: the
// first bin, from the top, at which the running count reaches `need`.
__global__ void __launch_bounds__(1024) topk_pick_bin_kernel(TopkScratch* sc, int level, uint32_t k) {
  __shared__ uint32_t wsum[33];
  __shared__ uint32_t s_digit, s_cum;
  const uint32_t need = level == 0 ? k : sc->st.need;
  const uint32_t old_prefix = sc->st.prefix;
  if (threadIdx.x == 0) {
    s_digit = 0;
    s_cum = 0xFFFFFFFFu;
  }
  const int b1 = kTopkBins - 1 - 2 * static_cast<int>(threadIdx.x), b2 = b1 - 1;
  const uint32_t c1 = sc->hist[level][b1], c2 = sc->hist[level][b2];
  uint32_t total;
  const uint32_t above = block_excl_scan(c1 + c2, wsum, total);  // count in bins above b1
  if (above < need && above + c1 >= need) {
    s_digit = b1;
    s_cum = above;
  } else if (above + c1 < need && above + c1 + c2 >= need) {
    s_digit = b2;
    s_cum = above + c1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t digit = s_digit, cum = s_cum;
    if (cum == 0xFFFFFFFFu) {  // fewer than `need` elements in total: take everything
      digit = 0;
      cum = total - sc->hist[level][0];
    }
    const uint32_t prefix = level == 0 ? digit : level == 1 ? ((old_prefix << 11) | digit) : ((old_prefix << 9) | digit);
    sc->st.prefix = prefix;
    sc->st.need = need - cum;  // elements still to take from inside the chosen bin
    if (level == 2) {
      sc->st.threshold = prefix;
      sc->st.need_eq = need - cum;
    }
  }
}

// Blocks own contiguous ranges so that compaction preserves index order.
__device__ __forceinline__ void block_range(int64_t n, int nblocks, int b, int64_t& lo, int64_t& hi) {
  int64_t per = (n + nblocks - 1) / nblocks;
  per = (per + 1023) / 1024 * 1024;
  lo = static_cast<int64_t>(b) * per;
  hi = lo + per;
  if (lo > n) lo = n;
  if (hi > n) hi = n;
}

__global__ void __launch_bounds__(1024) topk_count_blocks_kernel(const float* __restrict__ res, int64_t n,
                                                                 TopkScratch* sc) {
  __shared__ uint32_t s_gt, s_eq;
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
}

__global__ void topk_scan_blocks_kernel(TopkScratch* sc, int nblocks) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  uint32_t g = 0, e = 0;
  for (int b = 0; b < nblocks; ++b) {
    sc->off_gt[b] = g;
    sc->off_eq[b] = e;
    g += sc->blk_gt[b];
    e += sc->blk_eq[b];
  }
}

__global__ void __launch_bounds__(1024) topk_compact_kernel(float* __restrict__ res, int64_t n, TopkScratch* sc,
                                                            uint2* __restrict__ pairs, uint32_t k) {
  __shared__ uint32_t ws_a[33], ws_b[33];
  const uint32_t T = sc->st.threshold;
  const uint32_t need_eq = sc->st.need_eq;
  int64_t lo, hi;
  block_range(n, gridDim.x, blockIdx.x, lo, hi);
  uint32_t eq_base = sc->off_eq[blockIdx.x];
  // selected elements that precede this block
  uint32_t out_base = sc->off_gt[blockIdx.x] + (eq_base < need_eq ? eq_base : need_eq);
  for (int64_t t0 = lo; t0 < hi; t0 += blockDim.x) {
    const int64_t i = t0 + threadIdx.x;
    float a = 0.f;
    uint32_t key = 0;
    bool in = i < hi;
    if (in) {
      a = res[i];
      key = mag_key(a);
    }
    const uint32_t is_eq = in && key == T;
    uint32_t eq_total;
    const uint32_t eq_rank = eq_base + block_excl_scan(is_eq, ws_a, eq_total);
    const uint32_t sel = in && (key > T || (is_eq && eq_rank < need_eq));
    uint32_t sel_total;
    const uint32_t pos = out_base + block_excl_scan(sel, ws_b, sel_total);
    if (sel && pos < k) {
      pairs[pos] = make_uint2(static_cast<uint32_t>(i), __float_as_uint(a));
      res[i] = 0.f;  // sent: nothing left to feed back for this entry
    }
    eq_base += eq_total;
    out_base += sel_total;
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

int select_blocks(int64_t n) {
  int64_t b = (n + 8191) / 8192;
  if (b < 1) b = 1;
  if (b > kTopkMaxBlocks) b = kTopkMaxBlocks;
  return static_cast<int>(b);
}

}  // namespace

size_t topk_scratch_bytes() { return sizeof(TopkScratch); }

cudaError_t launch_topk_select(const TopkArgs& a, cudaStream_t s) {
  if (a.n <= 0 || a.k <= 0 || a.k > a.n) return cudaErrorInvalidValue;
  TopkScratch* sc = static_cast<TopkScratch*>(a.scratch);
  note_launch(10);
  const int grid = static_cast<int>(std::min<int64_t>((a.n + 4095) / 4096, 148 * 4));
  topk_clear_kernel<<<8, 256, 0, s>>>(sc);
  if (a.grad_is_bf16)
    topk_adjust_hist_kernel<true><<<grid, 512, 0, s>>>(a.grad, a.residual, a.n, sc);
  else
    topk_adjust_hist_kernel<false><<<grid, 512, 0, s>>>(a.grad, a.residual, a.n, sc);
  topk_pick_bin_kernel<<<1, 1024, 0, s>>>(sc, 0, static_cast<uint32_t>(a.k));
  topk_hist_level_kernel<<<grid, 512, 0, s>>>(a.residual, a.n, sc, 1);
  topk_pick_bin_kernel<<<1, 1024, 0, s>>>(sc, 1, static_cast<uint32_t>(a.k));
  topk_hist_level_kernel<<<grid, 512, 0, s>>>(a.residual, a.n, sc, 2);
  topk_pick_bin_kernel<<<1, 1024, 0, s>>>(sc, 2, static_cast<uint32_t>(a.k));
  const int nb = select_blocks(a.n);
  topk_count_blocks_kernel<<<nb, 1024, 0, s>>>(a.residual, a.n, sc);
  topk_scan_blocks_kernel<<<1, 32, 0, s>>>(sc, nb);
  topk_compact_kernel<<<nb, 1024, 0, s>>>(a.residual, a.n, sc, static_cast<uint2*>(a.pairs),
                                          static_cast<uint32_t>(a.k));
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
