// Allreduce (SUM / AVG) with the reduction done inside the NVSwitch (NVLS), sm_100a.
//
// Every rank owns a buffer of the group's NVLS region: the same offset of all ranks' buffers is
// bound to one NVLink multicast object, so a `multimem.ld_reduce` on the multicast address returns
// the sum over all ranks' copies (added up in the switch, 16-bit floats accumulated in fp32) and a
// `multimem.st` writes all copies at once.  Per GPU the links carry about (1 + 1/ws) * N bytes in
// each direction instead of the 2 * (ws-1)/ws * N of the point-to-point two-shot, and no SM spends
// time adding.
//
//   stage 0  copy my input (rounded to the wire type) into my own buffer      [local]
//   stage 1  owner of chunk q = rank: ld_reduce the chunk through the switch, apply the scale,
//            multimem.st the result over every rank's copy, write my own output directly
//   stage 2  copy the other chunks from my buffer into my output               [local]
//
// The three stages are software-pipelined over tiles (TilePlan): in iteration `it` a CTA stages
// tile it, reduces tile it-1 and copies out tile it-2, so the local HBM passes overlap the link
// phase.  Each element is reduced by exactly one rank, hence all ranks end with identical bits.
// Flags, epochs, bounded waits and the status block are those of the peer-memory kernels; the
// signal pads stay in the unicast arena.
//
// These are NVLS `multimem` instructions on a multicast address.  No TMA and no cluster multicast
// is used here or anywhere else in the library.
//
// Fills the role of the reference's bandwidth-optimal large-message path, the chunked ring
// (reference csrc/backend/ProcessGroupMCCL.cpp:1712-1959).
#include <cstdlib>

#include "kernels/coll_common.cuh"

namespace mccl {
namespace kern {
namespace {

template <typename T, typename W>
__global__ void __launch_bounds__(512) nvls_allreduce_kernel(const __grid_constant__ CollParams p) {
  using U = Unit<T, W>;
  using Acc = typename U::Acc;
  CtaCtx k = make_ctx(p);
  const RankCtx& c = *k.c;
  stamp(k, 0);
  if (!enter_collective(k)) return;
  stamp(k, 1);

  const int64_t n = p.count;
  const int64_t units = (n + U::N - 1) / U::N;
  const int64_t chunk_units = (units + c.ws - 1) / c.ws;
  if (!range_ok(k, 0, static_cast<size_t>(chunk_units) * c.ws * 16, p.nvls_capacity, 30)) return;
  char* stage = c.nvls_uc + p.nvls_offset;
  char* mc = c.nvls_mc + p.nvls_offset;
  const T* in = static_cast<const T*>(c.in);
  T* out = static_cast<T*>(c.out);
  const bool in_al = is_aligned16(in), out_al = is_aligned16(out);
  const bool scaled = p.op == AVG || p.scale != 1.0f;

  const TilePlan tp = TilePlan::make(chunk_units, k.nctas, k.nthreads, p.tile_bytes);
  const int64_t my_tiles = tp.count_for(k.cta, k.nctas);
  const int64_t own_base = static_cast<int64_t>(c.rank) * chunk_units;
  const uint32_t peers = ((1u << c.ws) - 1u) & ~(1u << c.rank);

  for (int64_t it = 0; it < my_tiles + 2; ++it) {
    // ---- stage 0: my contribution to tile `it` of every chunk -> my buffer -------------------
    if (it < my_tiles) {
      const int64_t u0 = tp.begin(k.cta, k.nctas, it), u1 = tp.end(k.cta, k.nctas, it);
      for (int d = 0; d < c.ws; ++d) {
        int q = c.rank + d;
        if (q >= c.ws) q -= c.ws;
        const int64_t base = static_cast<int64_t>(q) * chunk_units;
        for (int64_t ub = u0; ub < u1; ub += static_cast<int64_t>(k.nthreads) * kUnroll) {
          uint4 v[kUnroll];
#pragma unroll
          for (int i = 0; i < kUnroll; ++i) {
            const int64_t u = base + ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
            if (u < base + u1 && u < units) {
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
            const int64_t u = base + ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
            if (u < base + u1 && u < units) stg16(stage + u * 16, v[i]);
          }
        }
      }
      if (it == my_tiles - 1) stamp(k, 2);
      signal_all(k, 0, static_cast<uint32_t>(it + 1));
    }
    // ---- stage 1: reduce tile it-1 of my chunk in the switch, broadcast the result -----------
    if (it >= 1 && it - 1 < my_tiles) {
      if (!wait_all(k, 0, -1, static_cast<uint32_t>(it))) return;
      if (it == my_tiles) stamp(k, 3);
      const int64_t u0 = tp.begin(k.cta, k.nctas, it - 1), u1 = tp.end(k.cta, k.nctas, it - 1);
      for (int64_t ub = u0; ub < u1; ub += static_cast<int64_t>(k.nthreads) * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int i = 0; i < kUnroll; ++i) {
          const int64_t u = own_base + ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
          if (u < own_base + u1 && u < units) v[i] = MultimemSum<W>::ld(mc + u * 16);
        }
#pragma unroll
        for (int i = 0; i < kUnroll; ++i) {
          const int64_t u = own_base + ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
          if (u < own_base + u1 && u < units) {
            Acc a[U::N];
            if (scaled) {
              U::unpack_W(v[i], a);
#pragma unroll
              for (int j = 0; j < U::N; ++j) a[j] = Traits<T>::scale(a[j], p.scale);
              v[i] = U::pack_W(a);
            }
            multimem_st16(mc + u * 16, v[i]);
            if (U::kSame && out_al && (u + 1) * U::N <= n) {
              stg16(out + u * U::N, v[i]);
            } else {
              U::unpack_W(v[i], a);  // exactly what the peers receive
              U::store_T(out, u * U::N, n, out_al, a);
            }
          }
        }
      }
      if (it == my_tiles) stamp(k, 4);
      signal_all(k, 1, static_cast<uint32_t>(it));
    }
    // ---- stage 2: tile it-2 of the other chunks: my buffer -> my output ----------------------
    if (it >= 2 && it - 2 < my_tiles) {
      if (!wait_mask(k, 1, peers, static_cast<uint32_t>(it - 1))) return;
      if (it == my_tiles + 1) stamp(k, 5);
      const int64_t u0 = tp.begin(k.cta, k.nctas, it - 2), u1 = tp.end(k.cta, k.nctas, it - 2);
      constexpr int kOut = 8;
      for (int d = 1; d < c.ws; ++d) {
        int q = c.rank + d;
        if (q >= c.ws) q -= c.ws;
        const int64_t base = static_cast<int64_t>(q) * chunk_units;
        for (int64_t ub = u0; ub < u1; ub += static_cast<int64_t>(k.nthreads) * kOut) {
          uint4 v[kOut];
#pragma unroll
          for (int i = 0; i < kOut; ++i) {
            const int64_t u = base + ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
            if (u < base + u1 && u < units) v[i] = ldg16(stage + u * 16);
          }
#pragma unroll
          for (int i = 0; i < kOut; ++i) {
            const int64_t u = base + ub + k.tid + static_cast<int64_t>(i) * k.nthreads;
            if (u < base + u1 && u < units) {
              if (U::kSame && out_al && (u + 1) * U::N <= n) {
                stg16(out + u * U::N, v[i]);
              } else {
                Acc a[U::N];
                U::unpack_W(v[i], a);
                U::store_T(out, u * U::N, n, out_al, a);
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
// Split form for large messages.  The two local passes need no peer and no co-residency, so they
// run as ordinary full-grid kernels at HBM speed instead of on the 64 CTAs a flag-waiting kernel
// may use, and only the link phase stays in the kernel that talks to the peers:
//   nvls_stage_in_kernel      input (rounded to the wire type) -> my NVLS buffer       [full grid]
//   nvls_reduce_bcast_kernel  wait for everybody's staging; owner of a chunk reduces it in the
//                             switch, scales, multimem.st's it to all ranks and writes its own
//                             output; wait for everybody's stores                     [<= 64 CTAs]
//   nvls_stage_out_kernel     the other chunks: my NVLS buffer -> output               [full grid]
// All three are stream-ordered on the collective's lane; with two lanes, the staging passes of
// one segment overlap the link phase of the other.
// ---------------------------------------------------------------------------
template <typename T, typename W>
__global__ void __launch_bounds__(512) nvls_stage_in_kernel(const __grid_constant__ CollParams p) {
  using U = Unit<T, W>;
  using Acc = typename U::Acc;
  const RankCtx& c = p.ctx[0];
  const int64_t n = p.count;
  const int64_t units = (n + U::N - 1) / U::N;
  char* stage = c.nvls_uc + p.nvls_offset;
  const T* in = static_cast<const T*>(c.in);
  const bool in_al = is_aligned16(in);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t ub = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; ub < units; ub += stride * kUnroll) {
    uint4 v[kUnroll];
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      const int64_t u = ub + i * stride;
      if (u < units) {
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
      const int64_t u = ub + i * stride;
      if (u < units) stg16(stage + u * 16, v[i]);
    }
  }
}

template <typename T, typename W>
__global__ void __launch_bounds__(512) nvls_stage_out_kernel(const __grid_constant__ CollParams p) {
  using U = Unit<T, W>;
  using Acc = typename U::Acc;
  const RankCtx& c = p.ctx[0];
  const int64_t n = p.count;
  const int64_t units = (n + U::N - 1) / U::N;
  const int64_t chunk_units = (units + c.ws - 1) / c.ws;
  const int64_t own0 = static_cast<int64_t>(c.rank) * chunk_units, own1 = own0 + chunk_units;
  const char* stage = c.nvls_uc + p.nvls_offset;
  T* out = static_cast<T*>(c.out);
  const bool out_al = is_aligned16(out);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t ub = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; ub < units; ub += stride * kUnroll) {
    uint4 v[kUnroll];
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      const int64_t u = ub + i * stride;
      if (u < units && (u < own0 || u >= own1)) v[i] = ldg16(stage + u * 16);
    }
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
      const int64_t u = ub + i * stride;
      if (u < units && (u < own0 || u >= own1)) {  // the owner wrote its own chunk itself
        if (U::kSame && out_al && (u + 1) * U::N <= n) {
          stg16(out + u * U::N, v[i]);
        } else {
          Acc a[U::N];
          U::unpack_W(v[i], a);
          U::store_T(out, u * U::N, n, out_al, a);
        }
      }
    }
  }
}

template <typename T, typename W>
__global__ void __launch_bounds__(512) nvls_reduce_bcast_kernel(const __grid_constant__ CollParams p) {
  using U = Unit<T, W>;
  using Acc = typename U::Acc;
  CtaCtx k = make_ctx(p);
  const RankCtx& c = *k.c;
  stamp(k, 0);
  if (!enter_collective(k)) return;
  stamp(k, 1);
  const int64_t n = p.count;
  const int64_t units = (n + U::N - 1) / U::N;
  const int64_t chunk_units = (units + c.ws - 1) / c.ws;
  if (!range_ok(k, 0, static_cast<size_t>(chunk_units) * c.ws * 16, p.nvls_capacity, 31)) return;
  char* mc = c.nvls_mc + p.nvls_offset;
  T* out = static_cast<T*>(c.out);
  const bool out_al = is_aligned16(out);
  const bool scaled = p.op == AVG || p.scale != 1.0f;
  // my staging pass is an earlier kernel of this stream, hence complete; tell the peers and wait
  // until every peer says the same
  stamp(k, 2);
  signal_all(k, 0);
  if (!wait_all(k, 0)) return;
  stamp(k, 3);
  const int64_t own0 = static_cast<int64_t>(c.rank) * chunk_units;
  const int64_t own1 = own0 + chunk_units < units ? own0 + chunk_units : units;
  constexpr int kIn = 8;  // round trips through the switch: keep many in flight
  const int64_t stride = static_cast<int64_t>(k.nctas) * k.nthreads;
  for (int64_t ub = own0 + static_cast<int64_t>(k.cta) * k.nthreads + k.tid; ub < own1; ub += stride * kIn) {
    uint4 v[kIn];
#pragma unroll
    for (int i = 0; i < kIn; ++i) {
      const int64_t u = ub + i * stride;
      if (u < own1) v[i] = MultimemSum<W>::ld(mc + u * 16);
    }
#pragma unroll
    for (int i = 0; i < kIn; ++i) {
      const int64_t u = ub + i * stride;
      if (u < own1) {
        Acc a[U::N];
        if (scaled) {
          U::unpack_W(v[i], a);
#pragma unroll
          for (int j = 0; j < U::N; ++j) a[j] = Traits<T>::scale(a[j], p.scale);
          v[i] = U::pack_W(a);
        }
        multimem_st16(mc + u * 16, v[i]);
        if (U::kSame && out_al && (u + 1) * U::N <= n) {
          stg16(out + u * U::N, v[i]);
        } else {
          U::unpack_W(v[i], a);
          U::store_T(out, u * U::N, n, out_al, a);
        }
      }
    }
  }
  stamp(k, 4);
  signal_all(k, 1);
  if (!wait_all(k, 1)) return;  // all peers' results have landed in my buffer
  stamp(k, 5);
  stamp(k, 6);
}

// ---------------------------------------------------------------------------
// In-place form for tensors that already live in multicast-bound memory (runtime/nvls_pool.h):
// no staging at all.  Barrier (every rank's tensor is ready), the owner of a chunk reduces it in
// the switch, scales it and multimem.st's the result over every rank's copy (its own included),
// barrier (everybody's chunks have landed).  Each GPU's SMs touch only N/ws bytes, the links carry
// (1 + 1/ws) N per direction, and the reduction costs no SM time: a gradient bucket is reduced by
// a grid of a few CTAs while backward keeps the rest of the GPU.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(512) nvls_inplace_kernel(const __grid_constant__ CollParams p) {
  using U = Unit<T, T>;
  using Acc = typename U::Acc;
  CtaCtx k = make_ctx(p);
  const RankCtx& c = *k.c;
  stamp(k, 0);
  if (!enter_collective(k)) return;
  stamp(k, 1);
  const int64_t units = p.count / U::N;  // the launcher guarantees whole 16-byte units
  const int64_t chunk_units = (units + c.ws - 1) / c.ws;
  if (!range_ok(k, p.nvls_offset, static_cast<size_t>(units) * 16, p.nvls_capacity, 32)) return;
  char* mc = c.nvls_mc + p.nvls_offset;
  const bool scaled = p.op == AVG || p.scale != 1.0f;
  stamp(k, 2);
  signal_all(k, 0);
  if (!wait_all(k, 0)) return;
  stamp(k, 3);
  const int64_t own0 = static_cast<int64_t>(c.rank) * chunk_units;
  const int64_t own1 = own0 + chunk_units < units ? own0 + chunk_units : units;
  constexpr int kIn = 8;
  const int64_t stride = static_cast<int64_t>(k.nctas) * k.nthreads;
  for (int64_t ub = own0 + static_cast<int64_t>(k.cta) * k.nthreads + k.tid; ub < own1; ub += stride * kIn) {
    uint4 v[kIn];
#pragma unroll
    for (int i = 0; i < kIn; ++i) {
      const int64_t u = ub + i * stride;
      if (u < own1) v[i] = MultimemSum<T>::ld(mc + u * 16);
    }
#pragma unroll
    for (int i = 0; i < kIn; ++i) {
      const int64_t u = ub + i * stride;
      if (u < own1) {
        if (scaled) {
          Acc a[U::N];
          U::unpack_W(v[i], a);
#pragma unroll
          for (int j = 0; j < U::N; ++j) a[j] = Traits<T>::scale(a[j], p.scale);
          v[i] = U::pack_W(a);
        }
        multimem_st16(mc + u * 16, v[i]);
      }
    }
  }
  stamp(k, 4);
  signal_all(k, 1);
  if (!wait_all(k, 1)) return;
  stamp(k, 5);
  stamp(k, 6);
}

// Threads per CTA of the kernels that only do the link phase (in-place and split forms).  They hold
// no shared memory and at most 128 registers per thread, so a 256-thread CTA takes half an SM's
// register file and can share the SM with other kernels' CTAs (a staging pass of the other lane, a
// backward GEMM) instead of waiting for a whole SM to drain.  MCCL_NVLS_THREADS overrides (128..512).
int link_threads() {
  static const int v = [] {
    const char* e = std::getenv("MCCL_NVLS_THREADS");
    int t = e ? std::atoi(e) : 256;
    if (t < 128) t = 128;
    if (t > 512) t = 512;
    return t / 32 * 32;
  }();
  return v;
}

template <typename T, typename W>
cudaError_t go_split(const CollParams& p, int ctas, const LaunchCfg& cfg, cudaStream_t s) {
  const int64_t units = (p.count + Unit<T, W>::N - 1) / Unit<T, W>::N;
  int64_t want = (units + 512 * kUnroll - 1) / (512 * kUnroll);
  const int copy_ctas = static_cast<int>(want < 1 ? 1 : want > 592 ? 592 : want);  // 4 CTAs per SM
  note_launch(2);
  nvls_stage_in_kernel<T, W><<<copy_ctas, 512, 0, s>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  e = do_launch(nvls_reduce_bcast_kernel<T, W>, p, ctas, link_threads(), 0, s);
  if (e != cudaSuccess) return e;
  nvls_stage_out_kernel<T, W><<<copy_ctas, 512, 0, s>>>(p);
  return cudaGetLastError();
}

template <typename T, typename W>
cudaError_t go(const CollParams& p, int ctas, const LaunchCfg& cfg, cudaStream_t s) {
  return do_launch(nvls_allreduce_kernel<T, W>, p, ctas, cfg.threads, 0, s);
}

}  // namespace

size_t nvls_allreduce_stage_bytes(size_t nbytes_wire, int ws) {
  const size_t units = (nbytes_wire + 15) / 16;
  const size_t chunk_units = (units + ws - 1) / ws;
  return chunk_units * ws * 16;
}

bool nvls_allreduce_supported(DType dtype, DType wire, int op) {
  if (op != SUM && op != AVG) return false;
  if (dtype == F32) return wire == F32 || wire == BF16 || wire == F16;
  if (dtype == F16 || dtype == BF16) return wire == dtype;
  return false;
}

cudaError_t launch_allreduce_nvls_inplace(const CollParams& p, DType dtype, LaunchCfg cfg, cudaStream_t s) {
  if (!nvls_allreduce_supported(dtype, dtype, p.op) || cfg.emulate_ranks > 0 || p.ctx[0].nvls_mc == nullptr)
    return cudaErrorNotSupported;
  if ((p.count * dtype_size(dtype)) % 16 != 0 || (p.nvls_offset % 16) != 0) return cudaErrorInvalidValue;
  // each rank only moves its own chunk: size the grid for count / ws
  const size_t own_bytes = p.count * dtype_size(dtype) / p.ctx[0].ws;
  const int ctas = clamp_ctas(cfg.ctas > 0 ? cfg.ctas : pick_ctas(own_bytes, p.ctx[0].ws, 0), cfg);
  if (dtype == F32) return do_launch(nvls_inplace_kernel<float>, p, ctas, link_threads(), 0, s);
  if (dtype == F16) return do_launch(nvls_inplace_kernel<__half>, p, ctas, link_threads(), 0, s);
  return do_launch(nvls_inplace_kernel<__nv_bfloat16>, p, ctas, link_threads(), 0, s);
}

cudaError_t launch_allreduce_nvls(const CollParams& p, DType dtype, DType wire, LaunchCfg cfg, cudaStream_t s,
                                  bool split) {
  if (!nvls_allreduce_supported(dtype, wire, p.op) || cfg.emulate_ranks > 0 || p.ctx[0].nvls_mc == nullptr)
    return cudaErrorNotSupported;
  const int ctas = clamp_ctas(cfg.ctas > 0 ? cfg.ctas : pick_ctas(p.count * dtype_size(wire), p.ctx[0].ws, 0), cfg);
  if (split) {
    if (dtype == F32 && wire == F32) return go_split<float, float>(p, ctas, cfg, s);
    if (dtype == F32 && wire == BF16) return go_split<float, __nv_bfloat16>(p, ctas, cfg, s);
    if (dtype == F32 && wire == F16) return go_split<float, __half>(p, ctas, cfg, s);
    if (dtype == F16) return go_split<__half, __half>(p, ctas, cfg, s);
    return go_split<__nv_bfloat16, __nv_bfloat16>(p, ctas, cfg, s);
  }
  if (dtype == F32 && wire == F32) return go<float, float>(p, ctas, cfg, s);
  if (dtype == F32 && wire == BF16) return go<float, __nv_bfloat16>(p, ctas, cfg, s);
  if (dtype == F32 && wire == F16) return go<float, __half>(p, ctas, cfg, s);
  if (dtype == F16) return go<__half, __half>(p, ctas, cfg, s);
  return go<__nv_bfloat16, __nv_bfloat16>(p, ctas, cfg, s);
}

}  // namespace kern
}  // namespace mccl
