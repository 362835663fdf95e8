// Standalone elementwise kernels: dst = op(dst, src), buf *= s, dst = (dst+src)*s
// and dtype casts.  On the hot path these operations are fused into the
// collective kernels; the standalone forms serve the local (world size 1,
// unfused fallback) paths and the kernel unit tests.
//
// Each thread handles 16-byte vectors in a grid-stride loop; unaligned bases and
// tails fall back to guarded scalar accesses.  Integer scaling follows the
// averaging rules of vec.cuh (i32 rounds, i64/u8 truncate).
// Parity: reference csrc/metal/shaders.metal:196-731 (accumulate_chunk_*,
// elementwise_min/max/product_*, scale_inplace_*, accumulate_scale_*).
#include <type_traits>

#include "kernels/api.h"
#include "kernels/launch_count.h"
#include "kernels/vec.cuh"

namespace mccl {
namespace kern {

namespace {

template <typename T, int OP>
__global__ void __launch_bounds__(256) ew_reduce_kernel(T* __restrict__ dst, const T* __restrict__ src,
                                                        int64_t n) {
  using Acc = typename Traits<T>::Acc;
  constexpr int N = VecOf<T>::N;
  const bool al = is_aligned16(dst) && is_aligned16(src);
  const int64_t vecs = (n + N - 1) / N;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < vecs; v += stride) {
    typename VecOf<T>::U a, b;
    a.raw = ld_vec_guarded<T>(dst, v, n, al);
    b.raw = ld_vec_guarded<T>(src, v, n, al);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      Acc r = Reduce<T, OP>::apply(Traits<T>::load(a.e[j]), Traits<T>::load(b.e[j]));
      a.e[j] = Traits<T>::store(r);
    }
    st_vec_guarded<T>(dst, v, n, al, a.raw);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) ew_scale_kernel(T* __restrict__ buf, int64_t n, float s) {
  constexpr int N = VecOf<T>::N;
  const bool al = is_aligned16(buf);
  const int64_t vecs = (n + N - 1) / N;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < vecs; v += stride) {
    typename VecOf<T>::U a;
    a.raw = ld_vec_guarded<T>(buf, v, n, al);
#pragma unroll
    for (int j = 0; j < N; ++j) a.e[j] = Traits<T>::store(Traits<T>::scale(Traits<T>::load(a.e[j]), s));
    st_vec_guarded<T>(buf, v, n, al, a.raw);
  }
}

__global__ void __launch_bounds__(256) ew_scale_f64_kernel(double* __restrict__ buf, int64_t n, double s) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) buf[i] *= s;
}

template <typename T>
__global__ void __launch_bounds__(256) ew_accscale_kernel(T* __restrict__ dst, const T* __restrict__ src,
                                                          int64_t n, float s) {
  using Acc = typename Traits<T>::Acc;
  constexpr int N = VecOf<T>::N;
  const bool al = is_aligned16(dst) && is_aligned16(src);
  const int64_t vecs = (n + N - 1) / N;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < vecs; v += stride) {
    typename VecOf<T>::U a, b;
    a.raw = ld_vec_guarded<T>(dst, v, n, al);
    b.raw = ld_vec_guarded<T>(src, v, n, al);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      Acc r = Traits<T>::load(a.e[j]) + Traits<T>::load(b.e[j]);
      a.e[j] = Traits<T>::store(Traits<T>::scale(r, s));
    }
    st_vec_guarded<T>(dst, v, n, al, a.raw);
  }
}

template <typename D, typename S>
__global__ void __launch_bounds__(256) cast_kernel(D* __restrict__ dst, const S* __restrict__ src, int64_t n,
                                                   float s) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  // 4 elements per thread per step: 16-byte accesses on the fp32 side, 8 on the 16-bit side.
  const int64_t quads = n / 4;
  const bool al = is_aligned16(dst) && is_aligned16(src);
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (al) {
    for (int64_t q = i; q < quads; q += stride) {
      S in4[4];
      *reinterpret_cast<typename std::conditional<sizeof(S) == 4, uint4, uint2>::type*>(in4) =
          *reinterpret_cast<const typename std::conditional<sizeof(S) == 4, uint4, uint2>::type*>(src + q * 4);
      D out4[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) out4[j] = Traits<D>::store(Traits<S>::load(in4[j]) * s);
      *reinterpret_cast<typename std::conditional<sizeof(D) == 4, uint4, uint2>::type*>(dst + q * 4) =
          *reinterpret_cast<typename std::conditional<sizeof(D) == 4, uint4, uint2>::type*>(out4);
    }
    for (int64_t e = quads * 4 + i; e < n; e += stride) dst[e] = Traits<D>::store(Traits<S>::load(src[e]) * s);
  } else {
    for (int64_t e = i; e < n; e += stride) dst[e] = Traits<D>::store(Traits<S>::load(src[e]) * s);
  }
}

inline int grid_for(int64_t work_items, int threads) {
  int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = 148 * 8;  // a multiple of the SM count; grid-stride covers the rest
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

template <typename T>
cudaError_t reduce_dispatch_op(T* d, const T* s, int64_t n, RedOp op, cudaStream_t st) {
  constexpr int N = VecOf<T>::N;
  int g = grid_for((n + N - 1) / N, 256);
  switch (op) {
    case SUM:
    case AVG: ew_reduce_kernel<T, SUM><<<g, 256, 0, st>>>(d, s, n); break;
    case MIN: ew_reduce_kernel<T, MIN><<<g, 256, 0, st>>>(d, s, n); break;
    case MAX: ew_reduce_kernel<T, MAX><<<g, 256, 0, st>>>(d, s, n); break;
    case PRODUCT: ew_reduce_kernel<T, PRODUCT><<<g, 256, 0, st>>>(d, s, n); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_ew_reduce(void* dst, const void* src, int64_t n, DType t, RedOp op, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  note_launch();
  switch (t) {
    case F32: return reduce_dispatch_op((float*)dst, (const float*)src, n, op, s);
    case F64: return reduce_dispatch_op((double*)dst, (const double*)src, n, op, s);
    case F16: return reduce_dispatch_op((__half*)dst, (const __half*)src, n, op, s);
    case BF16: return reduce_dispatch_op((__nv_bfloat16*)dst, (const __nv_bfloat16*)src, n, op, s);
    case I32: return reduce_dispatch_op((int32_t*)dst, (const int32_t*)src, n, op, s);
    case I64: return reduce_dispatch_op((int64_t*)dst, (const int64_t*)src, n, op, s);
    case U8: return reduce_dispatch_op((uint8_t*)dst, (const uint8_t*)src, n, op, s);
    case BOOL: return reduce_dispatch_op((bool8*)dst, (const bool8*)src, n, op, s);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_ew_scale(void* buf, int64_t n, DType t, double scale, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  note_launch();
  float f = static_cast<float>(scale);
  switch (t) {
    case F32: ew_scale_kernel<float><<<grid_for((n + 3) / 4, 256), 256, 0, s>>>((float*)buf, n, f); break;
    case F64: ew_scale_f64_kernel<<<grid_for(n, 256), 256, 0, s>>>((double*)buf, n, scale); break;
    case F16: ew_scale_kernel<__half><<<grid_for((n + 7) / 8, 256), 256, 0, s>>>((__half*)buf, n, f); break;
    case BF16:
      ew_scale_kernel<__nv_bfloat16><<<grid_for((n + 7) / 8, 256), 256, 0, s>>>((__nv_bfloat16*)buf, n, f);
      break;
    case I32: ew_scale_kernel<int32_t><<<grid_for((n + 3) / 4, 256), 256, 0, s>>>((int32_t*)buf, n, f); break;
    case I64: ew_scale_kernel<int64_t><<<grid_for((n + 1) / 2, 256), 256, 0, s>>>((int64_t*)buf, n, f); break;
    case U8: ew_scale_kernel<uint8_t><<<grid_for((n + 15) / 16, 256), 256, 0, s>>>((uint8_t*)buf, n, f); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_ew_accumulate_scale(void* dst, const void* src, int64_t n, DType t, double scale,
                                       cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  note_launch();
  float f = static_cast<float>(scale);
  switch (t) {
    case F32:
      ew_accscale_kernel<float><<<grid_for((n + 3) / 4, 256), 256, 0, s>>>((float*)dst, (const float*)src, n, f);
      break;
    case F16:
      ew_accscale_kernel<__half><<<grid_for((n + 7) / 8, 256), 256, 0, s>>>((__half*)dst, (const __half*)src, n, f);
      break;
    case BF16:
      ew_accscale_kernel<__nv_bfloat16>
          <<<grid_for((n + 7) / 8, 256), 256, 0, s>>>((__nv_bfloat16*)dst, (const __nv_bfloat16*)src, n, f);
      break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_cast(void* dst, DType dt, const void* src, DType st, int64_t n, float scale,
                        cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  note_launch();
  int g = grid_for((n + 3) / 4, 256);
  if (dt == F16 && st == F32) cast_kernel<__half, float><<<g, 256, 0, s>>>((__half*)dst, (const float*)src, n, scale);
  else if (dt == BF16 && st == F32)
    cast_kernel<__nv_bfloat16, float><<<g, 256, 0, s>>>((__nv_bfloat16*)dst, (const float*)src, n, scale);
  else if (dt == F32 && st == F16)
    cast_kernel<float, __half><<<g, 256, 0, s>>>((float*)dst, (const __half*)src, n, scale);
  else if (dt == F32 && st == BF16)
    cast_kernel<float, __nv_bfloat16><<<g, 256, 0, s>>>((float*)dst, (const __nv_bfloat16*)src, n, scale);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace kern
}  // namespace mccl
