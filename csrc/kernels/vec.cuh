// 16-byte vector access and per-dtype arithmetic traits shared by every kernel.
//
// A "vector" is one uint4 (16 bytes) holding 16/sizeof(T) elements.  All
// reductions of 16-bit floats are carried in fp32 and narrowed once; bool is
// stored as one byte and reduced logically (SUM/MAX = OR, PRODUCT/MIN = AND).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels/api.h"

namespace mccl {
namespace kern {

struct bool8 { uint8_t v; };  // tag type: 1-byte logical element

template <typename T> struct Traits;
template <> struct Traits<float> {
  using Acc = float;
  static __device__ __forceinline__ Acc load(float x) { return x; }
  static __device__ __forceinline__ float store(Acc a) { return a; }
  static __device__ __forceinline__ Acc scale(Acc a, float s) { return a * s; }
};
template <> struct Traits<double> {
  using Acc = double;
  static __device__ __forceinline__ Acc load(double x) { return x; }
  static __device__ __forceinline__ double store(Acc a) { return a; }
  static __device__ __forceinline__ Acc scale(Acc a, float s) { return a * static_cast<double>(s); }
};
template <> struct Traits<__half> {
  using Acc = float;
  static __device__ __forceinline__ Acc load(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half store(Acc a) { return __float2half_rn(a); }
  static __device__ __forceinline__ Acc scale(Acc a, float s) { return a * s; }
};
template <> struct Traits<__nv_bfloat16> {
  using Acc = float;
  static __device__ __forceinline__ Acc load(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 store(Acc a) { return __float2bfloat16_rn(a); }
  static __device__ __forceinline__ Acc scale(Acc a, float s) { return a * s; }
};
template <> struct Traits<int32_t> {
  using Acc = int32_t;
  static __device__ __forceinline__ Acc load(int32_t x) { return x; }
  static __device__ __forceinline__ int32_t store(Acc a) { return a; }
  // integer average: round to nearest, halves away from zero
  static __device__ __forceinline__ Acc scale(Acc a, float s) {
    return static_cast<int32_t>(roundf(static_cast<float>(a) * s));
  }
};
template <> struct Traits<int64_t> {
  using Acc = int64_t;
  static __device__ __forceinline__ Acc load(int64_t x) { return x; }
  static __device__ __forceinline__ int64_t store(Acc a) { return a; }
  // 64-bit integer average truncates towards zero
  static __device__ __forceinline__ Acc scale(Acc a, float s) {
    return static_cast<int64_t>(static_cast<double>(a) * static_cast<double>(s));
  }
};
template <> struct Traits<uint8_t> {
  using Acc = uint32_t;
  static __device__ __forceinline__ Acc load(uint8_t x) { return x; }
  static __device__ __forceinline__ uint8_t store(Acc a) { return static_cast<uint8_t>(a); }
  static __device__ __forceinline__ Acc scale(Acc a, float s) {
    return static_cast<uint32_t>(static_cast<float>(a & 0xFFu) * s);
  }
};
template <> struct Traits<bool8> {
  using Acc = uint32_t;
  static __device__ __forceinline__ Acc load(bool8 x) { return x.v ? 1u : 0u; }
  static __device__ __forceinline__ bool8 store(Acc a) { return bool8{static_cast<uint8_t>(a ? 1 : 0)}; }
  static __device__ __forceinline__ Acc scale(Acc a, float) { return a; }
};

// OP value meaning "MIN, MAX or PRODUCT chosen at run time" (see apply_rt).
constexpr int kRuntimeOp = 100;

// MIN / MAX propagate NaNs like torch and NCCL do (a comparison-only select would drop a NaN
// depending on which side it is on).  For integer accumulators the tests fold away.
template <typename A> __device__ __forceinline__ A nan_min(A a, A b) { return a != a ? a : (b != b ? b : (b < a ? b : a)); }
template <typename A> __device__ __forceinline__ A nan_max(A a, A b) { return a != a ? a : (b != b ? b : (b > a ? b : a)); }

template <typename T, int OP> struct Reduce {
  using Acc = typename Traits<T>::Acc;
  // Run-time choice among MIN / MAX / PRODUCT (the rarely used operators share
  // one kernel instantiation; SUM and AVG have their own fast one).
  static __device__ __forceinline__ Acc apply_rt(int op, Acc a, Acc b) {
    const Acc mn = nan_min(a, b), mx = nan_max(a, b), pr = a * b;
    return op == MIN ? mn : op == MAX ? mx : pr;
  }
  static __device__ __forceinline__ Acc apply(Acc a, Acc b) {
    if (OP == SUM || OP == AVG) return a + b;
    if (OP == PRODUCT) return a * b;
    if (OP == MIN) return nan_min(a, b);
    return nan_max(a, b);
  }
};
template <int OP> struct Reduce<bool8, OP> {
  using Acc = uint32_t;
  static __device__ __forceinline__ Acc apply_rt(int op, Acc a, Acc b) { return op == MAX ? (a | b) : (a & b); }
  static __device__ __forceinline__ Acc apply(Acc a, Acc b) {
    if (OP == SUM || OP == AVG || OP == MAX) return a | b;
    return a & b;
  }
};
// u8 arithmetic wraps modulo 256 like the tensor dtype does.
template <int OP> struct Reduce<uint8_t, OP> {
  using Acc = uint32_t;
  static __device__ __forceinline__ Acc apply_rt(int op, Acc a, Acc b) {
    const Acc mn = b < a ? b : a, mx = b > a ? b : a, pr = (a * b) & 0xFFu;
    return op == MIN ? mn : op == MAX ? mx : pr;
  }
  static __device__ __forceinline__ Acc apply(Acc a, Acc b) {
    if (OP == SUM || OP == AVG) return (a + b) & 0xFFu;
    if (OP == PRODUCT) return (a * b) & 0xFFu;
    if (OP == MIN) return b < a ? b : a;
    return b > a ? b : a;
  }
};

template <typename T> struct VecOf {
  static constexpr int N = 16 / sizeof(T);
  union U {
    uint4 raw;
    T e[N];
    __device__ U() {}
  };
};

// Plain global 16-byte accesses.  `volatile`-free on purpose: ordering comes
// from the acquire/release flag protocol, and the no-allocate hint keeps
// streamed peer data out of L1.
__device__ __forceinline__ uint4 ld16(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st16(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Loads vector `vi` of a T array holding n elements; lanes past n read as zero.
// `aligned` says the array base is 16-byte aligned.
template <typename T>
__device__ __forceinline__ uint4 ld_vec_guarded(const T* base, int64_t vi, int64_t n, bool aligned) {
  constexpr int N = VecOf<T>::N;
  int64_t e0 = vi * N;
  if (aligned && e0 + N <= n) return ld16(base + e0);
  typename VecOf<T>::U u;
  u.raw = make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int j = 0; j < N; ++j)
    if (e0 + j < n) u.e[j] = base[e0 + j];
  return u.raw;
}
template <typename T>
__device__ __forceinline__ void st_vec_guarded(T* base, int64_t vi, int64_t n, bool aligned, uint4 v) {
  constexpr int N = VecOf<T>::N;
  int64_t e0 = vi * N;
  if (aligned && e0 + N <= n) {
    st16(base + e0, v);
    return;
  }
  typename VecOf<T>::U u;
  u.raw = v;
#pragma unroll
  for (int j = 0; j < N; ++j)
    if (e0 + j < n) base[e0 + j] = u.e[j];
}

__device__ __forceinline__ bool is_aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

}  // namespace kern
}  // namespace mccl
