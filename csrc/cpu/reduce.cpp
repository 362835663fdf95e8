#include "cpu/reduce.h"

#include <algorithm>
#include <cmath>
#include <limits>
#include <thread>
#include <type_traits>
#include <vector>

#include "common/errors.h"

namespace mccl {

namespace {

using Op = c10d::ReduceOp::RedOpType;

// Splits [0, n) over a few threads once the range is large enough to pay for it.
template <typename F>
void parallel_range(int64_t n, F&& body) {
  constexpr int64_t kMinPerThread = 1 << 20;
  int64_t want = std::min<int64_t>(8, n / kMinPerThread);
  unsigned hw = std::thread::hardware_concurrency();
  if (hw > 0) want = std::min<int64_t>(want, hw);
  if (want <= 1) {
    body(0, n);
    return;
  }
  std::vector<std::thread> th;
  int64_t per = (n + want - 1) / want;
  for (int64_t t = 0; t < want; ++t) {
    int64_t b = t * per, e = std::min(n, b + per);
    if (b >= e) break;
    th.emplace_back([=, &body] { body(b, e); });
  }
  for (auto& t : th) t.join();
}

// MIN / MAX that give the same bits whichever operand comes first: a NaN on either side yields
// the canonical quiet NaN (as torch and NCCL propagate it), and of +0 / -0 the minimum is -0 and
// the maximum +0.  Two ranks that reduce the same pair in opposite orders therefore agree.
template <typename A>
inline A ordered_min(A x, A y) {
  if constexpr (std::is_floating_point<A>::value) {
    if (std::isnan(x) || std::isnan(y)) return std::numeric_limits<A>::quiet_NaN();
    if (x == y) return std::signbit(x) ? x : y;
  }
  return y < x ? y : x;
}
template <typename A>
inline A ordered_max(A x, A y) {
  if constexpr (std::is_floating_point<A>::value) {
    if (std::isnan(x) || std::isnan(y)) return std::numeric_limits<A>::quiet_NaN();
    if (x == y) return std::signbit(x) ? y : x;
  }
  return y > x ? y : x;
}

template <typename T, typename Acc>
void reduce_typed(T* d, const T* s, int64_t n, Op op) {
  parallel_range(n, [=](int64_t b, int64_t e) {
    switch (op) {
      case Op::SUM:
      case Op::AVG:
        for (int64_t i = b; i < e; ++i) d[i] = static_cast<T>(static_cast<Acc>(d[i]) + static_cast<Acc>(s[i]));
        break;
      case Op::PRODUCT:
        for (int64_t i = b; i < e; ++i) d[i] = static_cast<T>(static_cast<Acc>(d[i]) * static_cast<Acc>(s[i]));
        break;
      case Op::MIN:
        for (int64_t i = b; i < e; ++i) {
          Acc x = static_cast<Acc>(d[i]), y = static_cast<Acc>(s[i]);
          d[i] = static_cast<T>(ordered_min<Acc>(x, y));
        }
        break;
      case Op::MAX:
        for (int64_t i = b; i < e; ++i) {
          Acc x = static_cast<Acc>(d[i]), y = static_cast<Acc>(s[i]);
          d[i] = static_cast<T>(ordered_max<Acc>(x, y));
        }
        break;
      default:
        throw TensorError("unsupported reduce op");
    }
  });
}

void reduce_bool(bool* d, const bool* s, int64_t n, Op op) {
  switch (op) {
    case Op::SUM:
    case Op::MAX:
      for (int64_t i = 0; i < n; ++i) d[i] = d[i] || s[i];
      break;
    case Op::PRODUCT:
    case Op::MIN:
      for (int64_t i = 0; i < n; ++i) d[i] = d[i] && s[i];
      break;
    default:
      throw TensorError("reduce op not supported for bool tensors");
  }
}

}  // namespace

bool is_reduce_dtype(at::ScalarType t) {
  switch (t) {
    case at::kFloat:
    case at::kDouble:
    case at::kHalf:
    case at::kBFloat16:
    case at::kInt:
    case at::kLong:
    case at::kByte:
    case at::kBool:
      return true;
    default:
      return false;
  }
}

void cpu_reduce_into(void* dst, const void* src, int64_t n, at::ScalarType dtype, Op op) {
  switch (dtype) {
    case at::kFloat: reduce_typed<float, float>((float*)dst, (const float*)src, n, op); break;
    case at::kDouble: reduce_typed<double, double>((double*)dst, (const double*)src, n, op); break;
    case at::kHalf: reduce_typed<at::Half, float>((at::Half*)dst, (const at::Half*)src, n, op); break;
    case at::kBFloat16:
      reduce_typed<at::BFloat16, float>((at::BFloat16*)dst, (const at::BFloat16*)src, n, op);
      break;
    case at::kInt: reduce_typed<int32_t, int32_t>((int32_t*)dst, (const int32_t*)src, n, op); break;
    case at::kLong: reduce_typed<int64_t, int64_t>((int64_t*)dst, (const int64_t*)src, n, op); break;
    case at::kByte: reduce_typed<uint8_t, uint8_t>((uint8_t*)dst, (const uint8_t*)src, n, op); break;
    case at::kBool: reduce_bool((bool*)dst, (const bool*)src, n, op); break;
    default:
      throw TensorError(std::string("unsupported dtype for reduction: ") + c10::toString(dtype));
  }
}

void cpu_scale_inplace(void* buf, int64_t n, at::ScalarType dtype, double scale) {
  switch (dtype) {
    case at::kFloat: {
      float* p = (float*)buf;
      float s = static_cast<float>(scale);
      parallel_range(n, [=](int64_t b, int64_t e) { for (int64_t i = b; i < e; ++i) p[i] *= s; });
      break;
    }
    case at::kDouble: {
      double* p = (double*)buf;
      for (int64_t i = 0; i < n; ++i) p[i] *= scale;
      break;
    }
    case at::kHalf: {
      at::Half* p = (at::Half*)buf;
      float s = static_cast<float>(scale);
      for (int64_t i = 0; i < n; ++i) p[i] = static_cast<at::Half>(static_cast<float>(p[i]) * s);
      break;
    }
    case at::kBFloat16: {
      at::BFloat16* p = (at::BFloat16*)buf;
      float s = static_cast<float>(scale);
      for (int64_t i = 0; i < n; ++i) p[i] = static_cast<at::BFloat16>(static_cast<float>(p[i]) * s);
      break;
    }
    case at::kInt: {
      int32_t* p = (int32_t*)buf;
      float s = static_cast<float>(scale);
      for (int64_t i = 0; i < n; ++i) p[i] = static_cast<int32_t>(std::round(static_cast<float>(p[i]) * s));
      break;
    }
    case at::kLong: {
      int64_t* p = (int64_t*)buf;
      for (int64_t i = 0; i < n; ++i) p[i] = static_cast<int64_t>(static_cast<double>(p[i]) * scale);
      break;
    }
    case at::kByte: {
      uint8_t* p = (uint8_t*)buf;
      float s = static_cast<float>(scale);
      for (int64_t i = 0; i < n; ++i) p[i] = static_cast<uint8_t>(static_cast<float>(p[i]) * s);
      break;
    }
    default:
      throw TensorError(std::string("unsupported dtype for scaling: ") + c10::toString(dtype));
  }
}

void cpu_accumulate_and_scale(void* dst, const void* src, int64_t n, at::ScalarType dtype,
                              double scale) {
  float s = static_cast<float>(scale);
  switch (dtype) {
    case at::kFloat: {
      float* d = (float*)dst;
      const float* a = (const float*)src;
      for (int64_t i = 0; i < n; ++i) d[i] = (d[i] + a[i]) * s;
      break;
    }
    case at::kHalf: {
      at::Half* d = (at::Half*)dst;
      const at::Half* a = (const at::Half*)src;
      for (int64_t i = 0; i < n; ++i)
        d[i] = static_cast<at::Half>((static_cast<float>(d[i]) + static_cast<float>(a[i])) * s);
      break;
    }
    case at::kBFloat16: {
      at::BFloat16* d = (at::BFloat16*)dst;
      const at::BFloat16* a = (const at::BFloat16*)src;
      for (int64_t i = 0; i < n; ++i)
        d[i] = static_cast<at::BFloat16>((static_cast<float>(d[i]) + static_cast<float>(a[i])) * s);
      break;
    }
    case at::kDouble: {
      double* d = (double*)dst;
      const double* a = (const double*)src;
      for (int64_t i = 0; i < n; ++i) d[i] = (d[i] + a[i]) * scale;
      break;
    }
    default:
      throw TensorError("accumulate_and_scale supports floating dtypes only");
  }
}

}  // namespace mccl
