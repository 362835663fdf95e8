// Argument validation shared by every collective entry point.
//
// Rules (reference csrc/common/TensorChecks.hpp:10-33 and
// csrc/backend/ProcessGroupMCCL.cpp:64-67,1040-1045): tensors live on cpu or
// cuda, are dense and contiguous (a non-contiguous in-place output is rejected
// loudly rather than silently copied), and have one of the supported dtypes
// f32, f64, f16, bf16, i32, i64, u8, bool.  A rejected call leaves the process
// group usable.
#pragma once

#include <ATen/ATen.h>
#include <torch/csrc/distributed/c10d/Types.hpp>

#include "common/errors.h"
#include "compression/compressor.h"
#include "kernels/api.h"

namespace mccl {

inline bool dtype_supported(at::ScalarType t) {
  switch (t) {
    case at::kFloat: case at::kDouble: case at::kHalf: case at::kBFloat16:
    case at::kInt: case at::kLong: case at::kByte: case at::kBool:
      return true;
    default:
      return false;
  }
}

inline void check_tensor(const at::Tensor& t, const char* what) {
  MCCL_CHECK_TENSOR(t.defined(), what << ": undefined tensor");
  MCCL_CHECK_TENSOR(t.device().is_cpu() || t.device().is_cuda(),
                    what << ": tensors must live on cpu or cuda, got " << t.device());
  MCCL_CHECK_TENSOR(!t.is_sparse() && t.layout() == at::kStrided, what << ": dense strided tensors only");
  MCCL_CHECK_TENSOR(t.is_contiguous(), what << ": tensor must be contiguous (call .contiguous() first)");
  MCCL_CHECK_TENSOR(dtype_supported(t.scalar_type()),
                    what << ": unsupported dtype " << c10::toString(t.scalar_type())
                         << " (supported: float32 float64 float16 bfloat16 int32 int64 uint8 bool)");
}

inline void check_single(const std::vector<at::Tensor>& v, const char* what) {
  MCCL_CHECK_TENSOR(v.size() == 1, what << ": expected exactly one tensor, got " << v.size());
  check_tensor(v[0], what);
}

inline void check_same(const at::Tensor& a, const at::Tensor& b, const char* what) {
  MCCL_CHECK_TENSOR(a.scalar_type() == b.scalar_type(), what << ": dtype mismatch");
  MCCL_CHECK_TENSOR(a.numel() == b.numel(), what << ": element count mismatch (" << a.numel() << " vs " << b.numel() << ")");
  MCCL_CHECK_TENSOR(a.device() == b.device(), what << ": device mismatch");
}

inline kern::DType to_kern_dtype(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return kern::F32;
    case at::kDouble: return kern::F64;
    case at::kHalf: return kern::F16;
    case at::kBFloat16: return kern::BF16;
    case at::kInt: return kern::I32;
    case at::kLong: return kern::I64;
    case at::kByte: return kern::U8;
    case at::kBool: return kern::BOOL;
    default: throw TensorError(std::string("unsupported dtype ") + c10::toString(t));
  }
}

inline kern::RedOp to_kern_op(c10d::ReduceOp::RedOpType op) {
  switch (op) {
    case c10d::ReduceOp::SUM: return kern::SUM;
    case c10d::ReduceOp::AVG: return kern::AVG;
    case c10d::ReduceOp::MIN: return kern::MIN;
    case c10d::ReduceOp::MAX: return kern::MAX;
    case c10d::ReduceOp::PRODUCT: return kern::PRODUCT;
    default: throw TensorError("unsupported reduce op (supported: SUM AVG MIN MAX PRODUCT)");
  }
}

inline void check_reduce_op(c10d::ReduceOp::RedOpType op, at::ScalarType t) {
  (void)to_kern_op(op);
  MCCL_CHECK_TENSOR(!(t == at::kBool && op == c10d::ReduceOp::AVG), "AVG is not defined for bool tensors");
}

inline WireDType to_wire_dtype(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return WireDType::F32;
    case at::kHalf: return WireDType::F16;
    case at::kBFloat16: return WireDType::BF16;
    default: return WireDType::OTHER;
  }
}

}  // namespace mccl
