// Portable host reductions: the CPU-tensor data path, the oracle for the CUDA
// elementwise kernels and the timed CPU baseline.
//
// Semantics (shared with the device kernels):
//  * SUM/AVG/MIN/MAX/PRODUCT over f32, f64, f16, bf16, i32, i64, u8, bool.
//  * 16-bit floats are widened to fp32 for every operation and narrowed once.
//  * bool: SUM and MAX are logical OR, PRODUCT and MIN are logical AND.
//  * AVG is "accumulate, then scale by 1/world": i32 rounds to nearest
//    (half away from zero), i64 and u8 truncate towards zero, bool rejects it.
// Parity: reference csrc/metal/AccelerateOps.mm:29-276 and
// csrc/metal/shaders.metal:622-665 (integer AVG rules).
#pragma once

#include <ATen/ATen.h>
#include <torch/csrc/distributed/c10d/Types.hpp>

namespace mccl {

// dst[i] = op(dst[i], src[i]); AVG accumulates like SUM (scaling is separate).
void cpu_reduce_into(void* dst, const void* src, int64_t count, at::ScalarType dtype,
                     c10d::ReduceOp::RedOpType op);
// buf[i] = buf[i] * scale with the integer rules above.
void cpu_scale_inplace(void* buf, int64_t count, at::ScalarType dtype, double scale);
// dst[i] = (dst[i] + src[i]) * scale (floating dtypes).
void cpu_accumulate_and_scale(void* dst, const void* src, int64_t count, at::ScalarType dtype,
                              double scale);

bool is_reduce_dtype(at::ScalarType t);

}  // namespace mccl
