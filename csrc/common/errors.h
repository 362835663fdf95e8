// Exception hierarchy of the native layer.  Every failure that reaches Python
// is one of these (pybind maps std::runtime_error to RuntimeError).
// Parity: reference csrc/common/Errors.hpp:9-66 (MetalError becomes DeviceError).
#pragma once

#include <sstream>
#include <stdexcept>
#include <string>

namespace mccl {

class MCCLError : public std::runtime_error {
 public:
  explicit MCCLError(const std::string& m) : std::runtime_error("MCCL: " + m) {}
};
class TransportError : public MCCLError {
 public:
  explicit TransportError(const std::string& m) : MCCLError("transport: " + m) {}
};
class DeviceError : public MCCLError {
 public:
  explicit DeviceError(const std::string& m) : MCCLError("device: " + m) {}
};
class TensorError : public MCCLError {
 public:
  explicit TensorError(const std::string& m) : MCCLError("tensor: " + m) {}
};
class TimeoutError : public MCCLError {
 public:
  explicit TimeoutError(const std::string& m) : MCCLError("timeout: " + m) {}
};
class ProtocolError : public MCCLError {
 public:
  explicit ProtocolError(const std::string& m) : MCCLError("protocol: " + m) {}
};

}  // namespace mccl

#define MCCL_CHECK_T(ExcType, cond, ...)                                   \
  do {                                                                     \
    if (!(cond)) {                                                         \
      std::ostringstream _mccl_oss;                                        \
      _mccl_oss << __VA_ARGS__ << " (" #cond " failed at " << __FILE__     \
                << ":" << __LINE__ << ")";                                 \
      throw ExcType(_mccl_oss.str());                                      \
    }                                                                      \
  } while (0)

#define MCCL_CHECK(cond, ...) MCCL_CHECK_T(::mccl::MCCLError, cond, __VA_ARGS__)
#define MCCL_CHECK_TENSOR(cond, ...) MCCL_CHECK_T(::mccl::TensorError, cond, __VA_ARGS__)
#define MCCL_CHECK_TRANSPORT(cond, ...) MCCL_CHECK_T(::mccl::TransportError, cond, __VA_ARGS__)

#define MCCL_CUDA_CHECK(expr)                                              \
  do {                                                                     \
    cudaError_t _e = (expr);                                               \
    if (_e != cudaSuccess) {                                               \
      std::ostringstream _mccl_oss;                                        \
      _mccl_oss << #expr << " -> " << cudaGetErrorName(_e) << ": "         \
                << cudaGetErrorString(_e) << " at " << __FILE__ << ":"     \
                << __LINE__;                                               \
      throw ::mccl::DeviceError(_mccl_oss.str());                          \
    }                                                                      \
  } while (0)
