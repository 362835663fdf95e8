// Host-side gradient compressors (the CPU data path and the oracle for the
// fused GPU kernels).
//
// FP16: fp32 payloads travel as IEEE half (round-to-nearest-even, NaN/Inf
// preserved, half-subnormal results flushed to signed zero); fp16 payloads pass
// through; other dtypes are rejected.
//
// TopK (fp32 only): k = max(1, floor(count * ratio)).  The compressor keeps one
// fp32 error-feedback residual per `stable_id` (the identity of the gradient
// bucket).  compress(): adjusted = g + residual; select the k entries of
// largest |adjusted| (ties broken towards the lower index); emit them sorted by
// index; residual = adjusted with the k sent entries zeroed.  Wire format:
// [u32 k][k x (u32 index, f32 value)].  decompress(): zero-fill then scatter,
// rejecting out-of-range indices.  At most 1024 residual buffers are kept; on
// overflow all are dropped.
// Parity: reference csrc/compression/Compression.hpp:22-52,
// FP16Compression.cpp:16-165, TopKCompression.cpp:42-152.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace mccl {

enum class CompressionMode : int { NONE = 0, FP16 = 1, TOPK = 2 };

// Minimal dtype tag for host code that must not depend on ATen.
enum class WireDType : int { F32 = 0, F16 = 1, BF16 = 2, OTHER = 3 };

class Compressor {
 public:
  virtual ~Compressor() = default;
  // Returns the number of bytes written to dst (<= cap).
  virtual size_t compress(const void* src, size_t nbytes, void* dst, size_t cap, WireDType dtype,
                          uint64_t stable_id) = 0;
  // Expands `src` (csize bytes) into dst (nbytes of dtype).
  virtual void decompress(const void* src, size_t csize, void* dst, size_t nbytes,
                          WireDType dtype) = 0;
  virtual size_t max_compressed_size(size_t nbytes, WireDType dtype) const = 0;
  virtual std::string name() const = 0;
  virtual CompressionMode mode() const = 0;
};

class FP16Compressor : public Compressor {
 public:
  size_t compress(const void* src, size_t nbytes, void* dst, size_t cap, WireDType dtype,
                  uint64_t stable_id) override;
  void decompress(const void* src, size_t csize, void* dst, size_t nbytes, WireDType dtype) override;
  size_t max_compressed_size(size_t nbytes, WireDType dtype) const override;
  std::string name() const override { return "fp16"; }
  CompressionMode mode() const override { return CompressionMode::FP16; }
};

class TopKCompressor : public Compressor {
 public:
  explicit TopKCompressor(double ratio);
  size_t compress(const void* src, size_t nbytes, void* dst, size_t cap, WireDType dtype,
                  uint64_t stable_id) override;
  void decompress(const void* src, size_t csize, void* dst, size_t nbytes, WireDType dtype) override;
  size_t max_compressed_size(size_t nbytes, WireDType dtype) const override;
  std::string name() const override { return "topk"; }
  CompressionMode mode() const override { return CompressionMode::TOPK; }

  size_t k_for(size_t count) const;
  void reset_error_feedback();
  void reset_error_feedback(uint64_t stable_id);
  size_t residual_buffers() const;
  // Copy of the residual for `stable_id` (empty if none).
  std::vector<float> residual(uint64_t stable_id) const;

  static constexpr size_t kMaxResidualBuffers = 1024;

 private:
  double ratio_;
  mutable std::mutex mu_;
  std::unordered_map<uint64_t, std::vector<float>> residuals_;
};

std::unique_ptr<Compressor> make_compressor(CompressionMode mode, double param);
CompressionMode parse_compression_mode(const std::string& s);

// Scalar conversions shared with the CPU reduce path and the tests.
uint16_t float_to_half_bits(float f);
float half_bits_to_float(uint16_t h);
uint16_t float_to_bf16_bits(float f);
float bf16_bits_to_float(uint16_t h);

}  // namespace mccl
