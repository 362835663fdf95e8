#include "compression/compressor.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <numeric>

#include "common/errors.h"

namespace mccl {

// ---- scalar conversions ---------------------------------------------------

uint16_t float_to_half_bits(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const uint32_t absx = x & 0x7FFFFFFFu;
  if (absx >= 0x7F800000u) {  // Inf / NaN
    return static_cast<uint16_t>(sign | 0x7C00u | (absx > 0x7F800000u ? 0x0200u : 0));
  }
  if (absx >= 0x477FF000u) {  // rounds to >= 65520 -> Inf
    return static_cast<uint16_t>(sign | 0x7C00u);
  }
  if (absx < 0x38800000u) {  // below the smallest normal half: flush to signed zero
    return static_cast<uint16_t>(sign);
  }
  uint32_t mant = absx & 0x007FFFFFu;
  uint32_t exp = (absx >> 23) - 112;  // rebias 127 -> 15
  uint32_t h = (exp << 10) | (mant >> 13);
  uint32_t rem = mant & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) h += 1;  // round to nearest even
  return static_cast<uint16_t>(sign | h);
}

float half_bits_to_float(uint16_t h) {
  uint32_t sign = (static_cast<uint32_t>(h) & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1F;
  uint32_t mant = h & 0x3FF;
  uint32_t x;
  if (exp == 0) {
    if (mant == 0) {
      x = sign;
    } else {  // subnormal half -> normal float
      int e = -1;
      do {
        ++e;
        mant <<= 1;
      } while ((mant & 0x400) == 0);
      x = sign | ((112 - e) << 23) | ((mant & 0x3FF) << 13);
    }
  } else if (exp == 31) {
    x = sign | 0x7F800000u | (mant << 13);
  } else {
    x = sign | ((exp + 112) << 23) | (mant << 13);
  }
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}

uint16_t float_to_bf16_bits(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return static_cast<uint16_t>((x >> 16) | 0x0040u);  // quiet NaN
  uint32_t lsb = (x >> 16) & 1;
  x += 0x7FFFu + lsb;
  return static_cast<uint16_t>(x >> 16);
}

float bf16_bits_to_float(uint16_t h) {
  uint32_t x = static_cast<uint32_t>(h) << 16;
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}

// ---- FP16 -----------------------------------------------------------------

size_t FP16Compressor::max_compressed_size(size_t nbytes, WireDType dtype) const {
  return dtype == WireDType::F32 ? nbytes / 2 : nbytes;
}

size_t FP16Compressor::compress(const void* src, size_t nbytes, void* dst, size_t cap,
                                WireDType dtype, uint64_t) {
  if (dtype == WireDType::F16) {
    MCCL_CHECK(cap >= nbytes, "fp16 compressor: destination too small");
    std::memcpy(dst, src, nbytes);
    return nbytes;
  }
  MCCL_CHECK(dtype == WireDType::F32, "fp16 compression supports float32 and float16 tensors only");
  size_t n = nbytes / 4;
  MCCL_CHECK(cap >= n * 2, "fp16 compressor: destination too small");
  const float* s = static_cast<const float*>(src);
  uint16_t* d = static_cast<uint16_t*>(dst);
  for (size_t i = 0; i < n; ++i) d[i] = float_to_half_bits(s[i]);
  return n * 2;
}

void FP16Compressor::decompress(const void* src, size_t csize, void* dst, size_t nbytes,
                                WireDType dtype) {
  if (dtype == WireDType::F16) {
    MCCL_CHECK(csize == nbytes, "fp16 passthrough size mismatch");
    std::memcpy(dst, src, nbytes);
    return;
  }
  MCCL_CHECK(dtype == WireDType::F32, "fp16 compression supports float32 and float16 tensors only");
  size_t n = nbytes / 4;
  MCCL_CHECK(csize == n * 2, "fp16 payload size mismatch: " << csize << " vs " << n * 2);
  const uint16_t* s = static_cast<const uint16_t*>(src);
  float* d = static_cast<float*>(dst);
  for (size_t i = 0; i < n; ++i) d[i] = half_bits_to_float(s[i]);
}

// ---- TopK -----------------------------------------------------------------

TopKCompressor::TopKCompressor(double ratio) : ratio_(ratio) {
  MCCL_CHECK(ratio > 0.0 && ratio <= 1.0, "topk ratio must be in (0, 1], got " << ratio);
}

size_t TopKCompressor::k_for(size_t count) const {
  size_t k = static_cast<size_t>(std::floor(static_cast<double>(count) * ratio_));
  k = std::max<size_t>(k, 1);
  return std::min(k, count);
}

size_t TopKCompressor::max_compressed_size(size_t nbytes, WireDType) const {
  size_t count = nbytes / 4;
  return 4 + k_for(count) * 8;
}

size_t TopKCompressor::compress(const void* src, size_t nbytes, void* dst, size_t cap,
                                WireDType dtype, uint64_t stable_id) {
  MCCL_CHECK(dtype == WireDType::F32, "topk compression supports float32 tensors only");
  const size_t count = nbytes / 4;
  MCCL_CHECK(count > 0 && count <= 0xFFFFFFFFull, "topk: element count out of range");
  const size_t k = k_for(count);
  MCCL_CHECK(cap >= 4 + k * 8, "topk compressor: destination too small");
  const float* g = static_cast<const float*>(src);

  std::lock_guard<std::mutex> lk(mu_);
  auto it = residuals_.find(stable_id);
  if (it == residuals_.end()) {
    if (residuals_.size() >= kMaxResidualBuffers) residuals_.clear();
    it = residuals_.emplace(stable_id, std::vector<float>(count, 0.f)).first;
  } else if (it->second.size() != count) {
    it->second.assign(count, 0.f);
  }
  std::vector<float>& res = it->second;
  for (size_t i = 0; i < count; ++i) res[i] += g[i];  // res now holds `adjusted`

  std::vector<uint32_t> idx(count);
  std::iota(idx.begin(), idx.end(), 0u);
  auto bigger = [&](uint32_t a, uint32_t b) {
    float fa = std::fabs(res[a]), fb = std::fabs(res[b]);
    if (fa != fb) return fa > fb;
    return a < b;
  };
  if (k < count) std::nth_element(idx.begin(), idx.begin() + k, idx.end(), bigger);
  std::sort(idx.begin(), idx.begin() + k);

  uint8_t* out = static_cast<uint8_t*>(dst);
  uint32_t k32 = static_cast<uint32_t>(k);
  std::memcpy(out, &k32, 4);
  out += 4;
  for (size_t j = 0; j < k; ++j) {
    uint32_t i = idx[j];
    float v = res[i];
    std::memcpy(out, &i, 4);
    std::memcpy(out + 4, &v, 4);
    out += 8;
    res[i] = 0.f;  // sent: no residual left for this entry
  }
  return 4 + k * 8;
}

void TopKCompressor::decompress(const void* src, size_t csize, void* dst, size_t nbytes,
                                WireDType dtype) {
  MCCL_CHECK(dtype == WireDType::F32, "topk compression supports float32 tensors only");
  MCCL_CHECK(csize >= 4, "topk payload truncated");
  const uint8_t* in = static_cast<const uint8_t*>(src);
  uint32_t k;
  std::memcpy(&k, in, 4);
  MCCL_CHECK(csize == 4 + static_cast<size_t>(k) * 8, "topk payload size mismatch");
  const size_t count = nbytes / 4;
  float* d = static_cast<float*>(dst);
  std::memset(d, 0, nbytes);
  in += 4;
  for (uint32_t j = 0; j < k; ++j) {
    uint32_t i;
    float v;
    std::memcpy(&i, in, 4);
    std::memcpy(&v, in + 4, 4);
    in += 8;
    MCCL_CHECK(i < count, "topk index " << i << " out of range " << count);
    d[i] = v;
  }
}

void TopKCompressor::reset_error_feedback() {
  std::lock_guard<std::mutex> lk(mu_);
  residuals_.clear();
}
void TopKCompressor::reset_error_feedback(uint64_t stable_id) {
  std::lock_guard<std::mutex> lk(mu_);
  residuals_.erase(stable_id);
}
size_t TopKCompressor::residual_buffers() const {
  std::lock_guard<std::mutex> lk(mu_);
  return residuals_.size();
}
std::vector<float> TopKCompressor::residual(uint64_t stable_id) const {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = residuals_.find(stable_id);
  return it == residuals_.end() ? std::vector<float>() : it->second;
}

std::unique_ptr<Compressor> make_compressor(CompressionMode mode, double param) {
  switch (mode) {
    case CompressionMode::FP16: return std::make_unique<FP16Compressor>();
    case CompressionMode::TOPK: return std::make_unique<TopKCompressor>(param);
    default: return nullptr;
  }
}

CompressionMode parse_compression_mode(const std::string& s) {
  if (s == "fp16" || s == "FP16") return CompressionMode::FP16;
  if (s == "topk" || s == "TOPK") return CompressionMode::TOPK;
  return CompressionMode::NONE;
}

}  // namespace mccl
