// STFT / iSTFT front-end for CUDA tensors (argument checks, window padding,
// frame counts, kernel launches).  Semantics follow torch.stft / torch.istft
// with a one-sided complex64 spectrum [batch, n_fft/2+1, n_frames], reflect
// padding when `center`, and 1/sqrt(n_fft) scaling when `normalized`.
// Parity: reference csrc/transforms/Stft.hpp:27-55, Stft.mm:213-423,
// StftCommon.mm:11-70 (frame counts, reflect padding, window preparation).
// n_fft must be a power of two in [8, 4096] (the reference's Metal path had the
// same upper bound, reference csrc/transforms/StftMetalKernels.mm:209).
#pragma once

#include <ATen/ATen.h>

#include <string>

namespace mccl {

int64_t stft_num_frames(int64_t signal_len, int64_t n_fft, int64_t hop, bool center);
bool stft_cuda_supported(int64_t n_fft);

at::Tensor stft_forward(const at::Tensor& waveform, const at::Tensor& window, int64_t n_fft, int64_t hop_length,
                        int64_t win_length, bool center, bool normalized, const std::string& backend);
at::Tensor stft_backward(const at::Tensor& grad_spec, const at::Tensor& window, int64_t n_fft, int64_t hop_length,
                         int64_t win_length, bool center, bool normalized, int64_t length,
                         const std::string& backend);
at::Tensor istft_forward(const at::Tensor& spec, const at::Tensor& window, int64_t n_fft, int64_t hop_length,
                         int64_t win_length, bool center, bool normalized, int64_t length,
                         const std::string& backend);
at::Tensor istft_backward(const at::Tensor& grad_waveform, const at::Tensor& window, int64_t n_fft,
                          int64_t hop_length, int64_t win_length, bool center, bool normalized, int64_t n_frames,
                          const std::string& backend);

}  // namespace mccl
