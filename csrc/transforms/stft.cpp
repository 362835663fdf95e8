#include "transforms/stft.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <cmath>

#include "common/errors.h"
#include "kernels/stft_api.h"

namespace mccl {

namespace {

#define STFT_CK(expr)                                                             \
  do {                                                                            \
    cudaError_t _e = (expr);                                                      \
    if (_e != cudaSuccess) {                                                      \
      cudaGetLastError();                                                         \
      throw DeviceError(std::string(#expr) + ": " + cudaGetErrorString(_e));      \
    }                                                                             \
  } while (0)

void check_common(int64_t n_fft, int64_t hop, int64_t win_length, const at::Tensor& window,
                  const std::string& backend) {
  MCCL_CHECK_TENSOR(stft_cuda_supported(n_fft),
                    "n_fft must be a power of two in [8, " << kern::kStftMaxNfft << "], got " << n_fft);
  MCCL_CHECK_TENSOR(hop >= 1, "hop_length must be >= 1");
  MCCL_CHECK_TENSOR(win_length >= 1 && win_length <= n_fft, "win_length must be in [1, n_fft]");
  MCCL_CHECK_TENSOR(window.dim() == 1 && window.numel() == win_length, "window must be 1-D of win_length elements");
  MCCL_CHECK_TENSOR(backend == "auto" || backend == "cuda" || backend == "metal",
                    "the native STFT serves the CUDA backend (got '" << backend << "')");
}

// window of win_length centred inside n_fft zeros, fp32, on `like`'s device
at::Tensor prepare_window(const at::Tensor& window, int64_t n_fft, const at::Tensor& like) {
  at::Tensor w = window.to(like.device(), at::kFloat).contiguous();
  if (w.numel() == n_fft) return w;
  at::Tensor padded = at::zeros({n_fft}, w.options());
  const int64_t left = (n_fft - w.numel()) / 2;
  padded.narrow(0, left, w.numel()).copy_(w);
  return padded;
}

at::Tensor as_batch(const at::Tensor& x) {
  MCCL_CHECK_TENSOR(x.is_cuda() && x.scalar_type() == at::kFloat, "expected a float32 CUDA tensor");
  if (x.dim() == 1) return x.unsqueeze(0).contiguous();
  if (x.dim() == 3 && x.size(1) == 1) return x.squeeze(1).contiguous();
  MCCL_CHECK_TENSOR(x.dim() == 2, "expected [time], [batch, time] or [batch, 1, time]");
  return x.contiguous();
}

void spec_strides(const at::Tensor& spec, int64_t n_fft, int64_t& sb, int64_t& sf, int64_t& st) {
  MCCL_CHECK_TENSOR(spec.is_cuda() && spec.scalar_type() == at::kComplexFloat && spec.dim() == 3,
                    "expected a complex64 CUDA spectrum [batch, freq, frames]");
  MCCL_CHECK_TENSOR(spec.size(1) == n_fft / 2 + 1, "spectrum must have n_fft/2+1 frequency bins");
  sb = spec.stride(0);
  sf = spec.stride(1);
  st = spec.stride(2);
}

}  // namespace

bool stft_cuda_supported(int64_t n_fft) {
  return n_fft >= 8 && n_fft <= kern::kStftMaxNfft && (n_fft & (n_fft - 1)) == 0;
}

int64_t stft_num_frames(int64_t signal_len, int64_t n_fft, int64_t hop, bool center) {
  if (center) return 1 + signal_len / hop;
  MCCL_CHECK_TENSOR(signal_len >= n_fft, "signal shorter than n_fft without centering");
  return 1 + (signal_len - n_fft) / hop;
}

at::Tensor stft_forward(const at::Tensor& waveform, const at::Tensor& window, int64_t n_fft, int64_t hop,
                        int64_t win_length, bool center, bool normalized, const std::string& backend) {
  check_common(n_fft, hop, win_length, window, backend);
  at::Tensor x = as_batch(waveform);
  const int64_t B = x.size(0), T = x.size(1);
  const int64_t pad = center ? n_fft / 2 : 0;
  MCCL_CHECK_TENSOR(!center || T > pad, "reflect padding needs a signal longer than n_fft/2");
  const int64_t frames = stft_num_frames(T, n_fft, hop, center);
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor w = prepare_window(window, n_fft, x);
  at::Tensor out = at::empty({B, frames, n_fft / 2 + 1}, x.options().dtype(at::kComplexFloat));
  kern::FftFramesArgs a{};
  a.signal = x.data_ptr<float>();
  a.signal_len = T;
  a.window = w.data_ptr<float>();
  a.out = reinterpret_cast<float*>(out.data_ptr());
  a.batch = static_cast<int>(B);
  a.n_frames = static_cast<int>(frames);
  a.n_fft = static_cast<int>(n_fft);
  a.hop = static_cast<int>(hop);
  a.pad = static_cast<int>(pad);
  a.reflect = center ? 1 : 0;
  a.divide_envelope = 0;
  a.scale = normalized ? 1.0f / std::sqrt(static_cast<float>(n_fft)) : 1.0f;
  a.hermitian_weights = 0;
  STFT_CK(kern::launch_fft_frames(a, at::cuda::getCurrentCUDAStream()));
  return out.transpose(1, 2);  // [batch, freq, frames]; frames-major storage keeps the kernel's writes coalesced
}

at::Tensor stft_backward(const at::Tensor& grad_spec, const at::Tensor& window, int64_t n_fft, int64_t hop,
                         int64_t win_length, bool center, bool normalized, int64_t length,
                         const std::string& backend) {
  check_common(n_fft, hop, win_length, window, backend);
  int64_t sb, sf, st;
  spec_strides(grad_spec, n_fft, sb, sf, st);
  const int64_t B = grad_spec.size(0), frames = grad_spec.size(2);
  c10::cuda::CUDAGuard guard(grad_spec.device());
  at::Tensor w = prepare_window(window, n_fft, grad_spec);
  at::Tensor buf = at::empty({B, frames, n_fft}, grad_spec.options().dtype(at::kFloat));
  kern::IfftFramesArgs a{};
  a.spec = reinterpret_cast<const float*>(grad_spec.data_ptr());
  a.stride_b = sb;
  a.stride_f = sf;
  a.stride_t = st;
  a.window = w.data_ptr<float>();
  a.frames = buf.data_ptr<float>();
  a.batch = static_cast<int>(B);
  a.n_frames = static_cast<int>(frames);
  a.n_fft = static_cast<int>(n_fft);
  a.hermitian = 0;  // adjoint of the one-sided forward transform: upper bins contribute nothing
  a.scale = normalized ? 1.0f / std::sqrt(static_cast<float>(n_fft)) : 1.0f;
  auto stream = at::cuda::getCurrentCUDAStream();
  STFT_CK(kern::launch_ifft_frames(a, stream));
  at::Tensor out = at::empty({B, length}, buf.options());
  kern::OlaArgs o{};
  o.frames = buf.data_ptr<float>();
  o.window = w.data_ptr<float>();
  o.out = out.data_ptr<float>();
  o.batch = static_cast<int>(B);
  o.n_frames = static_cast<int>(frames);
  o.n_fft = static_cast<int>(n_fft);
  o.hop = static_cast<int>(hop);
  o.out_len = length;
  o.pad = center ? static_cast<int>(n_fft / 2) : 0;
  o.fold_reflect = center ? 1 : 0;
  o.normalize_envelope = 0;
  STFT_CK(kern::launch_ola_gather(o, stream));
  return out;
}

at::Tensor istft_forward(const at::Tensor& spec, const at::Tensor& window, int64_t n_fft, int64_t hop,
                         int64_t win_length, bool center, bool normalized, int64_t length,
                         const std::string& backend) {
  check_common(n_fft, hop, win_length, window, backend);
  int64_t sb, sf, st;
  spec_strides(spec, n_fft, sb, sf, st);
  const int64_t B = spec.size(0), frames = spec.size(2);
  MCCL_CHECK_TENSOR(length >= 1, "length must be >= 1");
  c10::cuda::CUDAGuard guard(spec.device());
  at::Tensor w = prepare_window(window, n_fft, spec);
  at::Tensor buf = at::empty({B, frames, n_fft}, spec.options().dtype(at::kFloat));
  kern::IfftFramesArgs a{};
  a.spec = reinterpret_cast<const float*>(spec.data_ptr());
  a.stride_b = sb;
  a.stride_f = sf;
  a.stride_t = st;
  a.window = w.data_ptr<float>();
  a.frames = buf.data_ptr<float>();
  a.batch = static_cast<int>(B);
  a.n_frames = static_cast<int>(frames);
  a.n_fft = static_cast<int>(n_fft);
  a.hermitian = 1;
  a.scale = (normalized ? std::sqrt(static_cast<float>(n_fft)) : 1.0f) / static_cast<float>(n_fft);
  auto stream = at::cuda::getCurrentCUDAStream();
  STFT_CK(kern::launch_ifft_frames(a, stream));
  at::Tensor out = at::empty({B, length}, buf.options());
  kern::OlaArgs o{};
  o.frames = buf.data_ptr<float>();
  o.window = w.data_ptr<float>();
  o.out = out.data_ptr<float>();
  o.batch = static_cast<int>(B);
  o.n_frames = static_cast<int>(frames);
  o.n_fft = static_cast<int>(n_fft);
  o.hop = static_cast<int>(hop);
  o.out_len = length;
  o.pad = center ? static_cast<int>(n_fft / 2) : 0;
  o.fold_reflect = 0;
  o.normalize_envelope = 1;
  STFT_CK(kern::launch_ola_gather(o, stream));
  return out;
}

at::Tensor istft_backward(const at::Tensor& grad_waveform, const at::Tensor& window, int64_t n_fft, int64_t hop,
                          int64_t win_length, bool center, bool normalized, int64_t n_frames,
                          const std::string& backend) {
  check_common(n_fft, hop, win_length, window, backend);
  at::Tensor g = as_batch(grad_waveform);
  const int64_t B = g.size(0), T = g.size(1);
  c10::cuda::CUDAGuard guard(g.device());
  at::Tensor w = prepare_window(window, n_fft, g);
  at::Tensor out = at::empty({B, n_frames, n_fft / 2 + 1}, g.options().dtype(at::kComplexFloat));
  kern::FftFramesArgs a{};
  a.signal = g.data_ptr<float>();
  a.signal_len = T;
  a.window = w.data_ptr<float>();
  a.out = reinterpret_cast<float*>(out.data_ptr());
  a.batch = static_cast<int>(B);
  a.n_frames = static_cast<int>(n_frames);
  a.n_fft = static_cast<int>(n_fft);
  a.hop = static_cast<int>(hop);
  a.pad = center ? static_cast<int>(n_fft / 2) : 0;
  a.reflect = 0;
  a.divide_envelope = 1;
  a.scale = (normalized ? std::sqrt(static_cast<float>(n_fft)) : 1.0f) / static_cast<float>(n_fft);
  a.hermitian_weights = 1;
  STFT_CK(kern::launch_fft_frames(a, at::cuda::getCurrentCUDAStream()));
  return out.transpose(1, 2);
}

}  // namespace mccl
