// Launchers of the STFT / iSTFT kernels (plain C++ header).
//
// Two kernels cover forward and backward of both transforms:
//   frames -> spectrum  (fft_frames):  one CTA per (batch, frame) loads n_fft
//       samples (reflect padding or an envelope division fused into the load),
//       multiplies by the window, runs a shared-memory radix-4 Stockham FFT and writes
//       the n_fft/2+1 one-sided bins.
//   spectrum -> frames  (ifft_frames): one CTA per (batch, frame) loads the
//       one-sided bins (Hermitian-extended for an inverse real FFT, or
//       zero-extended for the adjoint of the forward transform), runs the
//       inverse FFT, multiplies by the window and writes a real frame; a gather
//       kernel (ola_gather) then overlap-adds the frames without atomics and
//       either folds the reflect padding back (STFT backward) or divides by the
//       window envelope and trims (iSTFT forward).
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>

namespace mccl {
namespace kern {

constexpr int kStftMaxNfft = 4096;

struct FftFramesArgs {
  const float* signal;   // [batch, signal_len]
  int64_t signal_len;
  const float* window;   // [n_fft] (already padded to n_fft)
  float* out;            // [batch, n_frames, n_fft/2+1] interleaved complex
  int batch, n_frames, n_fft, hop;
  int pad;               // frame f starts at f*hop - pad in signal coordinates
  int reflect;           // 1: indices outside [0, signal_len) are reflected; 0: they read as zero
  int divide_envelope;   // 1: each sample is divided by the window-square envelope first (iSTFT backward)
  float scale;           // multiplied into every bin
  int hermitian_weights; // 1: bins 1..n_fft/2-1 are additionally doubled (iSTFT backward)
};

struct IfftFramesArgs {
  const float* spec;     // complex, addressed with the strides below (in complex elements)
  int64_t stride_b, stride_f, stride_t;
  const float* window;   // [n_fft]
  float* frames;         // [batch, n_frames, n_fft] real
  int batch, n_frames, n_fft;
  int hermitian;         // 1: inverse real FFT (mirror bins); 0: upper bins are zero (adjoint of forward)
  float scale;
};

struct OlaArgs {
  const float* frames;   // [batch, n_frames, n_fft]
  const float* window;   // [n_fft] (envelope mode)
  float* out;            // [batch, out_len]
  int batch, n_frames, n_fft, hop;
  int64_t out_len;
  int pad;               // output sample t corresponds to padded position t + pad
  int fold_reflect;      // 1: add the mirrored padded regions back (adjoint of reflect padding)
  int normalize_envelope;// 1: divide by sum of window^2 over the covering frames
};

cudaError_t launch_fft_frames(const FftFramesArgs& a, cudaStream_t s);
cudaError_t launch_ifft_frames(const IfftFramesArgs& a, cudaStream_t s);
cudaError_t launch_ola_gather(const OlaArgs& a, cudaStream_t s);

}  // namespace kern
}  // namespace mccl
