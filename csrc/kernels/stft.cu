// STFT / iSTFT kernels (sm_100a): block-per-frame shared-memory radix-2 FFT with
// the padding, windowing and scaling fused into the loads and stores, and an
// atomics-free gather overlap-add.  See stft_api.h for the decomposition.
// Replaces the reference's one-thread-per-frame Metal FFT (reference
// csrc/metal/shaders.metal:735-861) and its CPU-side padding and overlap-add
// (reference csrc/transforms/StftMetalKernels.mm:158-393).
#include <cuda_runtime.h>

#include "kernels/launch_count.h"
#include "kernels/stft_api.h"

namespace mccl {
namespace kern {

namespace {

__device__ __forceinline__ int bit_reverse(int x, int bits) { return __brev(static_cast<unsigned>(x)) >> (32 - bits); }

// In-place radix-2 FFT over `data` (n complex values, already in bit-reversed
// order).  `tw[k] = exp(-2*pi*i*k/n)`, k < n/2.  sign = -1 forward, +1 inverse.
__device__ __forceinline__ void fft_smem(float2* data, const float2* tw, int n, int log2n, float sign) {
  for (int s = 1; s <= log2n; ++s) {
    const int half = 1 << (s - 1);
    const int tstep = n >> s;
    for (int j = threadIdx.x; j < n / 2; j += blockDim.x) {
      const int pos = j & (half - 1);
      const int i0 = ((j >> (s - 1)) << s) + pos;
      const int i1 = i0 + half;
      float2 w = tw[pos * tstep];
      w.y *= -sign;  // table holds the forward twiddle (negative angle)
      const float2 a = data[i0], b = data[i1];
      const float2 t = make_float2(b.x * w.x - b.y * w.y, b.x * w.y + b.y * w.x);
      data[i0] = make_float2(a.x + t.x, a.y + t.y);
      data[i1] = make_float2(a.x - t.x, a.y - t.y);
    }
    __syncthreads();
  }
}

__device__ __forceinline__ void fill_twiddles(float2* tw, int n) {
  for (int k = threadIdx.x; k < n / 2; k += blockDim.x) {
    float sn, cs;
    sincospif(2.0f * static_cast<float>(k) / static_cast<float>(n), &sn, &cs);
    tw[k] = make_float2(cs, -sn);
  }
}

__device__ __forceinline__ int64_t reflect_index(int64_t i, int64_t len) {
  // reflect without repeating the edge sample: -1 -> 1, len -> len-2
  if (len == 1) return 0;
  const int64_t period = 2 * (len - 1);
  i %= period;
  if (i < 0) i += period;
  return i < len ? i : period - i;
}

// sum of window^2 over the frames covering padded position p
__device__ __forceinline__ float envelope_at(const float* window, int64_t p, int n_fft, int hop, int n_frames) {
  int64_t f_hi = p / hop;
  if (f_hi > n_frames - 1) f_hi = n_frames - 1;
  int64_t f_lo = (p - n_fft + hop) / hop;  // ceil((p - n_fft + 1) / hop) for non-negative values
  if (p - n_fft + 1 <= 0) f_lo = 0;
  float e = 0.f;
  for (int64_t f = f_lo; f <= f_hi; ++f) {
    const int64_t n = p - f * hop;
    if (n >= 0 && n < n_fft) {
      const float w = window[n];
      e += w * w;
    }
  }
  return e;
}

__global__ void __launch_bounds__(512) fft_frames_kernel(const FftFramesArgs a, int log2n) {
  extern __shared__ float2 smem[];
  float2* data = smem;
  float2* tw = smem + a.n_fft;
  const int frame = blockIdx.x, b = blockIdx.y;
  const int n = a.n_fft;
  fill_twiddles(tw, n);
  const float* sig = a.signal + static_cast<int64_t>(b) * a.signal_len;
  const int64_t start = static_cast<int64_t>(frame) * a.hop - a.pad;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    int64_t t = start + i;
    float v = 0.f;
    if (a.reflect) {
      v = sig[reflect_index(t, a.signal_len)];
    } else if (t >= 0 && t < a.signal_len) {
      v = sig[t];
      if (a.divide_envelope) {
        const float e = envelope_at(a.window, t + a.pad, n, a.hop, a.n_frames);
        v = e > 1e-11f ? v / e : 0.f;
      }
    }
    data[bit_reverse(i, log2n)] = make_float2(v * a.window[i], 0.f);
  }
  __syncthreads();
  fft_smem(data, tw, n, log2n, -1.0f);
  const int bins = n / 2 + 1;
  float2* out = reinterpret_cast<float2*>(a.out) + (static_cast<int64_t>(b) * a.n_frames + frame) * bins;
  for (int k = threadIdx.x; k < bins; k += blockDim.x) {
    float s = a.scale;
    if (a.hermitian_weights && k != 0 && k != n / 2) s *= 2.0f;
    float2 v = data[k];
    if (a.hermitian_weights && (k == 0 || k == n / 2)) v.y = 0.f;  // imaginary parts of DC/Nyquist are ignored by an inverse real FFT
    out[k] = make_float2(v.x * s, v.y * s);
  }
}

__global__ void __launch_bounds__(512) ifft_frames_kernel(const IfftFramesArgs a, int log2n) {
  extern __shared__ float2 smem[];
  float2* data = smem;
  float2* tw = smem + a.n_fft;
  const int frame = blockIdx.x, b = blockIdx.y;
  const int n = a.n_fft;
  fill_twiddles(tw, n);
  const float2* spec = reinterpret_cast<const float2*>(a.spec) + b * a.stride_b + frame * a.stride_t;
  for (int k = threadIdx.x; k < n; k += blockDim.x) {
    float2 v = make_float2(0.f, 0.f);
    if (k <= n / 2) {
      v = spec[k * a.stride_f];
      if (a.hermitian && (k == 0 || k == n / 2)) v.y = 0.f;
    } else if (a.hermitian) {
      const float2 m = spec[(n - k) * a.stride_f];
      v = make_float2(m.x, -m.y);
    }
    data[bit_reverse(k, log2n)] = v;
  }
  __syncthreads();
  fft_smem(data, tw, n, log2n, +1.0f);
  float* out = a.frames + (static_cast<int64_t>(b) * a.n_frames + frame) * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) out[i] = data[i].x * a.scale * a.window[i];
}

__device__ __forceinline__ float ola_at(const float* frames, int64_t p, int n_fft, int hop, int n_frames) {
  if (p < 0) return 0.f;
  int64_t f_hi = p / hop;
  if (f_hi > n_frames - 1) f_hi = n_frames - 1;
  int64_t f_lo = p - n_fft + 1 <= 0 ? 0 : (p - n_fft + hop) / hop;
  float acc = 0.f;
  for (int64_t f = f_lo; f <= f_hi; ++f) {
    const int64_t n = p - f * hop;
    if (n >= 0 && n < n_fft) acc += frames[f * n_fft + n];
  }
  return acc;
}

__global__ void __launch_bounds__(256) ola_gather_kernel(const OlaArgs a) {
  const int b = blockIdx.y;
  const float* frames = a.frames + static_cast<int64_t>(b) * a.n_frames * a.n_fft;
  float* out = a.out + static_cast<int64_t>(b) * a.out_len;
  const int64_t T = a.out_len;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < T; t += stride) {
    const int64_t p = t + a.pad;
    float v = ola_at(frames, p, a.n_fft, a.hop, a.n_frames);
    if (a.fold_reflect && a.pad > 0) {
      // adjoint of reflect padding: padded[pad - i] and padded[pad + 2T - 2 - i] also came from x[i]
      if (t >= 1 && t <= a.pad) v += ola_at(frames, a.pad - t, a.n_fft, a.hop, a.n_frames);
      if (t <= T - 2 && t >= T - 1 - a.pad) v += ola_at(frames, a.pad + 2 * T - 2 - t, a.n_fft, a.hop, a.n_frames);
    }
    if (a.normalize_envelope) {
      const float e = envelope_at(a.window, p, a.n_fft, a.hop, a.n_frames);
      v = e > 1e-11f ? v / e : 0.f;
    }
    out[t] = v;
  }
}

int ilog2(int n) {
  int l = 0;
  while ((1 << l) < n) ++l;
  return l;
}

bool valid_nfft(int n) { return n >= 8 && n <= kStftMaxNfft && (n & (n - 1)) == 0; }

}  // namespace

cudaError_t launch_fft_frames(const FftFramesArgs& a, cudaStream_t s) {
  if (!valid_nfft(a.n_fft) || a.batch <= 0 || a.n_frames <= 0) return cudaErrorInvalidValue;
  note_launch();
  const int threads = a.n_fft / 2 < 512 ? (a.n_fft / 2 < 32 ? 32 : a.n_fft / 2) : 512;
  const size_t smem = static_cast<size_t>(a.n_fft) * 8 + static_cast<size_t>(a.n_fft) * 4;
  fft_frames_kernel<<<dim3(a.n_frames, a.batch), threads, smem, s>>>(a, ilog2(a.n_fft));
  return cudaGetLastError();
}

cudaError_t launch_ifft_frames(const IfftFramesArgs& a, cudaStream_t s) {
  if (!valid_nfft(a.n_fft) || a.batch <= 0 || a.n_frames <= 0) return cudaErrorInvalidValue;
  note_launch();
  const int threads = a.n_fft / 2 < 512 ? (a.n_fft / 2 < 32 ? 32 : a.n_fft / 2) : 512;
  const size_t smem = static_cast<size_t>(a.n_fft) * 8 + static_cast<size_t>(a.n_fft) * 4;
  ifft_frames_kernel<<<dim3(a.n_frames, a.batch), threads, smem, s>>>(a, ilog2(a.n_fft));
  return cudaGetLastError();
}

cudaError_t launch_ola_gather(const OlaArgs& a, cudaStream_t s) {
  if (a.batch <= 0 || a.out_len <= 0) return cudaErrorInvalidValue;
  note_launch();
  int64_t blocks = (a.out_len + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  ola_gather_kernel<<<dim3(static_cast<unsigned>(blocks), a.batch), 256, 0, s>>>(a);
  return cudaGetLastError();
}

}  // namespace kern
}  // namespace mccl
