// STFT / iSTFT kernels (sm_100a): shared-memory radix-4 Stockham FFTs of half the frame length
// (real input / real output), several frames per CTA, twiddles computed once per CTA, with
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

// Both transforms work on REAL frames, so each frame is handled as a complex FFT of half the
// length: z[m] = x[2m] + i x[2m+1], Z = FFT_{N/2}(z), and one pass with the twiddles W_N^k
// separates / recombines the even and odd halves.  That halves the butterflies and the shared
// memory per frame.  A CTA computes the twiddle table once and then loops over frames, `fpc`
// frames at a time (several short frames keep all threads busy).
//
//   forward:  E[k] = (Z[k] + conj Z[h-k]) / 2,  O[k] = (Z[k] - conj Z[h-k]) / (2i),
//             X[k] = E[k] + W_N^k O[k],  k = 0..h  (h = N/2, Z[h] = Z[0])
//   inverse:  Z[k] = (X[k] + conj X[h-k]) + i W_N^{-k} (X[k] - conj X[h-k]),  z = IFFT_h(Z) (no 1/h),
//             y[2m] = Re z[m], y[2m+1] = Im z[m]   (y = unnormalised inverse of the Hermitian extension)

// Stockham autosort FFT over `fpc` independent transforms of length h stored back to back
// (natural order in, natural order out: no bit-reversal pass, whose shared-memory scatter would put
// a whole warp on one bank).  Radix-4 passes (four values per thread in registers; an odd log2(h)
// starts with one radix-2 pass) ping-pong between `a` and `b`; every pass reads at stride h/4 and
// writes runs of Ns consecutive values.  tw[t] = exp(-2*pi*i*t/(2h)), t < h; tw[t + h] = -tw[t].
// Returns the buffer that holds the result.
__device__ __forceinline__ float2 cmul_tw(float2 v, float2 w, float conj_sign) {
  // v * (w.x + i * conj_sign * w.y): conj_sign = +1 keeps the table's forward twiddle, -1 conjugates it
  const float wy = conj_sign * w.y;
  return make_float2(v.x * w.x - v.y * wy, v.x * wy + v.y * w.x);
}

__device__ __forceinline__ float2* fft_half_smem(float2* a, float2* b, const float2* tw, int h, int log2h, int fpc,
                                                 float sign) {
  const float cs = -sign;  // sign = -1: forward (table as stored); +1: inverse (conjugated)
  float2* src = a;
  float2* dst = b;
  int ns = 1;
  if (log2h & 1) {
    const int per = h / 2;
    for (int jj = threadIdx.x; jj < per * fpc; jj += blockDim.x) {
      const int f = jj >> (log2h - 1), j = jj & (per - 1);
      const float2 v0 = src[f * h + j], v1 = src[f * h + j + per];
      float2* d = dst + f * h + 2 * j;
      d[0] = make_float2(v0.x + v1.x, v0.y + v1.y);
      d[1] = make_float2(v0.x - v1.x, v0.y - v1.y);
    }
    __syncthreads();
    float2* t = src; src = dst; dst = t;
    ns = 2;
  }
  const int quarter = h / 4;
  for (; ns < h; ns *= 4) {
    const int tstep = h / (2 * ns);  // exp(-2*pi*i*r*k/(4*ns)) = tw[r * k * tstep]
    for (int jj = threadIdx.x; jj < quarter * fpc; jj += blockDim.x) {
      const int f = jj >> (log2h - 2), j = jj & (quarter - 1);
      const int k = j & (ns - 1);
      const int t1 = k * tstep, t3 = 3 * t1;
      const float2* x = src + f * h + j;
      float2 w3 = tw[t3 < h ? t3 : t3 - h];
      if (t3 >= h) w3 = make_float2(-w3.x, -w3.y);
      const float2 v0 = x[0];
      const float2 v1 = cmul_tw(x[quarter], tw[t1], cs);
      const float2 v2 = cmul_tw(x[2 * quarter], tw[2 * t1], cs);
      const float2 v3 = cmul_tw(x[3 * quarter], w3, cs);
      const float2 a0 = make_float2(v0.x + v2.x, v0.y + v2.y), a1 = make_float2(v0.x - v2.x, v0.y - v2.y);
      const float2 a2 = make_float2(v1.x + v3.x, v1.y + v3.y), a3 = make_float2(v1.x - v3.x, v1.y - v3.y);
      const float2 r3 = make_float2(cs * a3.y, -cs * a3.x);  // -i * a3 forward, +i * a3 inverse
      float2* d = dst + f * h + ((j - k) << 2) + k;
      d[0] = make_float2(a0.x + a2.x, a0.y + a2.y);
      d[ns] = make_float2(a1.x + r3.x, a1.y + r3.y);
      d[2 * ns] = make_float2(a0.x - a2.x, a0.y - a2.y);
      d[3 * ns] = make_float2(a1.x - r3.x, a1.y - r3.y);
    }
    __syncthreads();
    float2* t = src; src = dst; dst = t;
  }
  return src;
}

__device__ __forceinline__ float load_sample(const FftFramesArgs& a, const float* sig, int64_t t, int n) {
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
  return v;
}

__global__ void __launch_bounds__(256) fft_frames_kernel(const FftFramesArgs a, int log2h, int fpc) {
  extern __shared__ float2 smem[];
  const int n = a.n_fft, h = n / 2;
  float2* tw = smem;        // h twiddles W_N^k
  float2* data = smem + h;  // fpc * h values, and as many again for the ping-pong passes
  float2* pong = data + fpc * h;
  const int b = blockIdx.y;
  fill_twiddles(tw, n);
  const float* sig = a.signal + static_cast<int64_t>(b) * a.signal_len;
  const int bins = h + 1;
  for (int f0 = blockIdx.x * fpc; f0 < a.n_frames; f0 += gridDim.x * fpc) {
    __syncthreads();  // twiddles ready / previous frames' bins written
    for (int jj = threadIdx.x; jj < h * fpc; jj += blockDim.x) {
      const int f = jj >> log2h, m = jj & (h - 1);
      const int frame = f0 + f;
      float v0 = 0.f, v1 = 0.f;
      if (frame < a.n_frames) {
        const int64_t start = static_cast<int64_t>(frame) * a.hop - a.pad;
        const int64_t t0 = start + 2 * m;
        if (a.reflect && start >= 0 && start + n <= a.signal_len) {  // frame inside the signal: no index folding
          v0 = sig[t0];
          v1 = sig[t0 + 1];
        } else {
          v0 = load_sample(a, sig, t0, n);
          v1 = load_sample(a, sig, t0 + 1, n);
        }
        v0 *= a.window[2 * m];
        v1 *= a.window[2 * m + 1];
      }
      data[jj] = make_float2(v0, v1);
    }
    __syncthreads();
    const float2* res = fft_half_smem(data, pong, tw, h, log2h, fpc, -1.0f);
    for (int jj = threadIdx.x; jj < h * fpc; jj += blockDim.x) {
      const int f = jj >> log2h, k = jj & (h - 1);
      const int frame = f0 + f;
      if (frame >= a.n_frames) continue;
      const float2* d = res + f * h;
      const float2 zk = d[k];
      const float2 zm = d[(h - k) & (h - 1)];            // Z[h-k], with Z[h] = Z[0]
      const float2 e = make_float2(0.5f * (zk.x + zm.x), 0.5f * (zk.y - zm.y));
      const float2 o = make_float2(0.5f * (zk.y + zm.y), -0.5f * (zk.x - zm.x));   // (Zk - conj Zm) / (2i)
      const float2 w = tw[k];
      float2 v = make_float2(e.x + w.x * o.x - w.y * o.y, e.y + w.x * o.y + w.y * o.x);
      float sc = a.scale;
      if (a.hermitian_weights && k != 0) sc *= 2.0f;
      if (a.hermitian_weights && k == 0) v.y = 0.f;  // imaginary parts of DC/Nyquist are ignored by an inverse real FFT
      float2* out = reinterpret_cast<float2*>(a.out) + (static_cast<int64_t>(b) * a.n_frames + frame) * bins;
      out[k] = make_float2(v.x * sc, v.y * sc);
      if (k == 0) {  // Nyquist bin: X[h] = E[0] - O[0] (twiddle -1), from the same Z[0]
        float2 vn = make_float2(e.x - o.x, e.y - o.y);
        if (a.hermitian_weights) vn.y = 0.f;
        out[h] = make_float2(vn.x * a.scale, vn.y * a.scale);
      }
    }
  }
}

__global__ void __launch_bounds__(256) ifft_frames_kernel(const IfftFramesArgs a, int log2h, int fpc) {
  extern __shared__ float2 smem[];
  const int n = a.n_fft, h = n / 2;
  float2* tw = smem;
  float2* data = smem + h;
  float2* pong = data + fpc * h;
  const int b = blockIdx.y;
  fill_twiddles(tw, n);
  // hermitian: inverse real FFT of the one-sided bins.  Otherwise the adjoint of the forward
  // transform, Re(sum_{k<=h} X[k] e^{+2 pi i k n / N}), which equals half the inverse real FFT of the
  // same bins with the real parts of DC and Nyquist doubled.
  const float edge = a.hermitian ? 1.0f : 2.0f;
  const float post = a.hermitian ? a.scale : 0.5f * a.scale;
  for (int f0 = blockIdx.x * fpc; f0 < a.n_frames; f0 += gridDim.x * fpc) {
    __syncthreads();
    for (int jj = threadIdx.x; jj < h * fpc; jj += blockDim.x) {
      const int f = jj >> log2h, k = jj & (h - 1);
      const int frame = f0 + f;
      float2 z = make_float2(0.f, 0.f);
      if (frame < a.n_frames) {
        const float2* spec = reinterpret_cast<const float2*>(a.spec) + b * a.stride_b + frame * a.stride_t;
        float2 xk = spec[k * a.stride_f];
        float2 xm = spec[(h - k) * a.stride_f];
        if (k == 0) {  // pair (DC, Nyquist): imaginary parts do not take part
          xk = make_float2(edge * xk.x, 0.f);
          xm = make_float2(edge * xm.x, 0.f);
        }
        const float2 ep = make_float2(xk.x + xm.x, xk.y - xm.y);   // X[k] + conj X[h-k]
        const float2 dm = make_float2(xk.x - xm.x, xk.y + xm.y);   // X[k] - conj X[h-k]
        const float2 w = make_float2(tw[k].x, -tw[k].y);           // W_N^{-k}
        const float2 od = make_float2(dm.x * w.x - dm.y * w.y, dm.x * w.y + dm.y * w.x);
        z = make_float2(ep.x - od.y, ep.y + od.x);                 // E' + i O'
      }
      data[jj] = z;
    }
    __syncthreads();
    const float2* res = fft_half_smem(data, pong, tw, h, log2h, fpc, +1.0f);
    for (int jj = threadIdx.x; jj < h * fpc; jj += blockDim.x) {
      const int f = jj >> log2h, m = jj & (h - 1);
      const int frame = f0 + f;
      if (frame >= a.n_frames) continue;
      const float2 v = res[jj];
      float2* out = reinterpret_cast<float2*>(a.frames + (static_cast<int64_t>(b) * a.n_frames + frame) * n);
      out[m] = make_float2(v.x * post * a.window[2 * m], v.y * post * a.window[2 * m + 1]);
    }
  }
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

// Frames handled together by one CTA iteration and the grid: enough frames per iteration to give
// every thread butterflies, enough CTAs to fill the GPU a few times over, each looping over frames.
void frame_grid(int n_fft, int n_frames, int batch, int* fpc, int* grid_x, size_t* smem) {
  const int h = n_fft / 2;
  int f = 2048 / h;  // 256 threads, h/4 radix-4 groups per frame and pass: two groups per thread
  if (f < 1) f = 1;
  if (f > 8) f = 8;
  *fpc = f;
  int64_t want = (static_cast<int64_t>(n_frames) + f - 1) / f;
  int64_t cap = (148 * 8 + batch - 1) / batch;
  if (cap < 1) cap = 1;
  *grid_x = static_cast<int>(want < cap ? want : cap);
  *smem = (static_cast<size_t>(h) + 2 * static_cast<size_t>(f) * h) * sizeof(float2);  // <= 48 KB at n_fft 4096
}

}  // namespace

cudaError_t launch_fft_frames(const FftFramesArgs& a, cudaStream_t s) {
  if (!valid_nfft(a.n_fft) || a.batch <= 0 || a.n_frames <= 0) return cudaErrorInvalidValue;
  note_launch();
  int fpc, gx;
  size_t smem;
  frame_grid(a.n_fft, a.n_frames, a.batch, &fpc, &gx, &smem);
  fft_frames_kernel<<<dim3(gx, a.batch), 256, smem, s>>>(a, ilog2(a.n_fft / 2), fpc);
  return cudaGetLastError();
}

cudaError_t launch_ifft_frames(const IfftFramesArgs& a, cudaStream_t s) {
  if (!valid_nfft(a.n_fft) || a.batch <= 0 || a.n_frames <= 0) return cudaErrorInvalidValue;
  note_launch();
  int fpc, gx;
  size_t smem;
  frame_grid(a.n_fft, a.n_frames, a.batch, &fpc, &gx, &smem);
  ifft_frames_kernel<<<dim3(gx, a.batch), 256, smem, s>>>(a, ilog2(a.n_fft / 2), fpc);
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
