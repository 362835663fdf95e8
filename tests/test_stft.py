"""STFT / iSTFT kernels vs torch.stft / torch.istft on the CPU (the oracle).

Mirrors the reference's tests/test_stft_vdsp.py:22-124: forward parity < 1e-4, gradient
agreement, finite inverse, and a wall-clock guard for forward+backward.
"""
import time

import pytest
import torch

from mccl_b200.transforms import istft, resolve_backend, stft


def test_backend_names():
    assert resolve_backend("metal") == "cuda" and resolve_backend("vdsp") == "cpu" and resolve_backend("auto") == "auto"
    with pytest.raises(ValueError):
        resolve_backend("fftw")


def test_cpu_backend_matches_torch():
    x = torch.randn(2, 4000)
    w = torch.hann_window(512)
    got = stft(x, n_fft=512, hop_length=128, win_length=512, window=w, backend="vdsp")
    ref = torch.stft(x, 512, hop_length=128, win_length=512, window=w, center=True, return_complex=True)
    assert torch.allclose(got, ref)


def _cos(a, b):
    a, b = a.flatten().double(), b.flatten().double()
    return float((a @ b) / (a.norm() * b.norm() + 1e-30))


@pytest.mark.gpu
@pytest.mark.parametrize("n_fft,hop,win", [(2048, 512, 2048), (1024, 256, 1024), (512, 128, 400), (64, 16, 64)])
@pytest.mark.parametrize("center", [True, False])
@pytest.mark.parametrize("normalized", [False, True])
def test_stft_forward_and_backward_match_torch(cuda_device, n_fft, hop, win, center, normalized):
    torch.manual_seed(0)
    x = torch.randn(2, 48000 if n_fft > 64 else 1000)
    w = torch.hann_window(win, periodic=True)
    kw = dict(n_fft=n_fft, hop_length=hop, win_length=win)
    xr = x.clone().requires_grad_(True)
    ref = torch.stft(xr, window=w, center=center, normalized=normalized, return_complex=True, **kw)
    xg = x.to(cuda_device).requires_grad_(True)
    got = stft(xg, window=w.to(cuda_device), center=center, normalized=normalized, backend="cuda", **kw)
    assert got.shape == ref.shape
    assert float((ref - got.detach().cpu()).abs().max()) < 1e-4 * max(1.0, float(ref.abs().max()) / 30)
    # gradient of a generic real loss
    gr = torch.randn(ref.shape, dtype=torch.complex64)
    (ref * gr.conj()).real.sum().backward()
    (got * gr.to(cuda_device).conj()).real.sum().backward()
    assert _cos(xg.grad.cpu(), xr.grad) > 0.9999
    assert torch.allclose(xg.grad.cpu(), xr.grad, rtol=1e-3, atol=1e-3 * float(xr.grad.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("n_fft,hop", [(1024, 256), (512, 128), (2048, 512)])
@pytest.mark.parametrize("normalized", [False, True])
def test_istft_forward_and_backward_match_torch(cuda_device, n_fft, hop, normalized):
    torch.manual_seed(1)
    length = 24000
    w = torch.hann_window(n_fft, periodic=True)
    x = torch.randn(2, length)
    spec = torch.stft(x, n_fft, hop_length=hop, win_length=n_fft, window=w, center=True, normalized=normalized,
                      return_complex=True)
    spec = spec + 0.1 * torch.randn_like(spec)  # not exactly consistent: exercises the general case
    sr = spec.clone().requires_grad_(True)
    ref = torch.istft(sr, n_fft, hop_length=hop, win_length=n_fft, window=w, center=True, normalized=normalized,
                      length=length)
    sg = spec.to(cuda_device).requires_grad_(True)
    got = istft(sg, n_fft=n_fft, hop_length=hop, win_length=n_fft, window=w.to(cuda_device), length=length,
                normalized=normalized, backend="cuda")
    assert torch.isfinite(got).all()
    assert float((ref - got.detach().cpu()).abs().max()) < 1e-4
    gy = torch.randn(ref.shape)
    (ref * gy).sum().backward()
    (got * gy.to(cuda_device)).sum().backward()
    # compare only what an inverse real FFT can see (imaginary DC/Nyquist parts have no gradient)
    assert _cos(sg.grad.cpu().real, sr.grad.real) > 0.9999
    a, b = torch.view_as_real(sg.grad.cpu()), torch.view_as_real(sr.grad)
    assert torch.allclose(a, b, rtol=1e-3, atol=1e-3 * float(b.abs().max()))


@pytest.mark.gpu
def test_roundtrip_and_perf_guard(cuda_device):
    w = torch.hann_window(2048, device=cuda_device)
    x = torch.randn(2, 48000, device=cuda_device, requires_grad=True)
    kw = dict(n_fft=2048, hop_length=512, win_length=2048, window=w)
    for _ in range(2):  # warm-up
        stft(x, **kw).abs().sum().backward()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    s = stft(x, **kw)
    y = istft(s, length=48000, **kw)
    (y.square().sum() + s.abs().sum()).backward()
    torch.cuda.synchronize()
    assert (time.perf_counter() - t0) * 1e3 < 1000  # the reference's guard: fwd+bwd under one second
    assert float((y.detach() - x.detach()).abs().max()) < 1e-3  # hann/4-overlap satisfies the NOLA condition


@pytest.mark.gpu
def test_rejects_unsupported_sizes(cuda_device):
    x = torch.randn(1, 5000, device=cuda_device)
    with pytest.raises(ValueError):
        stft(x, n_fft=1000, hop_length=250, win_length=1000, window=torch.hann_window(1000, device=cuda_device),
             backend="cuda")
    # "auto" falls back to ATen for sizes the kernels do not cover
    out = stft(x, n_fft=1000, hop_length=250, win_length=1000, window=torch.hann_window(1000, device=cuda_device))
    assert out.shape[1] == 501
