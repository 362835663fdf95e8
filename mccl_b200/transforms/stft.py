"""STFT / iSTFT as differentiable ops backed by the sm_100a FFT kernels.

Same call signatures as the reference (``mccl/transforms/stft.py:138-185``):
``stft(waveform, *, n_fft, hop_length, win_length, window, center, normalized, backend)``
returns a complex ``[batch, freq, frames]`` spectrum, ``istft(spec, ..., length)`` a waveform.
Backends: ``"cuda"`` (native kernels; power-of-two ``n_fft`` up to 4096), ``"cpu"`` (ATen on
the host) and ``"auto"`` (native kernels for CUDA tensors when supported, ATen otherwise).
The reference's names ``"metal"`` and ``"vdsp"`` are accepted as aliases of ``"cuda"`` and
``"cpu"``; ``MCCL_STFT_BACKEND`` sets the default.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

_ALIASES = {"metal": "cuda", "vdsp": "cpu"}
_BACKENDS = frozenset({"cuda", "cpu", "auto"})


def resolve_backend(name: Optional[str]) -> str:
    raw = (name or os.environ.get("MCCL_STFT_BACKEND", "auto")).strip().lower()
    raw = _ALIASES.get(raw, raw)
    if raw not in _BACKENDS:
        raise ValueError(f"STFT backend must be one of {sorted(_BACKENDS | set(_ALIASES))}, got {name!r}")
    return raw


def _native_ok(t: torch.Tensor, n_fft: int) -> bool:
    return t.is_cuda and 8 <= n_fft <= 4096 and (n_fft & (n_fft - 1)) == 0


def _use_native(t: torch.Tensor, n_fft: int, backend: str) -> bool:
    b = resolve_backend(backend)
    if b == "cpu":
        return False
    if b == "cuda":
        if not _native_ok(t, n_fft):
            raise ValueError("backend='cuda' needs a CUDA tensor and a power-of-two n_fft in [8, 4096]")
        return True
    return _native_ok(t, n_fft)


class _StftFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, waveform, window, n_fft, hop_length, win_length, center, normalized):
        from .. import require_native
        native = require_native()
        ctx.in_shape = tuple(waveform.shape)
        x = waveform.squeeze(1) if waveform.dim() == 3 and waveform.size(1) == 1 else waveform
        x = x.contiguous().float()
        ctx.save_for_backward(window)
        ctx.cfg = (int(n_fft), int(hop_length), int(win_length), bool(center), bool(normalized), int(x.shape[-1]))
        return native._stft_forward(x, window, int(n_fft), int(hop_length), int(win_length), bool(center),
                                    bool(normalized), "cuda")

    @staticmethod
    def backward(ctx, grad_spec):
        from .. import require_native
        (window,) = ctx.saved_tensors
        n_fft, hop, win, center, normalized, length = ctx.cfg
        g = require_native()._stft_backward(grad_spec, window, n_fft, hop, win, center, normalized, length, "cuda")
        return g.reshape(ctx.in_shape), None, None, None, None, None, None


class _IstftFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, spec, window, n_fft, hop_length, win_length, length, center, normalized):
        from .. import require_native
        ctx.save_for_backward(window)
        ctx.cfg = (int(n_fft), int(hop_length), int(win_length), bool(center), bool(normalized), int(spec.shape[-1]))
        return require_native()._istft_forward(spec, window, int(n_fft), int(hop_length), int(win_length),
                                               bool(center), bool(normalized), int(length), "cuda")

    @staticmethod
    def backward(ctx, grad_waveform):
        from .. import require_native
        (window,) = ctx.saved_tensors
        n_fft, hop, win, center, normalized, frames = ctx.cfg
        g = require_native()._istft_backward(grad_waveform.contiguous(), window, n_fft, hop, win, center,
                                             normalized, frames, "cuda")
        return g, None, None, None, None, None, None, None


def stft(waveform: torch.Tensor, *, n_fft: int, hop_length: int, win_length: int, window: torch.Tensor,
         center: bool = True, normalized: bool = False, backend: str = "auto") -> torch.Tensor:
    """Complex one-sided STFT ``[batch, n_fft/2+1, frames]`` (torch.stft semantics, reflect padding)."""
    if _use_native(waveform, n_fft, backend):
        return _StftFn.apply(waveform, window, n_fft, hop_length, win_length, center, normalized)
    x = waveform.squeeze(1) if waveform.dim() == 3 and waveform.size(1) == 1 else waveform
    dev = x.device
    if resolve_backend(backend) == "cpu":
        x = x.cpu()
    out = torch.stft(x, n_fft, hop_length=hop_length, win_length=win_length, window=window.to(x.device),
                     center=center, pad_mode="reflect", normalized=normalized, onesided=True, return_complex=True)
    return out.to(dev)


def istft(spec: torch.Tensor, *, n_fft: int, hop_length: int, win_length: int, window: torch.Tensor, length: int,
          center: bool = True, normalized: bool = False, backend: str = "auto") -> torch.Tensor:
    """Inverse STFT returning ``[batch, length]`` (torch.istft semantics)."""
    if _use_native(spec, n_fft, backend):
        return _IstftFn.apply(spec, window, n_fft, hop_length, win_length, length, center, normalized)
    dev = spec.device
    s = spec.cpu() if resolve_backend(backend) == "cpu" else spec
    out = torch.istft(s, n_fft, hop_length=hop_length, win_length=win_length, window=window.to(s.device),
                      center=center, normalized=normalized, onesided=True, length=length)
    return out.to(dev)
