"""DSP transforms shipped with the backend: STFT / iSTFT with CPU-reference parity."""
from __future__ import annotations

import os

from .stft import istft, resolve_backend, stft

__all__ = ["stft", "istft", "resolve_backend", "is_available", "default_backend"]


def is_available() -> bool:
    """True when the native extension with the STFT kernels is loaded."""
    try:
        from .. import _C
        return _C is not None and hasattr(_C, "_stft_forward")
    except Exception:
        return False


def default_backend() -> str:
    return resolve_backend(os.environ.get("MCCL_STFT_BACKEND", "auto"))
