"""Parameter-layout helper (reference ``mccl/params.py:9-36``).

Collectives reject non-contiguous tensors, and DDP's flat buckets copy less
when every parameter is dense; this re-lays-out ``param.data`` in place.  It
never changes values or names, so ``state_dict()`` keys and checkpoints are
unaffected.
"""
from __future__ import annotations

import warnings
from typing import List

import torch.nn as nn


def ensure_contiguous_parameters(module: nn.Module, *, warn: bool = True) -> List[str]:
    """Make every parameter's storage contiguous; returns the names that changed.

    Call once after building the model and before wrapping it in
    ``DistributedDataParallel`` / creating the optimizer.
    """
    changed: List[str] = []
    for name, p in module.named_parameters():
        if p.data.is_contiguous():
            continue
        if warn:
            warnings.warn(f"parameter {name!r} is not contiguous; re-laying it out", RuntimeWarning, stacklevel=2)
        p.data = p.data.contiguous()
        changed.append(name)
    return changed


__all__ = ["ensure_contiguous_parameters"]
