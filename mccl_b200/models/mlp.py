"""MLP models used by the DDP throughput benchmarks and tests."""
from __future__ import annotations

import torch
import torch.nn as nn


class MLP94M(nn.Module):
    """The ~94 M parameter fp32 MLP of the headline DDP benchmark.

    ``Linear(2048,3072)-GELU``, nine ``Linear(3072,3072)-GELU`` blocks and
    ``Linear(3072,1000)``: 94.3 M parameters, 377 MB of fp32 gradients per step
    (the stand-in for the reference's ~96.5 M parameter dummy model,
    reference examples/ddp_utils.py:105-147).
    """

    def __init__(self, in_features: int = 2048, hidden: int = 3072, depth: int = 9, classes: int = 1000):
        super().__init__()
        layers = [nn.Linear(in_features, hidden), nn.GELU()]
        for _ in range(depth):
            layers += [nn.Linear(hidden, hidden), nn.GELU()]
        layers.append(nn.Linear(hidden, classes))
        self.net = nn.Sequential(*layers)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.net(x)


class TinyMLP(nn.Module):
    """``Linear(512,256)-ReLU-Linear(256,10)``: the CPU plumbing / smoke model."""

    def __init__(self):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(512, 256), nn.ReLU(), nn.Linear(256, 10))

    def forward(self, x):
        return self.net(x)


def num_parameters(m: nn.Module) -> int:
    return sum(p.numel() for p in m.parameters())
