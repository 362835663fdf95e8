"""Synthetic datasets and run statistics shared by the examples and benchmarks."""
from __future__ import annotations

import json
from typing import List

import torch


class SyntheticDataset:
    """Gaussian clusters: class c is N(mu_c, I) with fixed random means (learnable to ~0 loss).

    Deterministic per (seed, rank); yields batches forever (reference
    examples/ddp_utils.py:11-36 uses the same kind of data).
    """

    def __init__(self, input_dim: int, num_classes: int, seed: int = 0, rank: int = 0, spread: float = 3.0):
        g = torch.Generator().manual_seed(seed)
        self.means = torch.randn(num_classes, input_dim, generator=g) * spread
        self.gen = torch.Generator().manual_seed(seed * 1000 + 17 + rank)
        self.num_classes = num_classes

    def batch(self, n: int, device=None, pin: bool = False):
        y = torch.randint(0, self.num_classes, (n,), generator=self.gen)
        x = self.means[y] + torch.randn(n, self.means.shape[1], generator=self.gen)
        if pin and torch.cuda.is_available():
            x, y = x.pin_memory(), y.pin_memory()
        if device is not None:
            x, y = x.to(device, non_blocking=True), y.to(device, non_blocking=True)
        return x, y


def write_training_stats(path: str, mode: str, step_times: List[float], losses: List[float], batch_size: int,
                         world_size: int, total_params: int) -> dict:
    """Writes the run summary consumed by ``examples/benchmark_throughput.py`` (same keys as the reference)."""
    avg = sum(step_times) / len(step_times) if step_times else 0.0
    payload = {
        "mode": mode,
        "step_times": step_times,
        "losses": losses,
        "avg_step_time_s": avg,
        "throughput_samples_per_sec": (batch_size * world_size) / avg if avg > 0 else 0.0,
        "batch_size_per_rank": batch_size,
        "world_size": world_size,
        "global_batch_size": batch_size * world_size,
        "total_params": total_params,
    }
    with open(path, "w", encoding="utf-8") as f:
        json.dump(payload, f, indent=2)
    return payload
