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


class DevicePrefetcher:
    """Feeds a training loop from pinned host batches with the copy of batch i+1 behind step i.

    ``batches`` is any iterable of tuples of pinned CPU tensors.  ``next()`` returns the device copy
    of the next batch (the compute stream is made to wait for the copy) and at once enqueues the
    host->device copy of the batch after it on a side stream, so that copy overlaps the step that
    is about to be launched.  The reference's examples copy each batch synchronously at the top of
    the step (reference examples/ddp_dummy_train.py:196-204).
    """

    def __init__(self, batches, device):
        self._it = iter(batches)
        self._dev = torch.device(device)
        self._stream = torch.cuda.Stream(self._dev)
        self._ready = None  # (tensors, event) of the batch whose copy is in flight
        self._enqueue()

    def _enqueue(self):
        try:
            host = next(self._it)
        except StopIteration:
            self._ready = None
            return
        with torch.cuda.stream(self._stream):
            tensors = tuple(t.to(self._dev, non_blocking=True) for t in host)
            ev = torch.cuda.Event()
            ev.record(self._stream)
        self._ready = (tensors, ev)

    def next(self):
        if self._ready is None:
            raise StopIteration
        tensors, ev = self._ready
        cur = torch.cuda.current_stream(self._dev)
        cur.wait_event(ev)
        for t in tensors:
            t.record_stream(cur)
        self._enqueue()
        return tensors

    __next__ = next

    def __iter__(self):
        return self


class AsyncScalarReader:
    """Reads a per-step device scalar (the loss) on the host without stalling the launch of the next step.

    ``push(t)`` enqueues a device->host copy of ``t`` into a pinned slot and records an event;
    ``pop()`` waits for the OLDEST outstanding copy and returns its value as a float.  A loop that
    pushes step i's loss and pops step i-1's reads every step's loss while keeping one step of
    launches ahead of the GPU; ``drain()`` returns what is still outstanding.
    """

    def __init__(self, device, depth: int = 4):
        self._dev = torch.device(device)
        self._slots = [torch.empty(1, dtype=torch.float32).pin_memory() for _ in range(depth)]
        self._events = [torch.cuda.Event() for _ in range(depth)]
        self._head = 0   # next slot to fill
        self._count = 0  # outstanding copies

    def push(self, t: torch.Tensor) -> None:
        if self._count == len(self._slots):
            raise RuntimeError("AsyncScalarReader: pop() before pushing more than `depth` values")
        i = self._head
        self._slots[i].copy_(t.detach().reshape(1).to(torch.float32), non_blocking=True)
        self._events[i].record(torch.cuda.current_stream(self._dev))
        self._head = (i + 1) % len(self._slots)
        self._count += 1

    def pop(self) -> float:
        if self._count == 0:
            raise RuntimeError("AsyncScalarReader: nothing outstanding")
        i = (self._head - self._count) % len(self._slots)
        self._events[i].synchronize()
        self._count -= 1
        return float(self._slots[i][0])

    def __len__(self):
        return self._count

    def drain(self):
        return [self.pop() for _ in range(self._count)]
