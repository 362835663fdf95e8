"""Utilities: multi-process test harness, synthetic data, input prefetch / deferred loss read, run statistics."""
from .data import AsyncScalarReader, DevicePrefetcher, SyntheticDataset, write_training_stats
from .spawn import run_workers, next_port

__all__ = ["AsyncScalarReader", "DevicePrefetcher", "SyntheticDataset", "write_training_stats", "run_workers",
           "next_port"]
