"""Utilities: multi-process test harness, synthetic data, run statistics."""
from .data import SyntheticDataset, write_training_stats
from .spawn import run_workers, next_port

__all__ = ["SyntheticDataset", "write_training_stats", "run_workers", "next_port"]
