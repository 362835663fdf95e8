"""Model zoo of the benchmarks: the architectures named by the benchmark configs."""
from .mlp import MLP94M, TinyMLP, num_parameters

__all__ = ["MLP94M", "TinyMLP", "num_parameters"]
