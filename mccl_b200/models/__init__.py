"""Model zoo of the benchmarks: the architectures named by the benchmark configs."""
from .mlp import MLP94M, TinyMLP, num_parameters
from .resnet import ResNet50
from .gpt2 import GPT2, gpt2_medium, gpt2_tiny
from .heavy import HeavyDummyModel

__all__ = ["MLP94M", "TinyMLP", "ResNet50", "GPT2", "gpt2_medium", "gpt2_tiny", "HeavyDummyModel", "num_parameters"]
