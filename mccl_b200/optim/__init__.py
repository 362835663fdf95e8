"""Optimizers whose step is one fused sm_100a kernel."""
from .fused_adamw import FusedAdamW

__all__ = ["FusedAdamW"]
