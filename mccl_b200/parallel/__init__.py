"""Data-parallel integration: DDP communication hooks and helpers."""
from .ddp import (fused_avg_hook, topk_hook, TopKState, wrap_ddp, optimizer_in_backward_hook,
                  OptimizerInBackward, nvls_tensor_pool)

__all__ = ["fused_avg_hook", "topk_hook", "TopKState", "wrap_ddp", "optimizer_in_backward_hook",
           "OptimizerInBackward", "nvls_tensor_pool"]
