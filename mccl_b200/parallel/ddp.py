"""DistributedDataParallel integration.

Stock ``DistributedDataParallel`` works over the backend unchanged (it issues
one SUM allreduce per gradient bucket after dividing the bucket by the world
size in a separate elementwise pass).  The hooks here remove that extra pass:

* :func:`fused_avg_hook` -- the bucket is reduced by ONE kernel that also
  applies the 1/world scale (and, with ``MCCL_WIRE_DTYPE``, the fp32<->bf16
  wire cast) in its epilogue.
* :func:`topk_hook` -- fused top-k compressed allreduce with error feedback
  (select -> sparse exchange over NVLink -> deterministic scatter-add); the
  residual lives in a per-bucket fp32 buffer keyed by the bucket index.

Both return futures that are ordered on the communication stream, so no host
synchronisation happens between backward and the optimizer step.
"""
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel


def _backend_for(process_group, device):
    pg = process_group if process_group is not None else dist.distributed_c10d._get_default_group()
    return pg._get_backend(device)


def fused_avg_hook(process_group, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """DDP comm hook: ``bucket = sum_over_ranks(bucket) / world`` in one fused kernel."""
    buf = bucket.buffer()
    backend = _backend_for(process_group, buf.device)
    world = backend.size()
    work = backend.allreduce_scaled(buf, 1.0 / world)
    return work.get_future().then(lambda f: f.value()[0])


class TopKState:
    """Per-model state of :func:`topk_hook`: ratio and one fp32 residual per bucket."""

    def __init__(self, process_group=None, ratio: Optional[float] = None, warmup_dense_steps: int = 0):
        self.process_group = process_group
        self.ratio = float(ratio if ratio is not None else os.environ.get("MCCL_TOPK_RATIO", "0.01"))
        if not (0.0 < self.ratio <= 1.0):
            raise ValueError("ratio must be in (0, 1]")
        self.residuals: Dict[int, torch.Tensor] = {}
        self.warmup_dense_steps = warmup_dense_steps
        self.calls = 0

    def residual_for(self, bucket: dist.GradBucket) -> torch.Tensor:
        buf = bucket.buffer()
        idx = bucket.index()
        r = self.residuals.get(idx)
        if r is None or r.numel() != buf.numel() or r.device != buf.device:
            r = torch.zeros(buf.numel(), dtype=torch.float32, device=buf.device)
            self.residuals[idx] = r
        return r

    def reset(self) -> None:
        """Drops all residuals (they also restart at zero after a checkpoint resume)."""
        self.residuals.clear()


def topk_hook(state: TopKState, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """DDP comm hook: top-k compressed gradient averaging with error feedback."""
    buf = bucket.buffer()
    backend = _backend_for(state.process_group, buf.device)
    world = backend.size()
    if bucket.index() == 0:
        state.calls += 1
    if state.calls <= state.warmup_dense_steps:
        work = backend.allreduce_scaled(buf, 1.0 / world)
    else:
        work = backend.allreduce_topk(buf, state.residual_for(bucket), state.ratio, 1.0 / world)
    return work.get_future().then(lambda f: f.value()[0])


class OptimizerInBackward:
    """State of :func:`optimizer_in_backward_hook`: the fused optimizer and the process group."""

    def __init__(self, optimizer, process_group=None):
        self.optimizer = optimizer
        self.process_group = process_group
        self.backend = None   # resolved on first use
        self.scale = 1.0


def optimizer_in_backward_hook(state: OptimizerInBackward, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """DDP comm hook: fused-average allreduce, then the bucket's AdamW update, both off the main stream.

    One native call per bucket enqueues the allreduce kernel and, right behind it on the same
    communication stream, the AdamW kernel over the bucket's parameters; the returned future
    covers both.  The update therefore runs while later buckets are still being reduced and
    backward is still computing.  ``optimizer.step()`` afterwards only refreshes the step
    counters (and covers parameters that were not updated here, normally none).
    """
    buf = bucket.buffer()
    backend = state.backend
    if backend is None:
        backend = state.backend = _backend_for(state.process_group, buf.device)
        state.scale = 1.0 / backend.size()
    opt = state.optimizer
    if bucket.index() == 0:
        opt.begin_step_in_backward()
    plans = opt.bucket_plans(bucket.index(), bucket.parameters())
    grads = bucket.gradients()
    specs = []
    for plan, group, own, pos in plans:
        b1, b2 = group["betas"]
        specs.append((plan, [grads[i] for i in pos], group["lr"], b1, b2, group["eps"], group["weight_decay"]))
        opt.mark_bucket_stepped(own)
    work = backend.allreduce_adamw(buf, state.scale, specs, opt._bw_step)
    return work.get_future().then(_first_tensor)


def _first_tensor(fut):
    return fut.value()[0]


def _install_native_bucket_hook(ddp, optimizer, process_group) -> None:
    """Registers the C++ allreduce+AdamW hook on DDP's reducer (no Python per bucket).

    The optimizer's state is created up front and handed to the hook; a forward pre-hook pushes the
    current hyper-parameters and step number before every iteration.
    """
    from .. import require_native

    native = require_native()
    device = next(ddp.module.parameters()).device
    backend = _backend_for(process_group, device)
    state = native.BucketOptimizerState(backend, 1.0 / backend.size())
    optimizer.attach_native_hook(state)
    native._register_bucket_optimizer_hook(ddp.reducer, state)
    ddp._mccl_native_hook_state = state
    ddp.register_forward_pre_hook(lambda _m, _inp: optimizer.sync_native_hook())


def wrap_ddp(module: torch.nn.Module, *, device_ids=None, bucket_cap_mb: Optional[int] = None,
             compression: Optional[str] = None, fused_average: bool = True, process_group=None,
             optimizer_in_backward=None, **ddp_kwargs) -> DistributedDataParallel:
    """``DistributedDataParallel`` with the backend's fused hooks installed.

    ``compression`` (default: ``MCCL_COMPRESSION``) selects ``"topk"`` for the
    compressed hook; otherwise, on CUDA, the fused-average hook replaces DDP's
    separate divide pass.  ``bucket_cap_mb`` defaults to ``DDP_BUCKET_MB`` or 25.
    ``optimizer_in_backward`` takes a :class:`mccl_b200.optim.FusedAdamW` built over the
    module's parameters: each bucket is then updated right behind its allreduce (see
    :func:`optimizer_in_backward_hook`); keep calling ``optimizer.step()`` once per iteration.
    """
    if bucket_cap_mb is None:
        bucket_cap_mb = int(os.environ.get("DDP_BUCKET_MB", "25"))
    ddp_kwargs.setdefault("gradient_as_bucket_view", True)
    ddp = DistributedDataParallel(module, device_ids=device_ids, bucket_cap_mb=bucket_cap_mb,
                                  process_group=process_group, **ddp_kwargs)
    on_cuda = next(module.parameters()).is_cuda
    mode = compression if compression is not None else os.environ.get("MCCL_COMPRESSION", "none")
    if on_cuda and optimizer_in_backward is not None and mode != "topk":
        if os.environ.get("MCCL_PYTHON_BUCKET_HOOK", "0") == "1":
            ddp._mccl_oib_state = OptimizerInBackward(optimizer_in_backward, process_group)
            ddp.register_comm_hook(ddp._mccl_oib_state, optimizer_in_backward_hook)
        else:
            _install_native_bucket_hook(ddp, optimizer_in_backward, process_group)
    elif on_cuda and mode == "topk":
        ddp._mccl_topk_state = TopKState(process_group)
        ddp.register_comm_hook(ddp._mccl_topk_state, topk_hook)
    elif on_cuda and fused_average:
        ddp.register_comm_hook(process_group, fused_avg_hook)
    return ddp
