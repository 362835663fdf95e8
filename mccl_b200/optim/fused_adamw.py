"""FusedAdamW: ``torch.optim.AdamW`` semantics, one kernel launch per step.

The whole parameter set is updated by a single multi-tensor kernel
(``csrc/kernels/adamw.cu``) that streams (p, g, m, v) once: 28 bytes per fp32
parameter, the HBM floor of the update.  State is kept in the standard
``state[p] = {"step", "exp_avg", "exp_avg_sq"}`` layout, so ``state_dict()`` is
interchangeable with ``torch.optim.AdamW`` (checkpoints load either way).
``grad_scale`` lets a caller fold a deferred gradient scaling (for example the
1/world of a summed allreduce) into the update instead of a separate pass.
"""
from __future__ import annotations

from typing import Iterable

import torch

from .. import require_native


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2):
        if lr < 0 or eps < 0 or weight_decay < 0 or not (0 <= betas[0] < 1) or not (0 <= betas[1] < 1):
            raise ValueError("invalid AdamW hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self._plans = {}
        # DDP hands back bucket parameters as tensors that may be fresh Python objects: find ours by address
        self._by_ptr = {p.data_ptr(): (p, g) for g in self.param_groups for p in g["params"]}
        self._bw_cache = {}
        self._bw_touched = []
        self._bw_step = 0
        self._bw_done = set()

    def _plan_for(self, gi: int, params):
        key = (gi, tuple(p.data_ptr() for p in params))
        plan = self._plans.get(gi)
        if plan is None or plan[0] != key:
            native = require_native()
            ms, vs = [], []
            for p in params:
                st = self.state[p]
                if "exp_avg" not in st:
                    st["step"] = torch.tensor(0.0)
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                ms.append(st["exp_avg"])
                vs.append(st["exp_avg_sq"])
            plan = (key, native.AdamWPlan([p.data for p in params], ms, vs))
            self._plans[gi] = plan
        return plan[1]

    @torch.no_grad()
    def step(self, closure=None, *, grad_scale: float = 1.0):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for own in self._bw_touched:  # updated inside backward: only their step counters are left to refresh
            for p in own:
                self.state[p]["step"].fill_(float(self._bw_step))
                self._bw_done.add(id(p))
        self._bw_touched = []
        for gi, group in enumerate(self.param_groups):
            # parameters already updated inside backward are skipped
            params = [p for p in group["params"] if p.grad is not None and id(p) not in self._bw_done]
            if not params:
                continue
            if not all(p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() for p in params):
                raise RuntimeError("FusedAdamW handles contiguous float32 CUDA parameters "
                                   "(see mccl_b200.params.ensure_contiguous_parameters)")
            plan = self._plan_for(gi, params)
            st0 = self.state[params[0]]
            step = int(st0["step"].item()) + 1 if isinstance(st0["step"], torch.Tensor) else int(st0["step"]) + 1
            grads = [p.grad if p.grad.is_contiguous() else p.grad.contiguous() for p in params]
            b1, b2 = group["betas"]
            plan.step(grads, group["lr"], b1, b2, group["eps"], group["weight_decay"], step, grad_scale)
            for p in params:
                s = self.state[p]["step"]
                if isinstance(s, torch.Tensor):
                    s.fill_(float(step))  # host tensor, as torch.optim.AdamW keeps it by default
                else:
                    self.state[p]["step"] = step
        self._bw_done = set()
        return loss

    # ---- per-bucket stepping (optimizer inside backward) -----------------------
    def begin_step_in_backward(self) -> int:
        """Advances the shared step counter once per iteration; returns the new step."""
        self._bw_step = getattr(self, "_bw_step", None)
        any_p = next(p for g in self.param_groups for p in g["params"])
        st = self.state[any_p]
        cur = int(st["step"].item()) if "step" in st else 0
        self._bw_step = cur + 1
        self._bw_done = set()
        self._bw_touched = []
        return self._bw_step

    def bucket_plan(self, key, params):
        """``(plan, group)`` for one DDP bucket: the cached launch plan over the bucket's parameters."""
        ent = self._bw_cache.get(key)
        if ent is None or ent[0] != params[0].data_ptr():
            own = [self._by_ptr[p.data_ptr()][0] for p in params]
            group = self._by_ptr[own[0].data_ptr()][1]
            ent = (params[0].data_ptr(), own, group, self._plan_for(("bucket", key), own))
            self._bw_cache[key] = ent
        return ent[3], ent[2], ent[1]

    def mark_bucket_stepped(self, own) -> None:
        self._bw_touched.append(own)

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        self._plans.clear()  # state tensors were replaced
        self._bw_cache.clear()
