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
        self._by_ptr = {}
        self._index_params()
        self._bw_cache = {}
        self._bw_touched = []
        self._bw_step = 0
        self._bw_done = set()
        self._native_hook = None   # BucketOptimizerState when the native DDP hook is installed

    def _index_params(self) -> None:
        self._by_ptr = {p.data_ptr(): (p, gi) for gi, g in enumerate(self.param_groups) for p in g["params"]}

    def add_param_group(self, param_group) -> None:
        super().add_param_group(param_group)
        if hasattr(self, "_by_ptr"):  # the base constructor calls this before our fields exist
            self._index_params()
            self._bw_cache.clear()

    def _plan_for(self, gi, params):
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
        if self._native_hook is not None:  # parameters the native bucket hook updated during backward
            used_step, ptrs = self._native_hook.take_stepped()
            if ptrs:
                self._bw_step = used_step
                self._bw_touched.append([self._by_ptr[a][0] for a in ptrs if a in self._by_ptr])
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

    def bucket_plans(self, key, params):
        """Launch plans of one DDP bucket: a list of ``(plan, group, own_params, positions)``.

        A bucket may hold parameters of several param groups (for example weights with weight decay
        and biases without); each group gets its own plan so that every parameter is updated with its
        own group's hyper-parameters.  ``positions`` are the indices of the group's parameters inside
        ``params`` (and inside ``bucket.gradients()``).  The cache entry is keyed by the addresses of
        all the bucket's parameters, so a rebuilt bucket is noticed even if its first parameter stays.
        """
        sig = tuple(p.data_ptr() for p in params)
        ent = self._bw_cache.get(key)
        if ent is None or ent[0] != sig:
            by_group = {}
            for pos, p in enumerate(params):
                try:
                    own, gi = self._by_ptr[p.data_ptr()]
                except KeyError:
                    raise KeyError("a DDP bucket holds a parameter this optimizer was not given") from None
                by_group.setdefault(gi, ([], []))
                by_group[gi][0].append(own)
                by_group[gi][1].append(pos)
            plans = []
            for gi in sorted(by_group):
                own, pos = by_group[gi]
                plans.append((self._plan_for(("bucket", key, gi), own), self.param_groups[gi], own, pos))
            ent = (sig, plans)
            self._bw_cache[key] = ent
        return ent[1]

    # ---- native hook support ------------------------------------------------------
    def ensure_state(self) -> None:
        """Creates the AdamW state of every parameter (so that a native hook can be given the tensors)."""
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state[p]
                if "exp_avg" not in st:
                    st["step"] = torch.tensor(0.0)
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)

    def attach_native_hook(self, hook_state) -> None:
        """Hands parameters, state tensors and group indices to a ``BucketOptimizerState``."""
        self.ensure_state()
        for gi, group in enumerate(self.param_groups):
            for p in group["params"]:
                if not (p.is_cuda and p.dtype == torch.float32 and p.is_contiguous()):
                    raise RuntimeError("FusedAdamW handles contiguous float32 CUDA parameters")
                st = self.state[p]
                hook_state.add_param(p.data, st["exp_avg"], st["exp_avg_sq"], gi)
        self._native_hook = hook_state
        self.sync_native_hook()

    def sync_native_hook(self) -> None:
        """Pushes the groups' current hyper-parameters and the next step number to the native hook.

        Called before every forward: whatever a learning-rate scheduler did since the last step is
        what the bucket updates of the coming backward use.
        """
        if self._native_hook is None:
            return
        for gi, group in enumerate(self.param_groups):
            b1, b2 = group["betas"]
            self._native_hook.set_hyper(gi, group["lr"], b1, b2, group["eps"], group["weight_decay"])
        any_p = next(p for g in self.param_groups for p in g["params"])
        st = self.state[any_p]
        cur = int(st["step"].item()) if "step" in st else 0
        self._native_hook.set_step(cur + 1)

    def mark_bucket_stepped(self, own) -> None:
        self._bw_touched.append(own)

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        self._plans.clear()  # state tensors were replaced
        self._bw_cache.clear()
        if self._native_hook is not None:
            self.attach_native_hook(self._native_hook)
