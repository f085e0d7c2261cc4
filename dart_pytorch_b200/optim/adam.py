"""Adam with decoupled weight decay (reference: lib/core/optim/adam.dart:18-124).

``m = b1 m + (1-b1) g``; ``v = b2 v + (1-b2) g^2``; ``update = lr * (m / (1-b1^t)) / (sqrt(v / (1-b2^t)) + eps)``;
``update += lr * wd * p`` (decay applied to every parameter, as the reference does); parameters without a gradient are
skipped.  On the device this is one kernel over the arena: it reads the bf16 gradient (times the pending clip
coefficient), updates fp32 master / m / v and rewrites the bf16 working copy."""
from __future__ import annotations

import math

import torch

from .optimizer import Optimizer


class Adam(Optimizer):
    HYPER_SLOTS = 16

    def __init__(self, parameters, lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                 weight_decay: float = 0.0, weightDecay=None, arena=None, skip_nonfinite: bool = False):
        super().__init__(parameters, lr, arena)
        self.beta1, self.beta2, self.eps = float(beta1), float(beta2), float(eps)
        self.weight_decay = float(weight_decay if weightDecay is None else weightDecay)
        self.skip_nonfinite = skip_nonfinite
        self._step = 0
        self._m, self._v = {}, {}
        if self.arena is not None:
            n, dev = self.arena.numel, self.arena.device
            self.m = torch.zeros(n, dtype=torch.float32, device=dev)
            self.v = torch.zeros(n, dtype=torch.float32, device=dev)
            # {lr, 1-b1^t, 1-b2^t} read by the kernel from device memory, so a captured graph sees fresh values.
            self.hyper = torch.zeros(4, dtype=torch.float32, device=dev)
            # The host may queue many steps before the GPU runs the first; each step's values therefore get their own
            # pinned slot, reused only after the copy that read it has completed (an event per slot).
            self._hyper_ring = [torch.zeros(4, dtype=torch.float32).pin_memory() for _ in range(self.HYPER_SLOTS)]
            self._hyper_events = [None] * self.HYPER_SLOTS

    @property
    def step_count(self) -> int:
        return self._step

    def prepare_step(self) -> None:
        """Host half of a device step: advance ``t`` and publish {lr, bias corrections} to the device (async copy).
        Call outside a CUDA-graph capture; ``launch_step`` is the capturable half."""
        self._step += 1
        slot = self._step % self.HYPER_SLOTS
        done = self._hyper_events[slot]
        if done is not None:
            done.synchronize()               # the copy issued HYPER_SLOTS steps ago has read this slot
        host = self._hyper_ring[slot]
        host[0] = self.lr
        host[1] = 1.0 - self.beta1 ** self._step
        host[2] = 1.0 - self.beta2 ** self._step
        self.hyper.copy_(host, non_blocking=True)
        done = done if done is not None else torch.cuda.Event()
        done.record()
        self._hyper_events[slot] = done

    def launch_step(self) -> None:
        from ..ops import kernels as K
        a = self.arena
        master = a.master if a.master is not None else a.flat
        shadow = a.flat if a.master is not None else None
        K.adam_flat(master, shadow, a.grad, self.m, self.v, self._grad_ctrl(), self.lr, self.beta1, self.beta2, self.eps,
                    self.weight_decay, 1.0, 1.0, skip_if_nonfinite=self.skip_nonfinite, hyper=self.hyper)
        self.clip_pending = False

    def step(self) -> None:
        if self.arena is not None:
            self.prepare_step()
            self.launch_step()
            return
        self._step += 1
        bc1 = 1.0 - self.beta1 ** self._step
        bc2 = 1.0 - self.beta2 ** self._step
        # Parameters outside an arena (CPU models, odd dtypes): the same update, m = b1 m + (1-b1) g,
        # v = b2 v + (1-b2) g^2, p -= lr (m / bc1) / (sqrt(v / bc2) + eps) + lr wd p, as multi-tensor list ops.
        with torch.no_grad():
            ps, gs, ms, vs = [], [], [], []
            for p in self.parameters:
                if p.grad is None:
                    continue
                m = self._m.get(id(p))
                if m is None:
                    m = self._m[id(p)] = torch.zeros_like(p)
                    self._v[id(p)] = torch.zeros_like(p)
                ps.append(p)
                gs.append(p.grad if p.grad.dtype == p.dtype else p.grad.to(p.dtype))
                ms.append(m)
                vs.append(self._v[id(p)])
            if not ps:
                return
            torch._foreach_mul_(ms, self.beta1)
            torch._foreach_add_(ms, gs, alpha=1.0 - self.beta1)
            torch._foreach_mul_(vs, self.beta2)
            torch._foreach_addcmul_(vs, gs, gs, value=1.0 - self.beta2)
            denom = torch._foreach_div(vs, bc2)
            torch._foreach_sqrt_(denom)
            torch._foreach_add_(denom, self.eps)
            if self.weight_decay != 0.0:
                torch._foreach_add_(ps, torch._foreach_mul(ps, -self.lr * self.weight_decay))
            torch._foreach_addcdiv_(ps, ms, denom, value=-self.lr / bc1)
