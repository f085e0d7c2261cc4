"""Optimizer base: parameter list, mutable ``lr``, ``step()``, ``zeroGrad()``
(reference: lib/core/optim/optimizer.dart:12-33).

On a CUDA device the constructor re-homes the parameters into a ``ParamArena`` (flat weights, flat gradients, fp32
master copy for bf16 models) so that the update, the clip-norm reduction and gradient zeroing are single kernels."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..utils.arena import ParamArena


class Optimizer:
    def __init__(self, parameters: Sequence[torch.Tensor], lr: float, arena: Optional[bool] = None):
        self.parameters: List[torch.Tensor] = list(parameters)
        if not self.parameters:
            raise ValueError("Optimizer: empty parameter list")
        self.lr = float(lr)
        on_cuda = all(p.is_cuda for p in self.parameters)
        use_arena = on_cuda if arena is None else (arena and on_cuda)
        self.arena: Optional[ParamArena] = None
        if use_arena:
            existing = {id(getattr(p, "_dptb_arena", None)) for p in self.parameters}
            first = getattr(self.parameters[0], "_dptb_arena", None)
            if first is not None and len(existing) == 1 and len(first.params) == len(self.parameters):
                self.arena = first
            else:
                self.arena = ParamArena(self.parameters)
            self.ctrl = torch.zeros(4, dtype=torch.float32, device=self.arena.device)
            self.ctrl[1] = 1.0
            self.ctrl[2] = 1.0
            self.clip_pending = False
            self.arena.optimizer = self

    def step(self) -> None:
        raise NotImplementedError

    def zero_grad(self) -> None:
        if self.arena is not None:
            self.arena.zero_grad()
            return
        for p in self.parameters:
            p.grad = None

    zeroGrad = zero_grad

    def _grad_ctrl(self):
        """Device control block carrying the clip coefficient, or None when no clip is pending."""
        if self.arena is not None and self.clip_pending:
            return self.ctrl
        return None
