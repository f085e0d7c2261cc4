"""SGD with optional momentum and L2 weight decay (reference: lib/core/optim/sgd.dart:16-84):
``g += wd * p``; ``v = g`` on the first step, then ``v = momentum * v + g``; ``p -= lr * v``."""
from __future__ import annotations

import torch

from .optimizer import Optimizer


class SGD(Optimizer):
    def __init__(self, parameters, lr: float, momentum: float = 0.0, weight_decay: float = 0.0, weightDecay=None,
                 arena=None):
        super().__init__(parameters, lr, arena)
        self.momentum = float(momentum)
        self.weight_decay = float(weight_decay if weightDecay is None else weightDecay)
        self._velocity = {}
        self._steps = 0
        if self.arena is not None and self.momentum != 0.0:
            self._buf = torch.zeros(self.arena.numel, dtype=torch.float32, device=self.arena.device)
        else:
            self._buf = None

    def step(self) -> None:
        if self.arena is not None:
            from ..ops import kernels as K
            a = self.arena
            master = a.master if a.master is not None else a.flat
            shadow = a.flat if a.master is not None else None
            K.sgd_flat(master, shadow, a.grad, self._buf, self._grad_ctrl(), self.lr, self.momentum, self.weight_decay,
                       self._steps == 0)
            self.clip_pending = False
            self._steps += 1
            return
        with torch.no_grad():
            for p in self.parameters:
                if p.grad is None:
                    continue
                g = p.grad
                if self.weight_decay != 0.0:
                    g = g + self.weight_decay * p
                if self.momentum != 0.0:
                    v = self._velocity.get(id(p))
                    v = g.clone() if v is None else self.momentum * v + g
                    self._velocity[id(p)] = v
                    g = v
                p.sub_(self.lr * g)
        self._steps += 1
