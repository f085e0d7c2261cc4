"""Learning-rate schedules (reference: lib/core/optim/lr_scheduler.dart:36-145).  ``step()`` is called after
``optimizer.step()``: it increments ``stepCount`` and sets ``optimizer.lr = lrAt(stepCount)``."""
from __future__ import annotations

import math


class LRScheduler:
    def __init__(self, optimizer):
        self.optimizer = optimizer
        self.step_count = 0

    @property
    def stepCount(self) -> int:
        return self.step_count

    @property
    def last_lr(self) -> float:
        return self.optimizer.lr

    lastLr = last_lr

    def lr_at(self, step: int) -> float:
        raise NotImplementedError

    lrAt = lambda self, step: self.lr_at(step)  # noqa: E731

    def step(self) -> None:
        self.step_count += 1
        self.optimizer.lr = self.lr_at(self.step_count)


class StepLR(LRScheduler):
    """``lr = initialLr * gamma^(step // stepSize)``; the constructor sets ``optimizer.lr = initialLr``."""

    def __init__(self, optimizer, step_size: int, gamma: float = 0.1, initial_lr=None, stepSize=None, initialLr=None):
        super().__init__(optimizer)
        step_size = stepSize if stepSize is not None else step_size
        if step_size <= 0:
            raise ValueError("StepLR: stepSize must be > 0")
        self.step_size, self.gamma = int(step_size), float(gamma)
        init = initialLr if initialLr is not None else initial_lr
        self.initial_lr = float(optimizer.lr if init is None else init)
        optimizer.lr = self.initial_lr

    def lr_at(self, step: int) -> float:
        return self.initial_lr * (self.gamma ** (step // self.step_size))


class LinearWarmupCosineDecay(LRScheduler):
    """``t <= warm: max*t/warm``; ``t >= total: min``; else ``min + 0.5 (max-min)(1 + cos(pi (t-warm)/(total-warm)))``.
    The constructor sets ``optimizer.lr = lrAt(1)``."""

    def __init__(self, optimizer, warmup_steps=None, total_steps=None, max_lr=None, min_lr: float = 0.0,
                 warmupSteps=None, totalSteps=None, maxLr=None, minLr=None):
        super().__init__(optimizer)
        self.warmup_steps = int(warmupSteps if warmupSteps is not None else warmup_steps)
        self.total_steps = int(totalSteps if totalSteps is not None else total_steps)
        self.max_lr = float(maxLr if maxLr is not None else (max_lr if max_lr is not None else optimizer.lr))
        self.min_lr = float(minLr if minLr is not None else min_lr)
        if self.warmup_steps < 0 or self.total_steps <= 0 or self.warmup_steps > self.total_steps:
            raise ValueError("LinearWarmupCosineDecay: need 0 <= warmupSteps <= totalSteps, totalSteps > 0")
        if self.min_lr > self.max_lr:
            raise ValueError("LinearWarmupCosineDecay: minLr must not exceed maxLr")
        optimizer.lr = self.lr_at(1)

    def lr_at(self, step: int) -> float:
        if self.warmup_steps > 0 and step <= self.warmup_steps:
            return self.max_lr * step / self.warmup_steps
        if step >= self.total_steps:
            return self.min_lr
        span = self.total_steps - self.warmup_steps
        prog = (step - self.warmup_steps) / span
        return self.min_lr + 0.5 * (self.max_lr - self.min_lr) * (1.0 + math.cos(math.pi * prog))
