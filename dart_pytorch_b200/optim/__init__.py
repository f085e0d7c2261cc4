"""Optimizers, gradient clipping and learning-rate schedules (reference: lib/core/optim/*.dart)."""
from .optimizer import Optimizer
from .sgd import SGD
from .adam import Adam
from .grad_utils import clip_grad_norm, clipGradNorm, LazyScalar
from .lr_scheduler import LRScheduler, StepLR, LinearWarmupCosineDecay

__all__ = ["Optimizer", "SGD", "Adam", "clip_grad_norm", "clipGradNorm", "LazyScalar", "LRScheduler", "StepLR",
           "LinearWarmupCosineDecay"]
