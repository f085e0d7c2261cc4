"""dart_pytorch_b200: a Blackwell-native tensor / autograd / nn framework with the capabilities of dart_pytorch.

PyTorch is the framework layer; every hot op on a CUDA device is a hand-written sm_100a kernel from ``csrc/``
(loaded from ``_C/libdptb200.so``); CPU tensors run the fp32 reference formulas that double as the test oracle.
"""
from . import ops
from .tensor import Tensor, Device, DType
from . import nn, optim, models, io
from .nn import *  # noqa: F401,F403
from .optim import SGD, Adam, clip_grad_norm, clipGradNorm, StepLR, LinearWarmupCosineDecay, LRScheduler, Optimizer
from .models import GPT, GPTConfig
from .io import Checkpoint

__version__ = "0.1.0"
