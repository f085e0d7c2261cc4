"""``Tensor``: the reference's tensor API as a thin facade over ``torch.Tensor``.

The reference class owns storage (a host float list or a device handle) and a hand-written autograd tape
(lib/core/tensor/tensor.dart:47-672).  Here storage, autograd and device placement are PyTorch's; the facade supplies
the reference's constructors, method names and conventions (``fromList``, ``toList``, ``[1,1]`` reductions, per-row
``crossEntropy``, float token ids, ``noGrad``, ``assign`` keeping identity) and routes every op through
``dart_pytorch_b200.ops`` so CUDA tensors hit the native kernels.  ``nn`` modules accept either a facade tensor or a
raw ``torch.Tensor`` and answer in kind.
"""
from __future__ import annotations

import contextlib
from enum import Enum
from typing import Callable, List, Optional, Sequence

import torch

from . import dtype as _dt
from . import ops as F


class Device(str, Enum):
    CPU = "cpu"
    GPU = "cuda"


class DType(str, Enum):
    fp32 = "fp32"
    fp16 = "fp16"
    bf16 = "bf16"

    @property
    def itemBytes(self) -> int:
        """Bytes per stored element (reference: lib/core/tensor/dtype.dart:41-44)."""
        return 4 if self is DType.fp32 else 2

    item_bytes = itemBytes


AUTO_DEVICE_THRESHOLD = 4096  # reference: tensors of at least this many elements default to the GPU when one exists

_TORCH_DTYPES = {DType.fp32: torch.float32, DType.fp16: torch.float16, DType.bf16: torch.bfloat16}


def _resolve_device(device, length: int) -> torch.device:
    if device is None:
        use_gpu = length >= AUTO_DEVICE_THRESHOLD and torch.cuda.is_available()
        return torch.device("cuda" if use_gpu else "cpu")
    if isinstance(device, Device):
        return torch.device(device.value)
    return torch.device(device)


class Tensor:
    __slots__ = ("t", "_debug_children", "debug_node")

    # Called as ``hook(step_index, tensor)`` after every backward closure of a ``backward()`` call, in execution order
    # (reference: debugBackwardHook, lib/core/tensor/tensor.dart:42-45, fired at tensor.dart:562-563).  The tape is
    # torch's, which keeps no handle on a node's forward result, so ``tensor`` wraps the gradient that arrived at the
    # node (what the reference user reads as ``tensor.grad``); ``tensor.debug_node`` names the closure and
    # ``tensor.debugChildShapes`` lists the shapes of the gradients it handed on.
    debug_backward_hook: Optional[Callable[[int, "Tensor"], None]] = None

    def __init__(self, t: torch.Tensor):
        self.t = t
        self._debug_children = None
        self.debug_node = None

    # ---- factories -------------------------------------------------------------------------------
    @staticmethod
    def fromList(shape: Sequence[int], values: Sequence[float], device=None, requiresGrad: bool = False) -> "Tensor":
        n = 1
        for s in shape:
            n *= int(s)
        if len(values) != n:
            raise ValueError(f"Tensor.fromList: shape {list(shape)} needs {n} values, got {len(values)}")
        t = torch.tensor(list(values), dtype=torch.float32).reshape(*shape).to(_resolve_device(device, n))
        t.requires_grad_(requiresGrad)
        return Tensor(t)

    from_list = fromList
    fromFloat32List = fromList

    @staticmethod
    def fill(shape: Sequence[int], value: float, device=None, requiresGrad: bool = False) -> "Tensor":
        n = 1
        for s in shape:
            n *= int(s)
        t = torch.full(tuple(shape), float(value), dtype=torch.float32, device=_resolve_device(device, n))
        t.requires_grad_(requiresGrad)
        return Tensor(t)

    @staticmethod
    def fromFp16Bits(shape: Sequence[int], bits: Sequence[int]) -> "Tensor":
        """Read-only half-precision storage tensor on the CPU (reference: tensor.dart:155-180)."""
        t = torch.tensor(list(bits), dtype=torch.int32).to(torch.int16).view(torch.float16).reshape(*shape)
        return Tensor(t)

    @staticmethod
    def noGrad(fn: Callable):
        with torch.no_grad():
            return fn()

    no_grad = noGrad

    # ---- metadata --------------------------------------------------------------------------------
    @property
    def shape(self) -> List[int]:
        return list(self.t.shape)

    @property
    def length(self) -> int:
        return self.t.numel()

    @property
    def device(self) -> Device:
        return Device.GPU if self.t.is_cuda else Device.CPU

    @property
    def dtype(self) -> DType:
        return {torch.float16: DType.fp16, torch.bfloat16: DType.bf16}.get(self.t.dtype, DType.fp32)

    @property
    def requiresGrad(self) -> bool:
        return self.t.requires_grad

    @property
    def grad(self) -> Optional["Tensor"]:
        return None if self.t.grad is None else Tensor(self.t.grad)

    @property
    def debugChildShapes(self) -> List[List[int]]:
        """Shapes of this tensor's autograd children, for debugging a graph (reference: tensor.dart:74-76).  Leaf
        children report their own shape; interior children the shape their producer recorded, when it recorded one."""
        fn = self.t.grad_fn
        out: List[List[int]] = []
        for nxt, idx in (fn.next_functions if fn is not None else ()):
            if nxt is None:
                continue
            var = getattr(nxt, "variable", None)
            if var is not None:
                out.append(list(var.shape))
                continue
            meta = getattr(nxt, "_input_metadata", None)
            if meta is not None and idx < len(meta):
                out.append([int(s) for s in meta[idx].shape])
        return out

    @property
    def residentBytes(self) -> int:
        return self.t.numel() * self.t.element_size()

    # ---- conversions -----------------------------------------------------------------------------
    def toList(self) -> List[float]:
        return self.t.detach().float().reshape(-1).cpu().tolist()

    to_list = toList
    toFloat32List = toList

    def toFp32(self) -> "Tensor":
        return Tensor(self.t.detach().float())

    def toFp16(self) -> "Tensor":
        """Round-to-nearest-even half storage, saturating to +-Inf (reference: dtype.dart:84-120)."""
        if self.t.is_cuda:
            raise RuntimeError("toFp16: half storage tensors live on the CPU")
        bits = _dt.fp32_to_fp16_bits(self.t.detach().float().reshape(-1))
        return Tensor(bits.view(torch.float16).reshape(self.t.shape))

    def to(self, device) -> "Tensor":
        dev = _resolve_device(device, self.length)
        t = self.t.detach()
        if dev.type == "cuda" and t.dtype == torch.float16:
            t = t.float()
        return Tensor(t.to(dev))

    def clone(self) -> "Tensor":
        return Tensor(self.t.detach().clone())

    detach = clone

    def assign(self, src: "Tensor") -> None:
        """Overwrite the values in place, keeping this tensor's identity (optimizer state stays attached)."""
        s = src.t if isinstance(src, Tensor) else src
        if self.t.dtype == torch.float16 or s.dtype == torch.float16:
            raise RuntimeError("assign: half storage tensors are read-only; promote with toFp32() first")
        if list(s.shape) != list(self.t.shape):
            raise ValueError(f"assign: shape mismatch {list(s.shape)} vs {list(self.t.shape)}")
        if s.device.type != self.t.device.type:
            raise ValueError(f"assign: device mismatch {s.device.type} vs {self.t.device.type}")
        with torch.no_grad():
            self.t.copy_(s.to(self.t.device, self.t.dtype))

    def adoptCpuStorageFrom(self, source: "Tensor") -> None:
        """Take over ``source``'s CPU buffer, dtype included (how loaders swap half-precision weights into a model
        without a copy); this tensor keeps its shape, loses its autograd state, and ``source`` is left empty
        (reference: lib/core/tensor/tensor.dart:442-470)."""
        if self.t.is_cuda or source.t.is_cuda:
            raise RuntimeError("adoptCpuStorageFrom: both tensors must be on the CPU")
        if source.length != self.length:
            raise ValueError(f"adoptCpuStorageFrom: length mismatch, got {source.length}, expected {self.length}")
        self.t = source.t.detach().reshape(self.t.shape)
        source.t = torch.empty(0)

    adopt_cpu_storage_from = adoptCpuStorageFrom

    def sliceRows(self, start: int, end: int) -> "Tensor":
        if not (0 <= start <= end <= self.t.shape[0]):
            raise IndexError("sliceRows: range out of bounds")
        return Tensor(self.t.detach()[start:end].clone())

    def dispose(self) -> None:
        self.t = torch.empty(0)

    # ---- autograd --------------------------------------------------------------------------------
    def backward(self, freeGraph: bool = True) -> None:
        if not self.t.requires_grad:
            raise RuntimeError("backward: tensor does not require grad")
        hook = Tensor.debug_backward_hook
        handles = []
        if hook is not None and self.t.grad_fn is not None:
            counter = [0]
            seen, stack = set(), [self.t.grad_fn]
            while stack:
                fn = stack.pop()
                if fn is None or fn in seen:
                    continue
                seen.add(fn)

                def fire(grad_inputs, grad_outputs, fn=fn):
                    g = next((x for x in grad_outputs if x is not None), None)
                    node = Tensor(g.detach() if g is not None else torch.zeros(()))
                    node._debug_children = [list(x.shape) for x in grad_inputs if x is not None]
                    node.debug_node = fn.name()
                    hook(counter[0], node)
                    counter[0] += 1
                handles.append(fn.register_hook(fire))
                stack.extend(f for f, _ in fn.next_functions)
        try:
            self.t.backward(torch.ones_like(self.t), retain_graph=not freeGraph)
        finally:
            for h in handles:
                h.remove()

    def zeroGrad(self) -> None:
        self.t.grad = None

    # ---- arithmetic ------------------------------------------------------------------------------
    @staticmethod
    def _raw(x):
        return x.t if isinstance(x, Tensor) else x

    def __add__(self, o):
        return Tensor(F.add(self.t, self._raw(o)))

    def __radd__(self, o):
        return Tensor(F.add(self.t, self._raw(o)))

    def __sub__(self, o):
        return Tensor(F.sub(self.t, self._raw(o)))

    def __rsub__(self, o):
        return Tensor(F.sub(self._raw(o), self.t))

    def __mul__(self, o):
        return Tensor(F.mul(self.t, self._raw(o)))

    def __rmul__(self, o):
        return Tensor(F.mul(self.t, self._raw(o)))

    def __truediv__(self, o):
        return Tensor(F.div(self.t, self._raw(o)))

    def __neg__(self):
        return Tensor(F.mul(self.t, -1.0))

    def relu(self):
        return Tensor(F.relu(self.t))

    def sigmoid(self):
        return Tensor(F.sigmoid(self.t))

    def tanh(self):
        return Tensor(F.tanh(self.t))

    def abs(self):
        return Tensor(F.abs(self.t))

    def log(self):
        return Tensor(F.log(self.t))

    def pow(self, e: float):
        return Tensor(F.pow(self.t, float(e)))

    def sum(self):
        return Tensor(F.sum(self.t))

    def mean(self):
        return Tensor(F.mean(self.t))

    def reshape(self, shape: Sequence[int]):
        return Tensor(self.t.reshape(*shape))

    def transpose(self):
        return Tensor(F.transpose(self.t))

    def matmul(self, o):
        return Tensor(F.matmul(self.t, self._raw(o)))

    def layerNorm(self, gamma, beta, eps: float = 1e-5):
        return Tensor(F.layer_norm(self.t, self._raw(gamma), self._raw(beta), eps))

    def rmsNorm(self, gamma, eps: float = 1e-6):
        return Tensor(F.rms_norm(self.t, self._raw(gamma), eps))

    def softmax(self):
        return Tensor(F.softmax(self.t))

    def crossEntropy(self, targets):
        return Tensor(F.cross_entropy(self.t, self._raw(targets)))

    def embedding(self, indices):
        return Tensor(F.embedding(self.t, self._raw(indices)))

    def scatterRowsAdd(self, indices, totalRows: int):
        return Tensor(F.scatter_rows_add(self.t, self._raw(indices), totalRows))

    def scaledDotProductAttention(self, k, v, mask=None):
        return Tensor(F.sdpa(self.t, self._raw(k), self._raw(v), None if mask is None else self._raw(mask)))

    def dropout(self, p: float, training: bool = True, rng=None):
        return Tensor(F.dropout(self.t, p, training, rng))

    def aftFull(self, k, v, w, causal: bool = True):
        return Tensor(F.aft_full(self.t, self._raw(k), self._raw(v), self._raw(w), causal))

    def sliceTopLeft(self, rows: int, cols: int):
        return Tensor(F.slice_top_left(self.t, rows, cols))

    def im2colNhwc(self, batch: int, channels: int, ksize: int):
        return Tensor(F.im2col_nhwc(self.t, batch, channels, ksize))

    @staticmethod
    def concat(tensors: Sequence["Tensor"], axis: int = 0) -> "Tensor":
        return Tensor(F.concat([Tensor._raw(t) for t in tensors], axis))

    @staticmethod
    def splitRows(t: "Tensor", chunk: int) -> List["Tensor"]:
        return [Tensor(x) for x in F.split_rows(Tensor._raw(t), chunk)]

    def __repr__(self):
        return f"Tensor(shape={self.shape}, device={self.device.name}, dtype={self.dtype.name})"


# ---- helpers used by nn.Module.__call__ ---------------------------------------------------------
def unwrap_args(args, kwargs):
    wrapped = False

    def un(x):
        nonlocal wrapped
        if isinstance(x, Tensor):
            wrapped = True
            return x.t
        return x

    return wrapped or any(isinstance(a, Tensor) for a in args), tuple(un(a) for a in args), \
        {k: un(v) for k, v in kwargs.items()}


def wrap_like(out):
    if isinstance(out, torch.Tensor):
        return Tensor(out)
    if isinstance(out, tuple):
        return tuple(wrap_like(o) for o in out)
    if isinstance(out, list):
        return [wrap_like(o) for o in out]
    return out
