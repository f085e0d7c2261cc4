"""Reference arm of the headline benchmark: one GPT-2 124M training step composed out of the reference's own,
unmodified native CUDA library.

The reference (KellyKinyama/dart-pytorch) is a Dart package over ``dart:ffi``; no Dart SDK exists on the build or GPU
machines, so its Dart layer cannot execute.  Its device code is one translation unit (lib/native/src/engine.cu) that
builds with nvcc as-is into ``baseline/_ref/libdart_engine.so``.  This module restates, call for call, what the Dart
layer does *around* that library on the GPU path of ``bin/gpt_train.dart:111-131`` and drives the library's exported
functions in the same order with the same operands:

* ``T`` mirrors ``lib/core/tensor/tensor.dart`` on ``Device.GPU``: one native handle per tensor, every op result a
  freshly allocated handle, reverse-mode autograd by closures over children, ``backward(freeGraph: true)`` releasing
  intermediates as it walks (tensor.dart:539-585), ``_accumulateGrad`` (tensor.dart:621-637), host round trips exactly
  where the Dart code has them (``reshape`` ops.dart:458-477, ``clone`` tensor.dart:369-377, ``concat`` / ``splitRows``
  concat.dart:14-200, the row-broadcast gradient reduction tensor.dart:642-668).
* the module classes mirror ``lib/core/nn``: ``Linear`` (linear.dart:57-88), per-head projections and the per-head x
  per-sequence attention loop of ``MultiHeadAttention._callBatched`` (attention/multi_head_attention.dart:203-235),
  ``scaledDotProductAttention`` as transpose / matmul / scale / mask / softmax / matmul (tensor/attention.dart:43-58),
  the pre-LN block with the tanh GELU written in elementwise ops (transformer.dart:81-102), the weight-tied GPT
  (gpt.dart:150-167).
* ``Adam`` is the elementwise chain of optim/adam.dart:67-109 (decoupled weight decay), ``clip_grad_norm`` the
  host-side norm of optim/grad_utils.dart:7-40, ``LinearWarmupCosineDecay`` optim/lr_scheduler.dart:52-93.

Nothing of this repository's package, kernels or engine is imported here: the only native code on this path is
``libdart_engine.so``.  The library is fp32-only and single-GPU, so the arm reports ``dtype: fp32`` and is unavailable for
more than one GPU.  The library allocates a data and a gradient buffer per handle and the graph of one 16 x 1024 batch
does not fit in one GPU's memory, so a step of 16 sequences is run as several smaller forward/backward passes whose
gradients accumulate (``_accumulateGrad`` adds into an existing ``.grad``) before one clip + Adam; the split is chosen from
a dry run of the same graph on a shape-only engine and reported in ``config``.
"""
from __future__ import annotations

import ctypes
import json
import math
import os
import time
from typing import Callable, List, Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "libdart_engine.so")


# ---------------------------------------------------------------------------------------------------------------------
# Engines: the C ABI of lib/native/src/engine.cu, a NumPy restatement of it (CPU tests), and a shape-only planner.
# ---------------------------------------------------------------------------------------------------------------------

class CudaEngine:
    """ctypes binding of the unmodified reference library (lib/native/src/engine.cu:94-596)."""

    name = "libdart_engine.so"

    def __init__(self, path: str = LIB_PATH):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = L = ctypes.CDLL(path)
        vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.create_tensor.restype, L.create_tensor.argtypes = vp, [ci, ci, vp]
        L.destroy_tensor.restype, L.destroy_tensor.argtypes = None, [vp]
        L.get_tensor_data.restype, L.get_tensor_data.argtypes = None, [vp, vp]
        two = ("matmul_tensors", "add_tensors", "sub_tensors", "mul_tensors", "div_tensors", "add_tensor_scalar",
               "sub_tensor_scalar", "mul_tensor_scalar", "div_tensor_scalar", "add_tensor_row_broadcast",
               "softmax_backward", "cross_entropy_forward")
        one = ("tanh_tensor", "transpose_tensor", "sum_tensor", "mean_tensor", "softmax_forward")
        for n in two:
            f = getattr(L, n)
            f.restype, f.argtypes = vp, [vp, vp]
        for n in one:
            f = getattr(L, n)
            f.restype, f.argtypes = vp, [vp]
        L.pow_tensor.restype, L.pow_tensor.argtypes = vp, [vp, cf]
        L.layernorm_forward.restype, L.layernorm_forward.argtypes = vp, [vp, vp, vp, cf]
        L.layernorm_backward.restype, L.layernorm_backward.argtypes = vp, [vp, vp, vp, vp, vp, cf]
        L.cross_entropy_backward.restype, L.cross_entropy_backward.argtypes = vp, [vp, vp, vp]
        L.embedding_forward.restype, L.embedding_forward.argtypes = vp, [vp, vp, ci]
        L.embedding_backward.restype, L.embedding_backward.argtypes = None, [vp, vp, vp, ci]

    def create(self, rows: int, cols: int, data: Optional[np.ndarray]):
        ptr = None
        if data is not None:
            data = np.ascontiguousarray(data, dtype=np.float32)
            assert data.size == rows * cols
            ptr = data.ctypes.data_as(ctypes.c_void_p)
        h = self.lib.create_tensor(rows, cols, ptr)
        if not h:
            raise MemoryError("create_tensor returned null")
        return h

    def destroy(self, h) -> None:
        self.lib.destroy_tensor(h)

    def read(self, h, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        self.lib.get_tensor_data(h, out.ctypes.data_as(ctypes.c_void_p))
        return out

    def call(self, name: str, *args):
        """One exported function, by its C name; returns the new handle (or None for the in-place ones)."""
        return getattr(self.lib, name)(*args)


class NumpyEngine:
    """The same entry points on host arrays, following the kernels' formulas (lib/native/src/kernels/*.cuh).  Used to
    test the graph logic of this module on a machine without a GPU."""

    name = "numpy"

    def __init__(self):
        self.t = {}
        self.next = 1

    def _new(self, a: np.ndarray):
        h = self.next
        self.next += 1
        self.t[h] = np.array(a, dtype=np.float32)
        return h

    def create(self, rows, cols, data):
        a = np.zeros((rows, cols), np.float32) if data is None else np.asarray(data, np.float32).reshape(rows, cols)
        return self._new(a)

    def destroy(self, h):
        del self.t[h]

    def read(self, h, n):
        return self.t[h].reshape(-1).copy()

    def call(self, name, *args):
        t = self.t
        a = t[args[0]] if args and args[0] in t else None
        if name == "matmul_tensors":
            return self._new(a @ t[args[1]])
        arith = {"add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide}
        if name in ("add_tensors", "sub_tensors", "mul_tensors", "div_tensors"):
            return self._new(arith[name[:3]](a, t[args[1]].reshape(a.shape)))
        if name.endswith("_tensor_scalar"):
            return self._new(arith[name[:3]](a, t[args[1]].reshape(-1)[0]))
        if name == "add_tensor_row_broadcast":
            return self._new(a + t[args[1]].reshape(1, -1))
        if name == "tanh_tensor":
            return self._new(np.tanh(a))
        if name == "pow_tensor":
            return self._new(np.power(a, np.float32(args[1])))
        if name == "transpose_tensor":
            return self._new(a.T)
        if name == "sum_tensor":
            return self._new(a.sum(dtype=np.float64).reshape(1, 1))
        if name == "mean_tensor":
            return self._new(a.mean(dtype=np.float64).reshape(1, 1))
        if name == "softmax_forward":
            e = np.exp(a - a.max(1, keepdims=True))
            return self._new(e / e.sum(1, keepdims=True))
        if name == "softmax_backward":
            g = t[args[1]]
            return self._new((g - (g * a).sum(1, keepdims=True)) * a)
        if name == "layernorm_forward":
            g, b, eps = t[args[1]].reshape(1, -1), t[args[2]].reshape(1, -1), args[3]
            mu = a.mean(1, keepdims=True)
            var = ((a - mu) ** 2).mean(1, keepdims=True)
            return self._new((a - mu) / np.sqrt(var + eps) * g + b)
        if name == "layernorm_backward":
            g, go, eps = t[args[1]].reshape(1, -1), t[args[2]], args[5]
            mu = a.mean(1, keepdims=True)
            inv = 1.0 / np.sqrt(((a - mu) ** 2).mean(1, keepdims=True) + eps)
            xh = (a - mu) * inv
            dxh = go * g
            t[args[3]] += (go * xh).sum(0).reshape(t[args[3]].shape)
            t[args[4]] += go.sum(0).reshape(t[args[4]].shape)
            return self._new((dxh - dxh.mean(1, keepdims=True) - xh * (dxh * xh).mean(1, keepdims=True)) * inv)
        if name == "cross_entropy_forward":
            tg = (t[args[1]].reshape(-1) + 0.5).astype(np.int64)
            m = a.max(1, keepdims=True)
            lse = m[:, 0] + np.log(np.exp(a - m).sum(1))
            return self._new((lse - a[np.arange(a.shape[0]), tg]).reshape(-1, 1))
        if name == "cross_entropy_backward":
            tg = (t[args[1]].reshape(-1) + 0.5).astype(np.int64)
            e = np.exp(a - a.max(1, keepdims=True))
            p = e / e.sum(1, keepdims=True)
            p[np.arange(a.shape[0]), tg] -= 1.0
            return self._new(p * t[args[2]].reshape(-1, 1))
        if name == "embedding_forward":
            idx = (t[args[1]].reshape(-1) + 0.5).astype(np.int64)
            return self._new(a[idx])
        if name == "embedding_backward":
            idx = (t[args[0]].reshape(-1) + 0.5).astype(np.int64)
            np.add.at(t[args[2]], idx, t[args[1]])
            return None
        raise KeyError(name)


class ShapeEngine:
    """Allocates nothing and computes nothing: handles are counters and reads return zeros.  Running the step on it
    gives the exact sequence of allocations, hence the peak of live device bytes the real library would hold."""

    name = "shape-only"

    def __init__(self):
        self.next = 1

    def create(self, rows, cols, data):
        self.next += 1
        return self.next

    def destroy(self, h):
        pass

    def read(self, h, n):
        return np.zeros(n, dtype=np.float32)

    def call(self, name, *args):
        self.next += 1
        return None if name == "embedding_backward" else self.next


class Runtime:
    """What the Dart process keeps globally: the engine, the no-grad depth, and (for this arm) an account of the bytes
    the library holds (each native ``Tensor`` owns a data and a gradient buffer: engine.cu:24-58)."""

    def __init__(self, engine):
        self.e = engine
        self.no_grad = 0        # > 0 inside Tensor.noGrad and while backward closures run (see T.backward)
        self.live = 0
        self.peak = 0
        self.calls = 0          # exported-function calls that launch kernels
        self.h2d = 0
        self.d2h = 0

    def account(self, n_elems: int) -> None:
        self.live += 8 * n_elems
        if self.live > self.peak:
            self.peak = self.live


def _prod(shape: Sequence[int]) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


def _rows_cols(shape: Sequence[int]):
    return int(shape[0]), (_prod(shape[1:]) if len(shape) > 1 else 1)


# ---------------------------------------------------------------------------------------------------------------------
# Tensor + autograd (lib/core/tensor/*.dart, GPU device)
# ---------------------------------------------------------------------------------------------------------------------

class T:
    __slots__ = ("rt", "h", "shape", "requires_grad", "grad", "children", "back", "__weakref__")

    def __init__(self, rt: Runtime, shape: Sequence[int], handle, requires_grad: bool = False):
        self.rt, self.h, self.shape = rt, handle, [int(s) for s in shape]
        self.requires_grad, self.grad, self.children, self.back = requires_grad, None, (), None
        rt.account(self.length)

    # -- construction / host transfer (tensor.dart:128-236, 339-377) -------------------------------------------------
    @property
    def length(self) -> int:
        return _prod(self.shape)

    @staticmethod
    def upload(rt: Runtime, shape, data: np.ndarray, requires_grad: bool = False) -> "T":
        r, c = _rows_cols(shape)
        rt.h2d += 4 * r * c
        return T(rt, shape, rt.e.create(r, c, data), requires_grad)

    @staticmethod
    def fill(rt: Runtime, shape, value: float, requires_grad: bool = False) -> "T":
        return T.upload(rt, shape, np.full(_prod(shape), value, dtype=np.float32), requires_grad)

    def to_host(self) -> np.ndarray:
        self.rt.d2h += 4 * self.length
        return self.rt.e.read(self.h, self.length)

    def clone(self) -> "T":
        return T.upload(self.rt, self.shape, self.to_host())

    detach = clone

    def dispose(self) -> None:
        if self.grad is not None:
            self.grad.dispose()
            self.grad = None
        if self.h is not None:
            self.rt.e.destroy(self.h)
            self.rt.live -= 8 * self.length
            self.h = None

    def __del__(self):                      # the Dart finalizer (tensor.dart: destroyTensorFinalizer)
        try:
            if self.h is not None:
                self.rt.e.destroy(self.h)
                self.rt.live -= 8 * self.length
                self.h = None
        except Exception:
            pass

    def assign(self, source: "T") -> None:  # tensor.dart:390-426: adopt the source's handle
        assert source.length == self.length
        self.rt.e.destroy(self.h)
        self.rt.live -= 8 * self.length
        self.h, source.h = source.h, None

    # -- autograd core (tensor.dart:539-668) ------------------------------------------------------------------------
    def _set_backward(self, children, fn: Callable[[], None]) -> None:
        if self.rt.no_grad > 0:
            return
        self.children, self.back, self.requires_grad = tuple(children), fn, True

    def _accumulate(self, contribution: "T") -> None:
        assert contribution.length == self.length, (self.shape, contribution.shape)
        if self.grad is None:
            self.grad = contribution
        else:
            summed = self.grad + contribution
            self.grad.dispose()
            contribution.dispose()
            self.grad = summed

    def zero_grad(self) -> None:
        if self.grad is not None:
            self.grad.dispose()
            self.grad = None

    def backward(self, free_graph: bool = True) -> None:
        if self.grad is None:
            self.grad = T.fill(self.rt, self.shape, 1.0)
        ordered: List[T] = []
        visited = set()
        stack = [(self, 0)]
        visited.add(id(self))
        while stack:                         # the recursive post-order walk of tensor.dart:549-559, without recursion
            node, i = stack.pop()
            if i < len(node.children):
                stack.append((node, i + 1))
                c = node.children[i]
                if id(c) not in visited:
                    visited.add(id(c))
                    stack.append((c, 0))
            else:
                ordered.append(node)
        # The Dart closures run with graph recording on, so temporaries made inside them carry closures of their own
        # that nothing ever calls and the garbage collector frees later.  Here they are made without closures, which
        # changes no library call and lets reference counting free them at once (less memory held, never more).
        for t in reversed(ordered):
            if t.back is not None:
                self.rt.no_grad += 1
                try:
                    t.back()
                finally:
                    self.rt.no_grad -= 1
            if free_graph and t is not self and t.back is not None:
                if t.grad is not None:
                    t.grad.dispose()
                    t.grad = None
                if t.h is not None:
                    t.dispose()
                t.children, t.back = (), None
        if free_graph:
            self.children, self.back = (), None

    @staticmethod
    def _reduce_for_broadcast(g: "T", target_shape) -> "T":
        n = _prod(target_shape)
        if g.length == n:
            return g
        if n == 1:
            s = g.sum()
            g.dispose()
            return s
        assert len(target_shape) == 2 and target_shape[0] == 1 and g.shape[1] == target_shape[1]
        host = g.to_host().reshape(g.shape[0], g.shape[1]).sum(axis=0, dtype=np.float32)  # host loop in the reference
        out = T.upload(g.rt, target_shape, host)
        g.dispose()
        return out

    # -- binary ops (ops.dart:26-285) --------------------------------------------------------------------------------
    def _binary(self, other, op: str) -> "T":
        rt = self.rt
        rt.calls += 1
        if isinstance(other, (int, float)):
            s = T.fill(rt, [1, 1], float(other))
            h = rt.e.call(f"{op}_tensor_scalar", self.h, s.h)
            s.dispose()
            return T(rt, self.shape, h)
        if self.length == other.length:
            return T(rt, self.shape, rt.e.call(f"{op}_tensors", self.h, other.h))
        if other.length == 1:
            return T(rt, self.shape, rt.e.call(f"{op}_tensor_scalar", self.h, other.h))
        if (op == "add" and len(self.shape) == 2 and len(other.shape) == 2 and other.shape[0] == 1
                and other.shape[1] == self.shape[1]):
            return T(rt, self.shape, rt.e.call("add_tensor_row_broadcast", self.h, other.h))
        raise ValueError(f"{op}: incompatible shapes {self.shape} vs {other.shape}")

    def __add__(self, o) -> "T":
        out = self._binary(o, "add")
        a = self
        if isinstance(o, (int, float)):
            if a.requires_grad:
                out._set_backward([a], lambda: a._accumulate(out.grad.clone()))
        elif a.requires_grad or o.requires_grad:
            b = o

            def fn():
                g = out.grad
                if a.requires_grad:
                    a._accumulate(T._reduce_for_broadcast(g.clone(), a.shape))
                if b.requires_grad:
                    b._accumulate(T._reduce_for_broadcast(g.clone(), b.shape))
            out._set_backward([a, b], fn)
        return out

    def __sub__(self, o) -> "T":
        out = self._binary(o, "sub")
        a = self
        if isinstance(o, (int, float)):
            if a.requires_grad:
                out._set_backward([a], lambda: a._accumulate(out.grad.clone()))
        elif a.requires_grad or o.requires_grad:
            b = o

            def fn():
                g = out.grad
                if a.requires_grad:
                    a._accumulate(T._reduce_for_broadcast(g.clone(), a.shape))
                if b.requires_grad:
                    b._accumulate(T._reduce_for_broadcast(g * -1.0, b.shape))
            out._set_backward([a, b], fn)
        return out

    def __mul__(self, o) -> "T":
        out = self._binary(o, "mul")
        a = self
        if isinstance(o, (int, float)):
            if a.requires_grad:
                s = float(o)
                out._set_backward([a], lambda: a._accumulate(out.grad * s))
        elif a.requires_grad or o.requires_grad:
            b = o

            def fn():
                g = out.grad
                if a.requires_grad:
                    a._accumulate(T._reduce_for_broadcast(g * b, a.shape))
                if b.requires_grad:
                    b._accumulate(T._reduce_for_broadcast(g * a, b.shape))
            out._set_backward([a, b], fn)
        return out

    def __truediv__(self, o) -> "T":
        out = self._binary(o, "div")
        a = self
        if isinstance(o, (int, float)):
            if a.requires_grad:
                s = float(o)
                out._set_backward([a], lambda: a._accumulate(out.grad / s))
        elif a.requires_grad or o.requires_grad:
            raise NotImplementedError("tensor / tensor gradients are not on the GPT training path")
        return out

    # -- unary / shape ops (ops.dart:333-352, 387-409, 458-497, 529-575) ---------------------------------------------
    def tanh(self) -> "T":
        self.rt.calls += 1
        out = T(self.rt, self.shape, self.rt.e.call("tanh_tensor", self.h))
        if self.requires_grad:
            x, y = self, out

            def fn():
                g = out.grad
                x._accumulate(g - g * y * y)
            out._set_backward([x], fn)
        return out

    def pow(self, exp: float) -> "T":
        self.rt.calls += 1
        out = T(self.rt, self.shape, self.rt.e.call("pow_tensor", self.h, float(exp)))
        if self.requires_grad:
            x = self
            out._set_backward([x], lambda: x._accumulate(out.grad * x.pow(exp - 1) * exp))
        return out

    def reshape(self, new_shape) -> "T":
        assert _prod(new_shape) == self.length
        out = T.upload(self.rt, list(new_shape), self.to_host())          # download + upload: ops.dart:465-470
        if self.requires_grad:
            x = self
            out._set_backward([x], lambda: x._accumulate(out.grad.reshape(x.shape)))
        return out

    def transpose(self) -> "T":
        r, c = self.shape
        self.rt.calls += 1
        out = T(self.rt, [c, r], self.rt.e.call("transpose_tensor", self.h))
        if self.requires_grad:
            x = self
            out._set_backward([x], lambda: x._accumulate(out.grad.transpose()))
        return out

    def sum(self) -> "T":
        self.rt.calls += 1
        out = T(self.rt, [1, 1], self.rt.e.call("sum_tensor", self.h))
        if self.requires_grad:
            x = self

            def fn():
                ones = T.fill(x.rt, x.shape, 1.0)
                x._accumulate(ones * out.grad)
            out._set_backward([x], fn)
        return out

    def mean(self) -> "T":
        self.rt.calls += 1
        out = T(self.rt, [1, 1], self.rt.e.call("mean_tensor", self.h))
        if self.requires_grad:
            x, n = self, float(self.length)

            def fn():
                ones = T.fill(x.rt, x.shape, 1.0)
                x._accumulate(ones * (out.grad / n))
            out._set_backward([x], fn)
        return out

    # -- matmul (mat_mul.dart:13-76) ---------------------------------------------------------------------------------
    def matmul(self, o: "T") -> "T":
        if len(self.shape) > 2 and len(o.shape) == 2:
            k, n = self.shape[-1], o.shape[1]
            return self.reshape([self.length // k, k]).matmul(o).reshape(self.shape[:-1] + [n])
        m, k = self.shape
        assert o.shape[0] == k
        self.rt.calls += 1
        out = T(self.rt, [m, o.shape[1]], self.rt.e.call("matmul_tensors", self.h, o.h))
        if self.requires_grad or o.requires_grad:
            a, b = self, o

            def fn():
                g = out.grad
                if a.requires_grad:
                    bt = b.transpose()
                    contrib = g.matmul(bt)
                    bt.dispose()
                    a._accumulate(contrib)
                if b.requires_grad:
                    at = a.transpose()
                    contrib = at.matmul(g)
                    at.dispose()
                    b._accumulate(contrib)
            out._set_backward([a, b], fn)
        return out

    # -- layer norm (layer_norm.dart:16-80, 170-201) -----------------------------------------------------------------
    def layer_norm(self, gamma: "T", beta: "T", eps: float = 1e-5) -> "T":
        if len(self.shape) > 2:
            cols = self.shape[-1]
            return self.reshape([self.length // cols, cols]).layer_norm(gamma, beta, eps).reshape(self.shape)
        rt = self.rt
        rt.calls += 1
        out = T(rt, self.shape, rt.e.call("layernorm_forward", self.h, gamma.h, beta.h, eps))
        x = self

        def fn():
            if gamma.grad is None:
                gamma.grad = T.fill(rt, gamma.shape, 0.0)
            if beta.grad is None:
                beta.grad = T.fill(rt, beta.shape, 0.0)
            rt.calls += 1
            gx = T(rt, x.shape, rt.e.call("layernorm_backward", x.h, gamma.h, out.grad.h, gamma.grad.h,
                                          beta.grad.h, eps))
            if x.requires_grad:
                x._accumulate(gx)
            else:
                gx.dispose()
        out._set_backward([x, gamma, beta], fn)
        return out

    # -- softmax / cross entropy (softmax.dart:23-56, 100-160) -------------------------------------------------------
    def softmax(self) -> "T":
        rt = self.rt
        rt.calls += 1
        out = T(rt, self.shape, rt.e.call("softmax_forward", self.h))
        if self.requires_grad:
            x = self

            def fn():
                rt.calls += 1
                x._accumulate(T(rt, x.shape, rt.e.call("softmax_backward", out.h, out.grad.h)))
            out._set_backward([x], fn)
        return out

    def cross_entropy(self, targets: "T") -> "T":
        if len(self.shape) > 2:
            v = self.shape[-1]
            n = self.length // v
            return self.reshape([n, v]).cross_entropy(targets.reshape([n]))
        rt = self.rt
        rt.calls += 1
        loss = T(rt, [self.shape[0], 1], rt.e.call("cross_entropy_forward", self.h, targets.h))
        if self.requires_grad:
            x = self

            def fn():
                rt.calls += 1
                x._accumulate(T(rt, x.shape, rt.e.call("cross_entropy_backward", x.h, targets.h, loss.grad.h)))
            loss._set_backward([x], fn)
        return loss

    # -- embedding (embedding.dart:29-140) ---------------------------------------------------------------------------
    def embedding(self, indices: "T") -> "T":
        if len(indices.shape) > 1:
            return self.embedding(indices.reshape([indices.length])).reshape(indices.shape + [self.shape[1]])
        rt, n, table = self.rt, indices.length, self
        rt.calls += 1
        out = T(rt, [n, self.shape[1]], rt.e.call("embedding_forward", self.h, indices.h, n))
        if self.requires_grad:
            def fn():
                if table.grad is None:
                    table.grad = T.fill(rt, table.shape, 0.0)
                rt.calls += 1
                rt.e.call("embedding_backward", indices.h, out.grad.h, table.grad.h, n)
            out._set_backward([table], fn)
        return out

    # -- attention (attention.dart:18-59) ----------------------------------------------------------------------------
    def sdpa(self, k: "T", v: "T", mask: Optional["T"]) -> "T":
        scores = self.matmul(k.transpose()) * (1.0 / math.sqrt(self.shape[1]))
        if mask is not None:
            scores = scores + mask
        return scores.softmax().matmul(v)


def concat(tensors: List[T], axis: int) -> T:
    """concat.dart:14-147: download every input, splice on the host, upload; backward slices on the host."""
    rt = tensors[0].rt
    host = [t.to_host().reshape(t.shape) for t in tensors]
    out_host = np.concatenate(host, axis=axis)
    any_req = any(t.requires_grad for t in tensors)
    out = T.upload(rt, list(out_host.shape), out_host, requires_grad=any_req)
    if any_req:
        def fn():
            g = out.grad.to_host().reshape(out.shape)
            off = 0
            for t in tensors:
                n = t.shape[axis]
                if t.requires_grad:
                    sl = g[:, off:off + n] if axis == 1 else g[off:off + n]
                    t._accumulate(T.upload(rt, t.shape, np.ascontiguousarray(sl)))
                off += n
        out._set_backward(tensors, fn)
    return out


def split_rows(t: T, chunk: int) -> List[T]:
    """concat.dart:150-200: one download, one upload per chunk; each chunk's backward uploads a full-size, mostly
    zero gradient of the source."""
    rt = t.rt
    r, c = t.shape
    src = t.to_host().reshape(r, c)
    chunks = []
    for i in range(r // chunk):
        ch = T.upload(rt, [chunk, c], np.ascontiguousarray(src[i * chunk:(i + 1) * chunk]))
        if t.requires_grad:
            def fn(ch=ch, off=i * chunk):
                g = ch.grad.to_host().reshape(chunk, c)
                full = np.zeros((r, c), dtype=np.float32)
                full[off:off + chunk] = g
                t._accumulate(T.upload(rt, t.shape, full))
            ch._set_backward([t], fn)
        chunks.append(ch)
    return chunks


# ---------------------------------------------------------------------------------------------------------------------
# nn modules (lib/core/nn/*.dart)
# ---------------------------------------------------------------------------------------------------------------------

class Linear:
    def __init__(self, rt, rng, fin, fout, bias=True, std=0.02):
        self.weight = T.upload(rt, [fout, fin], rng.normal(0.0, std, fout * fin).astype(np.float32), True)
        self.bias = T.upload(rt, [1, fout], np.zeros(fout, np.float32), True) if bias else None
        self.fin, self.fout = fin, fout

    def __call__(self, x: T) -> T:
        if len(x.shape) > 2:
            flat = x.reshape([x.length // self.fin, self.fin])
            y = flat.matmul(self.weight.transpose())
            if self.bias is not None:
                y = y + self.bias
            return y.reshape(x.shape[:-1] + [self.fout])
        y = x.matmul(self.weight.transpose())
        return y + self.bias if self.bias is not None else y

    def parameters(self):
        return [self.weight] if self.bias is None else [self.weight, self.bias]


class LayerNorm:
    def __init__(self, rt, dim, eps=1e-5):
        self.gamma, self.beta, self.eps = T.fill(rt, [dim], 1.0, True), T.fill(rt, [dim], 0.0, True), eps

    def __call__(self, x):
        return x.layer_norm(self.gamma, self.beta, self.eps)

    def parameters(self):
        return [self.gamma, self.beta]


class MultiHeadAttention:
    """Per-head Linear projections and the batched path of attention/multi_head_attention.dart:203-235."""

    def __init__(self, rt, rng, dim, heads, bias=True):
        self.h, self.hd, self.dim = heads, dim // heads, dim
        self.wq = [Linear(rt, rng, dim, self.hd, bias) for _ in range(heads)]
        self.wk = [Linear(rt, rng, dim, self.hd, bias) for _ in range(heads)]
        self.wv = [Linear(rt, rng, dim, self.hd, bias) for _ in range(heads)]
        self.wo = Linear(rt, rng, dim, dim, True)

    def __call__(self, x: T, mask: Optional[T]) -> T:
        b, s = x.shape[0], x.shape[1]
        heads = []
        for h in range(self.h):
            q, k, v = self.wq[h](x), self.wk[h](x), self.wv[h](x)
            qs = split_rows(q.reshape([b * s, self.hd]), s)
            ks = split_rows(k.reshape([b * s, self.hd]), s)
            vs = split_rows(v.reshape([b * s, self.hd]), s)
            per_batch = [qs[i].sdpa(ks[i], vs[i], mask) for i in range(b)]
            heads.append(concat(per_batch, axis=0))
        cat = concat(heads, axis=1)
        return self.wo(cat.reshape([b, s, self.dim]))

    def parameters(self):
        ps = []
        for group in (self.wq, self.wk, self.wv):
            for l in group:
                ps += l.parameters()
        return ps + self.wo.parameters()


class TransformerBlock:
    """Pre-LN block, tanh GELU out of elementwise ops (transformer.dart:81-102); dropout p = 0 is the identity."""

    def __init__(self, rt, rng, dim, heads):
        self.ln1, self.ln2 = LayerNorm(rt, dim), LayerNorm(rt, dim)
        self.mha = MultiHeadAttention(rt, rng, dim, heads)
        self.ffn1, self.ffn2 = Linear(rt, rng, dim, 4 * dim), Linear(rt, rng, 4 * dim, dim)

    def __call__(self, x, mask):
        h = x + self.mha(self.ln1(x), mask)
        inner = self.ffn1(self.ln2(h))
        t = ((inner + inner.pow(3.0) * 0.044715) * 0.7978845608028654).tanh()
        act = inner * (t + 1.0) * 0.5
        return h + self.ffn2(act)

    def parameters(self):
        return (self.ln1.parameters() + self.ln2.parameters() + self.mha.parameters() + self.ffn1.parameters()
                + self.ffn2.parameters())


class GPT:
    """Weight-tied GPT with learned positions (gpt.dart:60-167, positional.dart:88-111, transformer_encoder.dart)."""

    def __init__(self, rt, vocab, ctx, dim, layers, heads, seed=0):
        rng = np.random.default_rng(seed)
        self.rt, self.ctx = rt, ctx
        self.wte = T.upload(rt, [vocab, dim], rng.normal(0.0, 0.02, vocab * dim).astype(np.float32), True)
        self.wpe = T.upload(rt, [ctx, dim], rng.normal(0.0, 0.02, ctx * dim).astype(np.float32), True)
        self.blocks = [TransformerBlock(rt, rng, dim, heads) for _ in range(layers)]
        self.final_norm = LayerNorm(rt, dim)

    def __call__(self, tokens: T) -> T:
        b, s = tokens.shape
        h = self.wte.embedding(tokens)
        positions = T.upload(self.rt, [b, s], np.tile(np.arange(s, dtype=np.float32), b))
        h = h + self.wpe.embedding(positions)
        mask = None
        if s > 1:
            m = np.triu(np.full((s, s), -1e9, dtype=np.float32), k=1)
            mask = T.upload(self.rt, [s, s], m)
        for blk in self.blocks:
            h = blk(h, mask)
        h = self.final_norm(h)
        return h.matmul(self.wte.transpose())

    def parameters(self):
        ps = [self.wte, self.wpe]
        for blk in self.blocks:
            ps += blk.parameters()
        return ps + self.final_norm.parameters()


# ---------------------------------------------------------------------------------------------------------------------
# Optimiser, clipping, schedule (lib/core/optim/*.dart)
# ---------------------------------------------------------------------------------------------------------------------

class Adam:
    def __init__(self, params, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
        self.params, self.lr, self.b1, self.b2, self.eps, self.wd = params, lr, beta1, beta2, eps, weight_decay
        self.t = 0
        self.m = [None] * len(params)
        self.v = [None] * len(params)

    def zero_grad(self):
        for p in self.params:
            p.zero_grad()

    def step(self):
        self.t += 1
        bc1, bc2 = 1.0 - self.b1 ** self.t, 1.0 - self.b2 ** self.t
        for i, p in enumerate(self.params):
            g = p.grad
            if g is None:
                continue
            if self.m[i] is None:
                self.m[i] = T.fill(p.rt, p.shape, 0.0)
                self.v[i] = T.fill(p.rt, p.shape, 0.0)
            m, v = self.m[i], self.v[i]
            m_beta = m * self.b1
            g1 = g * (1.0 - self.b1)
            m_sum = m_beta + g1
            m_beta.dispose(); g1.dispose()
            m.assign(m_sum)
            v_beta = v * self.b2
            g_sq = g * g
            g_sq_s = g_sq * (1.0 - self.b2)
            g_sq.dispose()
            v_sum = v_beta + g_sq_s
            v_beta.dispose(); g_sq_s.dispose()
            v.assign(v_sum)
            m_hat = m / bc1
            v_hat = v / bc2
            sqrt_v = v_hat.pow(0.5)
            v_hat.dispose()
            denom = sqrt_v + self.eps
            sqrt_v.dispose()
            ratio = m_hat / denom
            m_hat.dispose(); denom.dispose()
            update = ratio * self.lr
            ratio.dispose()
            if self.wd != 0.0:
                p_det = p.detach()
                wd = p_det * (self.lr * self.wd)
                p_det.dispose()
                new_update = update + wd
                update.dispose(); wd.dispose()
                update = new_update
            p_det = p.detach()
            new_p = p_det - update
            p_det.dispose(); update.dispose()
            p.assign(new_p)


def clip_grad_norm(params, max_norm: float) -> float:
    """optim/grad_utils.dart:7-40: the norm is summed on the host from downloaded gradients."""
    sum_sq = 0.0
    for p in params:
        if p.grad is not None:
            g = p.grad.to_host().astype(np.float64)
            sum_sq += float(np.dot(g, g))
    total = math.sqrt(sum_sq)
    if total <= max_norm or total == 0.0 or not math.isfinite(total):
        return total
    scale = max_norm / total
    for p in params:
        if p.grad is not None:
            p.grad.assign(p.grad * scale)
    return total


def lr_at(step, warmup, total, max_lr, min_lr):
    """optim/lr_scheduler.dart:82-92."""
    if step <= 0:
        return 0.0
    if step <= warmup:
        return max_lr if warmup == 0 else max_lr * step / warmup
    if step >= total:
        return min_lr
    prog = (step - warmup) / (total - warmup)
    return min_lr + 0.5 * (max_lr - min_lr) * (1.0 + math.cos(math.pi * prog))


# ---------------------------------------------------------------------------------------------------------------------
# One training step, as bin/gpt_train.dart:111-131 runs it
# ---------------------------------------------------------------------------------------------------------------------

class TrainState:
    def __init__(self, rt: Runtime, cfg: dict, lr=6e-4, weight_decay=0.1, warmup=100, total=1000):
        self.rt = rt
        self.model = GPT(rt, cfg["vocab_size"], cfg["max_ctx"], cfg["embed_dim"], cfg["num_layers"], cfg["num_heads"])
        self.params = self.model.parameters()
        self.opt = Adam(self.params, lr, 0.9, 0.95, 1e-8, weight_decay)
        self.sched = (warmup, total, lr, lr / 10)
        self.step_no = 0
        self.opt.lr = lr_at(1, *self.sched)

    def step(self, x: np.ndarray, y: np.ndarray, micro: int) -> float:
        """x, y: [B, S] token ids (host).  ``micro`` sequences per forward/backward pass; the gradients of the passes
        accumulate, each pass's loss is scaled by its share of the batch, then clip + Adam once."""
        rt = self.rt
        self.opt.zero_grad()
        b = x.shape[0]
        total_loss = 0.0
        for lo in range(0, b, micro):
            xs, ys = x[lo:lo + micro], y[lo:lo + micro]
            xt = T.upload(rt, list(xs.shape), xs.astype(np.float32))
            yt = T.upload(rt, list(ys.shape), ys.astype(np.float32))
            loss = self.model(xt).cross_entropy(yt).mean()
            if micro < b:
                loss = loss * (xs.shape[0] / b)
            loss.backward()
            total_loss += float(loss.to_host()[0])
            loss.dispose()
        clip_grad_norm(self.params, 1.0)
        self.opt.step()
        self.step_no += 1
        self.opt.lr = lr_at(self.step_no + 1, *self.sched)
        return total_loss


def plan_micro_batch(cfg: dict, batch: int, seq: int, budget_bytes: float):
    """Peak of live library bytes for one step, from a dry run on the shape-only engine with the model's layer count
    reduced to 1 and 2 (the peak is affine in the layer count and in the micro-batch), extrapolated to the real
    model; returns the largest power-of-two micro-batch <= ``batch`` that stays under ``budget_bytes`` and the
    predicted peaks."""
    def peak(layers, micro):
        rt = Runtime(ShapeEngine())
        small = dict(cfg, num_layers=layers)
        st = TrainState(rt, small)
        tok = np.zeros((micro, seq), dtype=np.int64)
        st.step(tok, tok, micro)
        return rt.peak

    p11, p21, p12 = peak(1, 1), peak(2, 1), peak(1, 2)
    per_layer_1 = p21 - p11
    p22 = peak(2, 2)
    per_layer_2 = p22 - p12
    L = cfg["num_layers"]

    def predict(micro):
        # affine in micro from the two measured points, at the real layer count
        at1 = p11 + (L - 1) * per_layer_1
        at2 = p12 + (L - 1) * per_layer_2
        return at1 + (micro - 1) * (at2 - at1)

    micro = batch
    while micro > 1 and predict(micro) > budget_bytes:
        micro //= 2
    return micro, {m: predict(m) for m in sorted({1, 2, 4, 8, batch})}


def run(args, metric, model_cfg, seq, clock_sampler_cls=None):
    def say(obj):
        obj.update({"impl": "reference", "metric": metric, "n_gpus": args.gpus})
        print(json.dumps(obj))

    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            say({"unavailable": "the reference has no multi-GPU path (single device, no NCCL build)"})
        return
    if not os.path.exists(LIB_PATH):
        say({"unavailable": f"{os.path.relpath(LIB_PATH, os.path.dirname(HERE))} is missing: the reference's native "
                            "library was not built (python -m baseline.reference_native --build <reference root>)"})
        return
    import torch  # CUDA events, memory query and the pinned staging buffers only; no torch op runs on this path
    if not torch.cuda.is_available():
        say({"unavailable": "no CUDA device"})
        return

    torch.cuda.set_device(0)
    free_b, total_b = torch.cuda.mem_get_info()
    batch = args.batch
    micro, predicted = plan_micro_batch(model_cfg, batch, seq, 0.80 * free_b)
    rt = Runtime(CudaEngine())
    st = TrainState(rt, model_cfg, total=max(1000, args.steps + args.warmup))

    # wall-clock allowance: the composed step takes tens of seconds, so the step counts asked for are cut to fit
    allowance = float(os.environ.get("DPTB200_REF_SECONDS", "420"))
    g = torch.Generator().manual_seed(1234)
    n_batches = args.warmup + args.steps
    xs = torch.randint(0, model_cfg["vocab_size"], (n_batches, batch, seq + 1), generator=g, dtype=torch.long)
    hx = xs[:, :, :-1].contiguous().pin_memory()
    hy = xs[:, :, 1:].contiguous().pin_memory()

    # Warm-up.  One full step of this arm takes minutes, so by default the context, the library's kernels and the
    # host paths are warmed by one step of a one-layer, 64-token model of the same code, and full-size warm-up steps
    # run only while they fit in a quarter of the allowance (``--warmup`` is an upper bound).
    t_begin = time.perf_counter()
    tiny_rt = Runtime(CudaEngine())
    tiny = TrainState(tiny_rt, dict(model_cfg, num_layers=1, max_ctx=64))
    tok = np.random.default_rng(0).integers(0, model_cfg["vocab_size"], (2, 64))
    tiny.step(tok, tok, 2)
    del tiny, tiny_rt
    torch.cuda.synchronize()
    per_step_guess = float(os.environ.get("DPTB200_REF_STEP_SECONDS", "240"))
    warm_done, loss = 0, float("nan")
    for i in range(args.warmup):
        if (time.perf_counter() - t_begin) + per_step_guess > 0.25 * allowance:
            break
        t_w = time.perf_counter()
        loss = st.step(hx[i].numpy(), hy[i].numpy(), micro)
        per_step_guess = time.perf_counter() - t_w
        warm_done += 1
    first_loss = loss
    torch.cuda.synchronize()

    sampler = clock_sampler_cls(0) if clock_sampler_cls is not None else None
    if sampler is not None:
        sampler.start()
    calls0, h2d0, d2h0 = rt.calls, rt.h2d, rt.d2h
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0.record()
    done = 0
    for i in range(args.steps):
        t_s = time.perf_counter()
        loss = st.step(hx[args.warmup + i].numpy(), hy[args.warmup + i].numpy(), micro)   # H2D of tokens, D2H of loss
        per_step_guess = time.perf_counter() - t_s
        done += 1
        if math.isnan(first_loss):
            first_loss = loss
        if (time.perf_counter() - t_begin) + per_step_guess > allowance:
            break
    e1.record()
    torch.cuda.synchronize()
    ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3)
    clocks = sampler.stop() if sampler is not None else None
    tokens = batch * seq * done
    value = tokens / (ms / 1e3)
    say({
        "value": value, "unit": "tokens/s", "steps": done, "warmup": warm_done, "steps_requested": args.steps,
        "warmup_requested": args.warmup, "ms_per_step": ms / done, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"model": "gpt2-124m", "global_batch": batch, "seq_len": seq, "parallelism": "dp1",
                   "optimizer": "adamw lr6e-4 wd0.1 clip1.0 warmup-cosine",
                   "micro_batch_per_pass": micro, "passes_per_step": (batch + micro - 1) // micro,
                   "why_split": "the library allocates data + grad per handle; one 16 x 1024 graph needs "
                                f"{predicted[batch] / 2**30:.0f} GiB, predicted peak at the chosen split "
                                f"{predicted.get(micro, 0) / 2**30:.0f} GiB of {total_b / 2**30:.0f} GiB",
                   "precision_note": "fp32 is the only precision the reference library has",
                   "path": "unmodified lib/native/src/engine.cu entry points, composed along bin/gpt_train.dart",
                   "steps_cut_to_fit_seconds": allowance,
                   "warmup_note": "one step of a 1-layer, 64-token model of the same code warms the context and "
                                  "kernels; full-size warm-up steps only while they fit a quarter of the allowance",
                   "cache_policy": "per-step working set far exceeds the 126 MB L2"},
        "clocks": clocks,
        # the reference's step is synchronous and feeds from host memory every step: its only number is end to end
        "e2e": {"value": value, "unit": "tokens/s", "ms_per_step": ms / done,
                "h2d_bytes_per_step": int((rt.h2d - h2d0) / done), "d2h_bytes_per_step": int((rt.d2h - d2h0) / done)},
        "gpu_launches": int(rt.calls - calls0),
        "peak_library_bytes": int(rt.peak),
        "loss_first": first_loss, "loss_last": loss,
    })
