"""Module base class and parameter helpers.

Same contract as the reference's ``Module`` (lib/core/nn/module.dart:10-46): a ``training`` flag toggled recursively
through ``submodules()``, an ordered ``parameters()`` list, ``zeroGrad()``; modules are callables.  Two additions serve
the device path:

* ``parameters()`` returns the *storage* leaves the optimizer updates (for example one fused QKV weight), while
  ``reference_parameters()`` returns views of the same storage in the reference's checkpoint order and shapes (per-head
  ``[hd, D]`` projections, ``[1, out]`` biases), which is what the DPTC reader / writer walks.
* ``to(device, dtype)`` moves every leaf in place, keeping tensor identity (optimizer state stays valid).
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch


def make_param(t: torch.Tensor) -> torch.Tensor:
    t = t.detach().clone()
    t.requires_grad_(True)
    return t


def seeded_generator(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed) & 0x7FFFFFFFFFFFFFFF)
    return g


def uniform_(shape, bound: float, seed: int, device=None, dtype=torch.float32) -> torch.Tensor:
    g = seeded_generator(seed)
    t = (torch.rand(*shape, generator=g, dtype=torch.float32) * 2.0 - 1.0) * bound
    return t.to(device=device, dtype=dtype)


def normal_(shape, std: float, seed: int, device=None, dtype=torch.float32) -> torch.Tensor:
    g = seeded_generator(seed)
    t = torch.randn(*shape, generator=g, dtype=torch.float32) * std
    return t.to(device=device, dtype=dtype)


class Module:
    def __init__(self):
        self.training = True

    # ---- structure -------------------------------------------------------------------------------
    def submodules(self) -> List["Module"]:
        return []

    def own_parameters(self) -> List[torch.Tensor]:
        """Storage leaves held directly by this module (not by its submodules)."""
        return []

    def own_reference_parameters(self) -> List[torch.Tensor]:
        """Checkpoint-order views of this module's own storage; default: the leaves themselves."""
        return [p.data for p in self.own_parameters()]

    def parameters(self) -> List[torch.Tensor]:
        out, seen = [], set()
        for p in self._walk_params(False):
            if id(p) not in seen:
                seen.add(id(p))
                out.append(p)
        return out

    def reference_parameters(self) -> List[torch.Tensor]:
        """Detached views in the reference's ``parameters()`` order; tied tensors appear once."""
        out, seen = [], set()
        for p in self._walk_params(True):
            key = (p.data_ptr(), tuple(p.shape), tuple(p.stride()))
            if key not in seen:
                seen.add(key)
                out.append(p)
        return out

    def _walk_params(self, reference: bool) -> Iterable[torch.Tensor]:
        yield from (self.own_reference_parameters() if reference else self.own_parameters())
        for m in self.submodules():
            yield from m._walk_params(reference)

    # ---- modes -----------------------------------------------------------------------------------
    def train(self) -> "Module":
        self.training = True
        for m in self.submodules():
            m.train()
        return self

    def eval(self) -> "Module":
        self.training = False
        for m in self.submodules():
            m.eval()
        return self

    def zero_grad(self) -> None:
        for p in self.parameters():
            if p.grad is not None and getattr(p, "_dptb_direct_grad", False):
                p.grad.zero_()
            else:
                p.grad = None

    zeroGrad = zero_grad

    # ---- placement -------------------------------------------------------------------------------
    def to(self, device=None, dtype: Optional[torch.dtype] = None) -> "Module":
        for p in self.parameters():
            new = p.data.to(device=device if device is not None else p.device,
                            dtype=dtype if (dtype is not None and p.is_floating_point()) else p.dtype)
            p.data = new
            p.grad = None
        for m in self.modules():
            m._moved(device, dtype)
        return self

    def _moved(self, device, dtype) -> None:
        """Hook for modules that hold non-parameter tensors."""

    def modules(self) -> List["Module"]:
        out = [self]
        for m in self.submodules():
            out.extend(m.modules())
        return out

    def cuda(self, dtype: Optional[torch.dtype] = None) -> "Module":
        return self.to("cuda", dtype)

    @property
    def device(self) -> torch.device:
        ps = self.parameters()
        return ps[0].device if ps else torch.device("cpu")

    @property
    def dtype(self) -> torch.dtype:
        ps = self.parameters()
        return ps[0].dtype if ps else torch.float32

    def num_scalars(self) -> int:
        return sum(p.numel() for p in self.parameters())

    # ---- call ------------------------------------------------------------------------------------
    def forward(self, *args, **kwargs):
        raise NotImplementedError

    def __call__(self, *args, **kwargs):
        from ..tensor import unwrap_args, wrap_like
        wrapped, args, kwargs = unwrap_args(args, kwargs)
        out = self.forward(*args, **kwargs)
        return wrap_like(out) if wrapped else out

    call = __call__
