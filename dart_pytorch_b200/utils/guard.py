"""Canary-padded buffers: catch a kernel that writes outside the tensor it was given.

The reference defends against silent corruption with bounds checks inside every kernel and an allocation guard added
after one such bug (reference: lib/native/src/engine.cu:33-49, lib/native/src/kernels/embedding.cuh:24-29).  The
kernels here take raw pointers, leading dimensions and extents, so the host-side equivalent of a memory checker is
cheap: allocate the output with a pad of known bit patterns on both sides, run the kernel on the payload view, and
verify afterwards that the pads still hold the pattern.  Used by the GPU tests on odd shapes (tails, rows below a
tile, padded leading dimensions); works for CPU tensors too.
"""
from __future__ import annotations

import contextlib
from typing import List, Sequence

import torch


class GuardError(AssertionError):
    pass


def _numel(shape: Sequence[int]) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class GuardedBuffer:
    """A contiguous tensor of ``shape`` inside a larger allocation: ``pad_elems`` canary elements before and after.

    ``tensor`` is the payload view to hand to a kernel (its data pointer keeps the alignment of the allocation when
    ``pad_elems * itemsize`` is a multiple of it; the default pad of 64 elements keeps 16-byte alignment for every
    dtype of two bytes or more).  ``check()`` raises ``GuardError`` naming the side and the first damaged offset."""

    def __init__(self, shape, dtype, device, pad_elems: int = 64):
        self.shape, self.dtype, self.pad_elems = tuple(int(s) for s in shape), dtype, int(pad_elems)
        n = _numel(self.shape)
        self.storage = torch.empty(n + 2 * self.pad_elems, dtype=dtype, device=device)
        self._pattern = self._make_pattern(self.pad_elems, dtype, device)
        self.tensor = self.storage[self.pad_elems:self.pad_elems + n].view(self.shape)
        self.rearm()

    @staticmethod
    def _make_pattern(n: int, dtype, device):
        # distinct neighbouring values, exactly representable in every supported dtype, never produced by a zero fill
        base = (torch.arange(n, device=device) % 13 + 3)
        return base.to(dtype) if dtype != torch.bool else (base % 2 == 0)

    def rearm(self) -> None:
        self.storage[:self.pad_elems] = self._pattern
        self.storage[self.storage.numel() - self.pad_elems:] = self._pattern

    def check(self, what: str = "") -> None:
        head = self.storage[:self.pad_elems]
        tail = self.storage[self.storage.numel() - self.pad_elems:]
        for side, part in (("before", head), ("after", tail)):
            bad = (part != self._pattern).nonzero()
            if bad.numel():
                i = int(bad[0])
                off = i - self.pad_elems if side == "before" else i
                raise GuardError(f"{what or 'buffer'} {self.shape} {self.dtype}: canary {side} the payload damaged at "
                                 f"element offset {off} ({int(bad.numel())} elements in all)")


class GuardPool:
    def __init__(self, pad_elems: int = 64):
        self.pad_elems, self.buffers, self.checked = pad_elems, [], 0

    def empty(self, shape, dtype, device) -> torch.Tensor:
        g = GuardedBuffer(shape, dtype, device, self.pad_elems)
        self.buffers.append(g)
        return g.tensor

    def check(self, what: str = "") -> None:
        for g in self.buffers:
            g.check(what)
            self.checked += 1


@contextlib.contextmanager
def guarded(pad_elems: int = 64):
    """``with guarded() as pool: out = pool.empty(...); kernel(..., out)``: every buffer is checked on exit."""
    pool = GuardPool(pad_elems)
    yield pool
    if pool.buffers and pool.buffers[0].storage.is_cuda:
        torch.cuda.synchronize()
    pool.check()
