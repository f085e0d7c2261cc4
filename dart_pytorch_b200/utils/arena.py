"""ParamArena: all parameters of a model re-homed into flat, contiguous device buffers.

The reference updates each parameter with its own chain of elementwise ops and reads every gradient back to the host
for clipping (lib/core/optim/adam.dart:41-111, lib/core/optim/grad_utils.dart:14-48).  With one flat range per model:

* the optimizer, the gradient-norm reduction and gradient zeroing are each ONE kernel over the range;
* every ``p.grad`` is a view of one flat gradient buffer that the backward kernels accumulate into directly
  (``p._dptb_direct_grad``), so the weight-gradient GEMMs write their results where the optimizer reads them;
* data-parallel buckets are contiguous slices of that buffer;
* fp32 master weights sit beside the bf16 working copies the forward reads (``master`` is what checkpoints save).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

ALIGN = 128  # elements; keeps every parameter 256-byte aligned in bf16 (TMA needs 16-byte bases)


class ParamArena:
    def __init__(self, params: Sequence[torch.Tensor], grad_dtype: Optional[torch.dtype] = None,
                 master: Optional[bool] = None, reverse_order: bool = True):
        """``reverse_order`` lays parameters out in reverse of ``params``: gradients then become final front-to-back in
        the order the backward produces them, which is what bucketed reduction wants."""
        params = [p for p in params]
        if not params:
            raise ValueError("ParamArena: no parameters")
        dev, dt = params[0].device, params[0].dtype
        for p in params:
            if p.device != dev or p.dtype != dt:
                raise ValueError("ParamArena: parameters must share device and dtype")
        self.params: List[torch.Tensor] = params
        order = list(reversed(params)) if reverse_order else params
        self.offsets = {}
        off = 0
        for p in order:
            self.offsets[id(p)] = off
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        self.numel = off
        self.device, self.dtype = dev, dt
        self.grad_dtype = grad_dtype or dt
        self.flat = torch.zeros(off, dtype=dt, device=dev)
        self.grad = torch.zeros(off, dtype=self.grad_dtype, device=dev)
        want_master = (dt != torch.float32) if master is None else master
        self.master = torch.zeros(off, dtype=torch.float32, device=dev) if want_master else None
        direct = dev.type == "cuda" and self.grad_dtype == dt
        with torch.no_grad():
            for p in params:
                o, n = self.offsets[id(p)], p.numel()
                view = self.flat[o:o + n].view(p.shape)
                view.copy_(p.data)
                if self.master is not None:
                    src = getattr(p, "_dptb_master_init", None)
                    self.master[o:o + n].copy_((src if src is not None else p.data).reshape(-1).float())
                p.data = view
                p.grad = self.grad[o:o + n].view(p.shape) if self.grad_dtype == dt else None
                p._dptb_direct_grad = direct
                p._dptb_arena = self
        self.ordered = order

    def master_view(self, p: torch.Tensor) -> torch.Tensor:
        """fp32 master values of ``p`` (the parameter itself when no master copy is kept)."""
        o, n = self.offsets[id(p)], p.numel()
        src = self.master if self.master is not None else self.flat
        return src[o:o + n].view(p.shape)

    def zero_grad(self) -> None:
        self.grad.zero_()

    def sync_from_params(self) -> None:
        """After parameter values were overwritten (checkpoint load): refresh the master copy."""
        if self.master is not None:
            self.master.copy_(self.flat.float())

    def sync_to_params(self) -> None:
        if self.master is not None:
            self.flat.copy_(self.master.to(self.dtype))

    def slices(self, bucket_elems: int, exclude=()):
        """Contiguous ``(start, end)`` ranges of about ``bucket_elems`` elements that respect parameter boundaries.
        Parameters in ``exclude`` (compared by identity) are left out: a range ends before one and the next starts
        after it."""
        skip = {id(p) for p in exclude}
        out, start, cur = [], 0, 0
        for p in self.ordered:
            n = (p.numel() + ALIGN - 1) // ALIGN * ALIGN
            if id(p) in skip:
                if cur > start:
                    out.append((start, cur))
                cur += n
                start = cur
                continue
            cur += n
            if cur - start >= bucket_elems:
                out.append((start, cur))
                start = cur
        if cur > start:
            out.append((start, cur))
        return out

    def ranges_of(self, params):
        """Merged ``(start, end)`` element ranges covered by ``params``."""
        spans = sorted((self.offsets[id(p)], self.offsets[id(p)] + (p.numel() + ALIGN - 1) // ALIGN * ALIGN)
                       for p in params)
        out = []
        for s, e in spans:
            if out and out[-1][1] == s:
                out[-1] = (out[-1][0], e)
            else:
                out.append((s, e))
        return out
