"""Global-norm gradient clipping (reference: lib/core/optim/grad_utils.dart:14-48).

Rules kept from the reference: the norm is the L2 norm over all non-null gradients; nothing is scaled when the norm is
zero, within ``max_norm`` or not finite; ``scale = max_norm / norm`` (no epsilon); ``max_norm <= 0`` raises; the
pre-clip norm is returned.

On a device arena the norm is a two-stage deterministic reduction over the flat gradient buffer and the clip
coefficient stays in device memory: the next optimizer step multiplies gradients by it inside its own kernel, so
clipping costs one read of the gradients and no host round trip.  The returned ``LazyScalar`` only synchronises when
it is converted to a float.  Pass ``materialize=True`` to also scale ``.grad`` in place."""
from __future__ import annotations

import math
from typing import Sequence

import torch


class LazyScalar:
    """A device scalar that converts to ``float`` on demand (that conversion is the only synchronisation)."""

    def __init__(self, tensor: torch.Tensor, index: int = 0):
        self._t, self._i = tensor, index

    def tensor(self) -> torch.Tensor:
        return self._t[self._i]

    def __float__(self) -> float:
        return float(self._t[self._i].item())

    def item(self) -> float:
        return float(self)

    def __repr__(self):
        return f"LazyScalar({float(self):.6g})"

    def __format__(self, spec):
        return format(float(self), spec)


def clip_grad_norm(parameters: Sequence[torch.Tensor], max_norm: float, materialize: bool = False):
    if max_norm <= 0:
        raise ValueError("clipGradNorm: maxNorm must be > 0")
    params = list(parameters.parameters) if hasattr(parameters, "arena") else list(parameters)
    arena = getattr(params[0], "_dptb_arena", None) if params else None
    if arena is not None and all(getattr(p, "_dptb_arena", None) is arena for p in params) \
            and len(params) == len(arena.params) and getattr(arena, "optimizer", None) is not None:
        from ..ops import kernels as K
        opt = arena.optimizer
        K.grad_norm(arena.grad, opt.ctrl, float(max_norm))
        if materialize:
            K.scale_by_ctrl(arena.grad, opt.ctrl)
            opt.clip_pending = False
        else:
            opt.clip_pending = True
        return LazyScalar(opt.ctrl, 0)
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return 0.0
    with torch.no_grad():
        # per-tensor norms in one list op, combined in double precision with a single host read
        norms = torch.stack([n.double() for n in torch._foreach_norm(grads, 2)])
        total = float(torch.sqrt((norms * norms).sum()))
        if total == 0.0 or not math.isfinite(total) or total <= max_norm:
            return total
        torch._foreach_mul_(grads, max_norm / total)
    return total


clipGradNorm = clip_grad_norm
