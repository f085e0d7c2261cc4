"""Data-parallel gradient reduction over the flat gradient arena.

The reference has no synchronous data parallelism: its "distributed" mode averages whole checkpoints every K local
steps over HTTP (lib/core/coop/param_avg.dart:20-123).  Here every rank holds a replica, gradients live in one flat
bf16 buffer (``utils/arena.py``) and are averaged across ranks between backward and clip.

``GradReducer(mode="nccl")`` is the library baseline: one ``all_reduce`` per bucket on a side stream.
``GradReducer(mode="fused")`` runs this package's own kernel per bucket (``csrc/dp_allreduce.cu``): peer / multimem
loads and stores over NVSwitch from inside the kernel, fused with the sum-of-squares partials that clipping needs.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class GradReducer:
    def __init__(self, arena, world_size: int, mode: str = "auto", bucket_mb: float = 32.0, group=None):
        self.arena, self.world = arena, world_size
        self.group = group
        self.mode = mode
        self.bucket_elems = int(bucket_mb * 1024 * 1024 / arena.grad.element_size())
        self.buckets = arena.slices(self.bucket_elems)
        self.impl = None
        if mode in ("auto", "fused"):
            try:
                from .dp_fused import FusedGradReducer
                self.impl = FusedGradReducer(arena, world_size, self.buckets, group)
                self.mode = "fused"
            except Exception as e:  # missing symmetric memory support etc.
                if mode == "fused":
                    raise
                self.mode = "nccl"
                self.fallback_reason = repr(e)
        else:
            self.mode = "nccl"

    def reduce(self, ctrl: Optional[torch.Tensor] = None, max_norm: float = 0.0) -> bool:
        """Average ``arena.grad`` across ranks (called after backward, before the optimizer).

        In fused mode the same kernels also produce the global gradient norm: when ``ctrl`` is given it receives
        {norm, clip scale for ``max_norm``, finite flag, sum of squares} and the method returns True, meaning no
        separate norm pass is needed.  In NCCL mode it returns False."""
        if self.world == 1:
            return False
        if self.impl is not None:
            self.impl.reduce()
            if ctrl is None:
                if not hasattr(self, "_ctrl"):
                    self._ctrl = torch.zeros(4, dtype=torch.float32, device=self.arena.device)
                ctrl = self._ctrl
                self.impl.finalize(ctrl, 0.0)
                return False
            self.impl.finalize(ctrl, max_norm)
            return True
        g = self.arena.grad
        for (s, e) in self.buckets:
            dist.all_reduce(g[s:e], op=dist.ReduceOp.AVG, group=self.group)
        return False
