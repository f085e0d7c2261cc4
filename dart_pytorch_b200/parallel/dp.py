"""Data-parallel gradient reduction over the flat gradient arena.

The reference has no synchronous data parallelism: its "distributed" mode averages whole checkpoints every K local
steps over HTTP (lib/core/coop/param_avg.dart:20-123).  Here every rank holds a replica, gradients live in one flat
bf16 buffer (``utils/arena.py``) and are averaged across ranks between backward and clip.

``GradReducer(mode="nccl")`` is the library baseline: one ``all_reduce`` per bucket.
``GradReducer(mode="fused")`` runs this package's own kernel per bucket (``csrc/dp_allreduce.cu``): peer / multimem
loads and stores over NVSwitch from inside the kernel, fused with the sum-of-squares partials that clipping needs.

With ``overlap=True`` (fused mode) a bucket is reduced on a side stream as soon as the backward pass has launched the
last kernel that accumulates into it, so NVLink traffic runs under the remaining backward compute.  The trigger needs
no autograd hooks: every kernel that accumulates straight into the arena asks for its target through
``ops.cuda._direct_grad``, which reports the parameter here.  The first step counts how often each parameter is touched
(a tied embedding is touched twice); from then on a parameter is final at its last touch, and a bucket is launched at
the next touch after all of its parameters became final -- by then the finalising kernels are on the stream.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class GradReducer:
    def __init__(self, arena, world_size: int, mode: str = "auto", bucket_mb: float = 32.0, group=None,
                 overlap: bool = False, exclude=()):
        """``exclude``: parameters that exist on this rank only (expert-parallel shards).  Their gradients are not
        averaged; their squared norm is summed over the ranks and folded into the global gradient norm."""
        self.arena, self.world = arena, world_size
        self.group = group
        self.mode = mode
        self.bucket_elems = int(bucket_mb * 1024 * 1024 / arena.grad.element_size())
        self.exclude = list(exclude)
        self.buckets = arena.slices(self.bucket_elems, exclude=self.exclude)
        self.local_ranges = arena.ranges_of(self.exclude) if self.exclude else []
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
        self.overlap = bool(overlap and self.impl is not None and world_size > 1)
        if self.overlap:
            self._side = torch.cuda.Stream()
            self._param_buckets: Dict[int, List[int]] = {}
            for p in arena.ordered:
                o = arena.offsets[id(p)]
                self._param_buckets[id(p)] = [b for b, (s, e) in enumerate(self.buckets) if o < e and o + p.numel() > s]
            self._bucket_params = [sum(1 for p in arena.ordered if b in self._param_buckets[id(p)])
                                   for b in range(len(self.buckets))]
            self._expected: Dict[int, int] = {}
            self._learned = False
            self._active = False

    # ---- overlap machinery ------------------------------------------------------------------------------
    def begin_step(self) -> None:
        """Call after the gradients were zeroed and before backward."""
        if not self.overlap:
            return
        from ..ops import cuda as _cu
        self._seen: Dict[int, int] = {}
        self._left = list(self._bucket_params)
        self._ready: List[int] = []
        self._launched = set()
        self._active = True
        _cu.set_grad_listener(self)

    def touch(self, p: torch.Tensor) -> None:
        """A kernel is about to accumulate into ``p.grad`` (called by ``ops.cuda._direct_grad``)."""
        if not self._active:
            return
        self._flush_ready()
        k = id(p)
        self._seen[k] = self._seen.get(k, 0) + 1
        if self._learned and self._seen[k] == self._expected.get(k, -1):
            self._ready.append(k)

    def _flush_ready(self) -> None:
        for k in self._ready:
            for b in self._param_buckets.get(k, ()):
                self._left[b] -= 1
                if self._left[b] == 0:
                    self._launch(b)
        self._ready.clear()

    def _launch(self, b: int, exposed: bool = False) -> None:
        from ..ops import cuda as _cu
        self._side.wait_stream(torch.cuda.current_stream())
        extra = _cu.param_side_stream(self.arena.grad.device)   # bias sums / norm parameter gradients may run there
        if extra is not None:
            self._side.wait_stream(extra)
        with torch.cuda.stream(self._side):
            self.impl.reduce_bucket(b, exposed=exposed)
        self._launched.add(b)

    def _finish_overlap(self) -> None:
        from ..ops import cuda as _cu
        _cu.set_grad_listener(None)
        self._active = False
        self._flush_ready()
        if not self._learned:
            self._expected = dict(self._seen)
            self._learned = True
        for b in range(len(self.buckets)):
            if b not in self._launched:
                self._launch(b, exposed=True)      # backward is over: these run alone, on the whole GPU
        torch.cuda.current_stream().wait_stream(self._side)

    def _fold_local_norm(self, ctrl: torch.Tensor, max_norm: float) -> None:
        """ctrl = {norm, scale, finite, sumsq} of the averaged ranges; add the ranks' own squared norms of the
        rank-local ranges (one tiny sum over the group) and recompute norm and clip scale on the device."""
        g = self.arena.grad
        local = torch.zeros(1, dtype=torch.float32, device=g.device)
        for s, e in self.local_ranges:
            # a rank-local expert already holds the summed contributions of every rank's tokens; the global loss is
            # the mean of the ranks' losses, so it takes the same 1 / world factor as the averaged ranges
            g[s:e].mul_(1.0 / self.world)
            local += g[s:e].float().pow(2).sum()
        dist.all_reduce(local, op=dist.ReduceOp.SUM, group=self.group)
        total = ctrl[3] + local[0]
        norm = total.sqrt()
        ctrl[3] = total
        ctrl[0] = norm
        finite = torch.isfinite(norm)
        ctrl[2] = finite.float()
        if max_norm > 0.0:
            ctrl[1] = torch.where(finite & (norm > max_norm), max_norm / norm, torch.ones_like(norm))

    # ---- reduction --------------------------------------------------------------------------------------
    def reduce(self, ctrl: Optional[torch.Tensor] = None, max_norm: float = 0.0) -> bool:
        """Average ``arena.grad`` across ranks (called after backward, before the optimizer).

        In fused mode the same kernels also produce the global gradient norm: when ``ctrl`` is given it receives
        {norm, clip scale for ``max_norm``, finite flag, sum of squares} and the method returns True, meaning no
        separate norm pass is needed.  In NCCL mode it returns False."""
        if self.world == 1:
            return False
        if self.impl is not None:
            if self.overlap and self._active:
                self._finish_overlap()
            else:
                self.impl.reduce()
            if ctrl is None:
                if not hasattr(self, "_ctrl"):
                    self._ctrl = torch.zeros(4, dtype=torch.float32, device=self.arena.device)
                ctrl = self._ctrl
                self.impl.finalize(ctrl, 0.0)
                return False
            self.impl.finalize(ctrl, max_norm)
            if self.local_ranges:
                self._fold_local_norm(ctrl, max_norm)
            return True
        g = self.arena.grad
        for (s, e) in self.buckets:
            dist.all_reduce(g[s:e], op=dist.ReduceOp.AVG, group=self.group)
        return False
