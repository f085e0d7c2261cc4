"""Trainer: the public training-step API (forward, backward, gradient reduction, clip, optimizer, schedule).

One call to ``Trainer.step(tokens, targets)`` does what the reference's training loops spell out op by op
(bin/gpt_train.dart:111-131): zeroGrad, loss, backward, clipGradNorm, optimizer step, scheduler step.  On a CUDA
device the whole device-side sequence is captured once into a CUDA graph and replayed, with inputs staged through
pinned host memory; the per-step host work is one small async copy of {lr, bias corrections} and the graph launch.
With ``world_size > 1`` gradients are reduced across ranks by ``parallel.dp`` between backward and clip.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ..optim.grad_utils import clip_grad_norm
from . import trace


class Trainer:
    def __init__(self, model, optimizer, scheduler=None, clip_norm: Optional[float] = None,
                 loss_fn: Optional[Callable] = None, use_graph: Optional[bool] = None, reducer=None):
        self.model, self.opt, self.sched = model, optimizer, scheduler
        self.clip_norm = clip_norm
        self.loss_fn = loss_fn or (lambda m, x, y: m.loss(x, y))
        self.reducer = reducer
        self.on_cuda = model.device.type == "cuda"
        self.use_graph = (self.on_cuda and getattr(optimizer, "arena", None) is not None) if use_graph is None \
            else (use_graph and self.on_cuda)
        self._graph = None
        self._static_x = self._static_y = None
        self._static_loss = None
        self._static_norm = None
        self._warm = 0
        # Warm-up steps and the capture share one side stream (autograd records the streams its nodes ran on; a
        # backward captured on a stream other than the one that warmed up would depend on uncaptured work).
        self._stream = torch.cuda.Stream() if self.use_graph else None
        self.last_norm = None
        self.kernels_per_step = None
        # Data parallel: a rank whose wait for its peers ran out poisons the step's gradient norm (NaN), so the update
        # must be skipped on every rank alike, and the device status word is polled now and then so that the run stops
        # with an error instead of training on with diverged replicas.
        self.health_every = 100 if reducer is not None else 0
        self._steps = 0
        if reducer is not None and hasattr(optimizer, "skip_nonfinite"):
            optimizer.skip_nonfinite = True

    # ---- one eager step (also what gets captured) -------------------------------------------------
    def _device_step(self, x, y, split_optimizer: bool):
        # Phases are named ranges (utils/trace.py): NVTX when enabled, device-timed under a PhaseTimer, else free.
        with trace.range("step/forward"):
            self.opt.zero_grad()
            loss = self.loss_fn(self.model, x, y)
        if self.reducer is not None and hasattr(self.reducer, "begin_step"):
            self.reducer.begin_step()          # buckets may be reduced under the rest of the backward pass
        with trace.range("step/backward"):
            loss.backward()
        norm = None
        clipped = False
        if self.reducer is not None:
            with trace.range("step/grad_reduce"):
                has_ctrl = self.clip_norm is not None and getattr(self.opt, "arena", None) is not None
                clipped = self.reducer.reduce(self.opt.ctrl if has_ctrl else None, self.clip_norm or 0.0)
            if clipped:
                from ..optim.grad_utils import LazyScalar
                self.opt.clip_pending = True
                norm = LazyScalar(self.opt.ctrl, 0)
        if self.clip_norm is not None and not clipped:
            with trace.range("step/clip"):
                norm = clip_grad_norm(self.opt, self.clip_norm)
        with trace.range("step/optimizer"):
            if split_optimizer:
                self.opt.launch_step()
            else:
                self.opt.step()
        return loss, norm

    def _capture(self, x, y):
        from .. import _native as N
        self._static_x = torch.empty_like(x)
        self._static_y = torch.empty_like(y)
        self._static_x.copy_(x)
        self._static_y.copy_(y)
        lib = N.load()
        lib.dptb_launch_count.restype = __import__("ctypes").c_longlong
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        before = lib.dptb_launch_count()
        with torch.cuda.graph(graph, stream=self._stream):
            loss, norm = self._device_step(self._static_x, self._static_y, split_optimizer=True)
        self.kernels_per_step = int(lib.dptb_launch_count() - before)
        self._static_loss = loss
        self._static_norm = norm
        self._graph = graph

    def step(self, x: torch.Tensor, y: torch.Tensor):
        """Run one optimisation step; returns the (device) loss tensor of this step.

        ``x`` / ``y`` may live in (pinned) host memory: they are copied to the device asynchronously."""
        dev = self.model.device
        self._steps += 1
        if self.health_every and self.on_cuda and self._steps % self.health_every == 0:
            from .. import _native
            _native.raise_on_device_error()    # synchronises; every `health_every` steps only
        if self.on_cuda and not x.is_cuda:
            x = x.to(dev, non_blocking=True)
            y = y.to(dev, non_blocking=True)
        splittable = hasattr(self.opt, "launch_step") and getattr(self.opt, "arena", None) is not None
        if self.use_graph and splittable:
            if self._graph is None and self._warm >= 2:
                self.opt.prepare_step()
                self._capture(x, y)   # capture does not execute; replay below runs this step
                self._graph.replay()
            elif self._graph is None:
                # Warm-up steps run eagerly (allocator, lazy module state, kernel attributes).
                self._warm += 1
                self._stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self._stream):
                    self.opt.prepare_step()
                    loss, norm = self._device_step(x, y, split_optimizer=True)
                torch.cuda.current_stream().wait_stream(self._stream)
                self.last_norm = norm
                if self.sched is not None:
                    self.sched.step()
                return loss
            else:
                self._static_x.copy_(x, non_blocking=True)
                self._static_y.copy_(y, non_blocking=True)
                self.opt.prepare_step()
                self._graph.replay()
            self.last_norm = self._static_norm
            if self.sched is not None:
                self.sched.step()
            return self._static_loss
        loss, norm = self._device_step(x, y, split_optimizer=False)
        self.last_norm = norm
        if self.sched is not None:
            self.sched.step()
        return loss
