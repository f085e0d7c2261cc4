"""Tracing hooks: NVTX ranges around the phases of a step, and CUDA-event phase timers.

The reference has no tracer: its demos print wall-clock ``ms/step`` from a ``Stopwatch`` and its autograd engine offers
one global ``debugBackwardHook`` (reference: bin/shakespeare_gpt_big.dart:67-95, lib/core/tensor/tensor.dart:42-45).
Here the phases of the training step (forward, backward, gradient reduction, clipping, optimizer), of the
tensor-parallel engine (prefill, decode step) and any user block can be wrapped in named ranges:

* ``DPTB200_NVTX=1`` (or ``enable_nvtx()``) emits NVTX ranges, which Nsight tools show on the timeline; without a
  profiler attached they cost a function call.  On a machine without CUDA they are no-ops.
* ``PhaseTimer`` measures the same ranges with CUDA events on the current stream (device time, no synchronisation
  until ``summary()``), for machines where no timeline tool is installed.

Neither is active by default, and a range never synchronises the device.
"""
from __future__ import annotations

import contextlib
import os
from typing import Dict, List, Optional, Tuple

import torch

_nvtx_on = os.environ.get("DPTB200_NVTX", "0") not in ("0", "", "false", "False")
_timer: Optional["PhaseTimer"] = None


def enable_nvtx(on: bool = True) -> None:
    global _nvtx_on
    _nvtx_on = bool(on)


def nvtx_enabled() -> bool:
    return _nvtx_on and torch.cuda.is_available()


class PhaseTimer:
    """Device time per named range, from CUDA events recorded on the stream that is current at the range's ends.

    ``with PhaseTimer() as t: ...`` installs it for the ranges opened inside; ``t.summary()`` synchronises once and
    returns ``{name: (calls, total_ms)}``.  Ranges may nest; a range on a CPU-only machine records wall-clock time."""

    def __init__(self):
        self._open: List[Tuple[str, object]] = []
        self._done: List[Tuple[str, object, object]] = []
        self._cuda = torch.cuda.is_available()

    def __enter__(self):
        global _timer
        self._prev = _timer
        _timer = self
        return self

    def __exit__(self, *exc):
        global _timer
        _timer = self._prev
        return False

    def _mark(self):
        if self._cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            return e
        import time
        return time.perf_counter()

    def push(self, name: str) -> None:
        self._open.append((name, self._mark()))

    def pop(self) -> None:
        name, start = self._open.pop()
        self._done.append((name, start, self._mark()))

    def summary(self) -> Dict[str, Tuple[int, float]]:
        if self._cuda:
            torch.cuda.synchronize()
        out: Dict[str, Tuple[int, float]] = {}
        for name, a, b in self._done:
            ms = a.elapsed_time(b) if self._cuda else (b - a) * 1e3
            calls, tot = out.get(name, (0, 0.0))
            out[name] = (calls + 1, tot + ms)
        return out


@contextlib.contextmanager
def range(name: str):
    """Named range: an NVTX range when enabled, a ``PhaseTimer`` entry when one is installed, else nothing."""
    nv = nvtx_enabled()
    t = _timer
    if nv:
        torch.cuda.nvtx.range_push(name)
    if t is not None:
        t.push(name)
    try:
        yield
    finally:
        if t is not None:
            t.pop()
        if nv:
            torch.cuda.nvtx.range_pop()
