"""Fused data-parallel gradient reduction: host side of ``csrc/dp_allreduce.cu``.

The flat gradient buffer of the parameter arena is moved into symmetric memory (allocated and exchanged through
``torch.distributed._symmetric_memory``: that is the plumbing; no collective library runs on the data path).  Per
bucket, one kernel of this package averages the bucket across ranks with multimem (NVSwitch in-switch reduction) or
plain peer loads / stores and leaves the bucket's sum of squares in a symmetric signal buffer; ``finalize`` turns those
into the clip control block on the device.  Clipping therefore needs no extra pass over the gradients in
data-parallel runs, and nothing returns to the host.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native as N

MAX_RANKS = 8
c_void_p, c_int, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong


class DpArgs(ctypes.Structure):
    _fields_ = [("bases", c_void_p * MAX_RANKS), ("pads", c_void_p * MAX_RANKS), ("mc_base", c_void_p),
                ("rank", c_int), ("world", c_int), ("bucket", c_int), ("num_buckets", c_int),
                ("start", c_ll), ("n", c_ll), ("cta_partial", c_void_p), ("cta_counter", c_void_p),
                ("epochs", c_void_p), ("grid", c_int), ("use_nvls", c_int), ("wait_ns", c_ll)]


def _declare(lib):
    lib.dptb_dp_pad_words.argtypes = [c_int]
    lib.dptb_dp_pad_words.restype = c_ll
    lib.dptb_dp_allreduce.argtypes = [ctypes.POINTER(DpArgs), c_void_p]
    lib.dptb_dp_allreduce.restype = c_int
    lib.dptb_dp_finalize.argtypes = [c_void_p, c_void_p, c_int, c_int, ctypes.c_float, c_void_p, c_ll, c_void_p]
    lib.dptb_dp_finalize.restype = c_int


class FusedGradReducer:
    def __init__(self, arena, world_size: int, buckets: List[Tuple[int, int]], group=None, grid: int = 32,
                 use_nvls: Optional[bool] = None, tail_grid: int = 148, max_skew_s: Optional[float] = None):
        """``grid``: CTAs of a bucket reduced under the backward pass (kept small so it does not take SMs from the
        backward kernels); ``tail_grid``: CTAs of a bucket launched after backward, when nothing is left to hide
        under.  ``max_skew_s``: how long a rank waits for its peers' gradients before it gives up and poisons the
        step's norm (default ``DPTB200_DP_MAX_SKEW_S`` or 30 s: a rank may be late by a checkpoint save or a log
        flush)."""
        import torch.distributed._symmetric_memory as symm_mem
        if world_size > MAX_RANKS:
            raise ValueError(f"fused data parallelism supports up to {MAX_RANKS} ranks per node")
        if arena.grad.dtype != torch.bfloat16:
            raise TypeError("fused data parallelism reduces bf16 gradients")
        self.lib = N.load()
        _declare(self.lib)
        self.arena, self.world = arena, world_size
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.buckets = buckets
        self.grid, self.tail_grid = grid, max(grid, tail_grid)
        if max_skew_s is None:
            max_skew_s = float(os.environ.get("DPTB200_DP_MAX_SKEW_S", "30"))
        self.wait_ns = int(max_skew_s * 1e9)
        dev = arena.device
        gname = self.group.group_name

        # Gradient buffer -> symmetric memory; every p.grad view is re-pointed at it.
        n = arena.numel
        sym_grad = symm_mem.empty(n, dtype=torch.bfloat16, device=dev)
        self.grad_handle = symm_mem.rendezvous(sym_grad, group=gname)
        sym_grad.copy_(arena.grad)
        arena.grad = sym_grad
        for p in arena.params:
            o = arena.offsets[id(p)]
            p.grad = sym_grad[o:o + p.numel()].view(p.shape)
        # Signal buffer: ready / done / sumsq words per (bucket, rank).
        nb = len(buckets)
        words = int(self.lib.dptb_dp_pad_words(nb))
        self.pad = symm_mem.empty(max(words, 64), dtype=torch.int32, device=dev)
        self.pad.zero_()
        self.pad_handle = symm_mem.rendezvous(self.pad, group=gname)
        self.bases = [int(p) for p in self.grad_handle.buffer_ptrs]
        self.pads = [int(p) for p in self.pad_handle.buffer_ptrs]
        mc = int(getattr(self.grad_handle, "multicast_ptr", 0) or 0)
        env = os.environ.get("DPTB200_DP_NVLS")
        want = (mc != 0) if use_nvls is None else use_nvls
        if env is not None:
            want = env not in ("0", "false", "False")
        self.use_nvls = bool(want and mc != 0)
        self.mc_base = mc
        # Local scratch: per-bucket CTA partials, counters and epochs.
        self.cta_partial = torch.zeros(nb * self.tail_grid, dtype=torch.float32, device=dev)
        self.cta_counter = torch.zeros(nb, dtype=torch.int32, device=dev)
        self.epochs = torch.zeros(nb, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)   # every rank's signal buffer is zeroed before anyone signals
        self._args = []
        for b, (s, e) in enumerate(buckets):
            a = DpArgs()
            for r in range(MAX_RANKS):
                a.bases[r] = self.bases[r] if r < world_size else None
                a.pads[r] = self.pads[r] if r < world_size else None
            a.mc_base = self.mc_base if self.use_nvls else None
            a.rank, a.world, a.bucket, a.num_buckets = self.rank, world_size, b, nb
            a.start, a.n = s, e - s
            a.cta_partial = self.cta_partial.data_ptr() + 4 * b * self.tail_grid
            a.cta_counter = self.cta_counter.data_ptr() + 4 * b
            a.epochs = self.epochs.data_ptr()
            a.grid, a.use_nvls, a.wait_ns = grid, int(self.use_nvls), self.wait_ns
            self._args.append(a)

    def reduce_bucket(self, b: int, exposed: bool = False) -> None:
        """``exposed``: nothing else runs beside this launch (it comes after backward), so it takes the whole GPU."""
        a = self._args[b]
        a.grid = self.tail_grid if exposed else self.grid
        N.check(self.lib.dptb_dp_allreduce(ctypes.byref(a), N.stream_ptr()), "dp_allreduce")

    def reduce(self) -> None:
        for b in range(len(self.buckets)):
            self.reduce_bucket(b, exposed=True)

    def finalize(self, ctrl: torch.Tensor, max_norm: float) -> None:
        """Wait for every rank's buckets and write {norm, scale, finite, sumsq} into ``ctrl`` (device)."""
        N.check(self.lib.dptb_dp_finalize(self.pad.data_ptr(), self.epochs.data_ptr(), len(self.buckets), self.world,
                                          float(max_norm), ctrl.data_ptr(), self.wait_ns, N.stream_ptr()),
                "dp_finalize")
