"""Tensor parallelism over NVLink peer memory: host side of the fused GEMM + all-reduce kernel (``csrc/gemm.cu``,
``dptb_gemm_allreduce``).

The reference has no tensor parallelism; its per-head ``Linear`` lists make head sharding natural
(lib/core/nn/attention/multi_head_attention.dart:58-94) but nothing shards.  Here QKV / gate / up are column-parallel
(each rank holds a slice of the output features, no communication), ``wo`` / ``down`` are row-parallel: every rank
multiplies its K-slice and the partial sums are reduced across ranks *inside the GEMM kernel's epilogue*, tile by tile,
through symmetric memory (``torch.distributed._symmetric_memory`` allocates and exchanges the buffers; no collective
library runs on the data path).  The reduced rows, plus bias and residual, land in every rank's copy of a symmetric
activation buffer.

``TpComm`` owns the symmetric buffers of one group: ``num_bufs`` activation buffers ``[max_rows, width]`` (the residual
stream ping-pongs between them), one partial-tile buffer, one flag array, and the local epoch / exit counters.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _native as N
from ..ops import kernels as K

MAX_RANKS = 8
c_void_p, c_int, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong


class TpArArgs(ctypes.Structure):
    _fields_ = [("world", c_int), ("rank", c_int), ("use_nvls", c_int), ("max_tiles", c_int),
                ("partial", c_void_p), ("partial_elems", c_ll),
                ("peer_partial", c_void_p * MAX_RANKS), ("mc_partial", c_void_p),
                ("out_peer", c_void_p * MAX_RANKS), ("mc_out", c_void_p),
                ("flags_peer", c_void_p * MAX_RANKS), ("epoch", c_void_p), ("exit_counter", c_void_p),
                ("mode", c_int)]


class TpAgArgs(ctypes.Structure):
    _fields_ = [("world", c_int), ("rank", c_int), ("rows_per_rank", c_ll),
                ("a_peer", c_void_p * MAX_RANKS), ("ready", c_void_p), ("epoch", c_void_p)]


class TpOneShotArgs(ctypes.Structure):
    _fields_ = [("world", c_int), ("rank", c_int), ("max_tiles", c_int), ("reserved", c_int),
                ("slots_peer", c_void_p * MAX_RANKS), ("epoch", c_void_p), ("exit_counter", c_void_p)]


class TpSignalArgs(ctypes.Structure):
    _fields_ = [("world", c_int), ("rank", c_int), ("ready_peer", c_void_p * MAX_RANKS), ("epoch", c_void_p)]


def _declare(lib):
    lib.dptb_tp_flag_words.argtypes = [c_int]
    lib.dptb_tp_flag_words.restype = c_ll
    lib.dptb_gemm_allreduce.argtypes = [ctypes.POINTER(N.GemmArgs), ctypes.POINTER(TpArArgs), c_void_p]
    lib.dptb_gemm_allreduce.restype = c_int
    lib.dptb_allgather_gemm.argtypes = [ctypes.POINTER(N.GemmArgs), ctypes.POINTER(TpAgArgs), c_void_p]
    lib.dptb_allgather_gemm.restype = c_int
    lib.dptb_tp_signal.argtypes = [ctypes.POINTER(TpSignalArgs), c_void_p]
    lib.dptb_tp_signal.restype = c_int
    lib.dptb_tp_wait_ready.argtypes = [c_void_p, c_void_p, c_int, c_int, c_void_p]
    lib.dptb_tp_wait_ready.restype = c_int
    lib.dptb_copy_async.argtypes = [c_void_p, c_void_p, c_ll, c_void_p]
    lib.dptb_copy_async.restype = c_int
    lib.dptb_gemm_skinny.argtypes = [ctypes.POINTER(N.GemmArgs), ctypes.POINTER(TpArArgs), c_void_p]
    lib.dptb_gemm_skinny.restype = c_int
    lib.dptb_gemm_skinny_oneshot.argtypes = [ctypes.POINTER(N.GemmArgs), ctypes.POINTER(TpOneShotArgs), c_void_p]
    lib.dptb_gemm_skinny_oneshot.restype = c_int


def shard_range(total: int, rank: int, world: int):
    """Contiguous equal split; ``total`` must divide."""
    if total % world:
        raise ValueError(f"cannot split {total} over {world} ranks")
    per = total // world
    return rank * per, (rank + 1) * per


class TpComm:
    def __init__(self, max_rows: int, width: int, group=None, num_bufs: int = 2, device=None,
                 use_nvls: Optional[bool] = None):
        import torch.distributed._symmetric_memory as symm_mem
        self.lib = N.load()
        _declare(self.lib)
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > MAX_RANKS:
            raise ValueError(f"tensor parallelism supports up to {MAX_RANKS} ranks per node")
        if width % 8:
            raise ValueError("TpComm: width must be a multiple of 8")
        dev = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.device, self.max_rows, self.width = dev, max_rows, width
        gname = self.group.group_name
        rows_pad = (max_rows + 127) // 128 * 128
        width_pad = (width + 255) // 256 * 256
        self.max_tiles = (rows_pad // 128) * (width_pad // 128)
        self.partial = symm_mem.empty(rows_pad * width_pad, dtype=torch.bfloat16, device=dev)
        self.partial.zero_()
        self._h_partial = symm_mem.rendezvous(self.partial, group=gname)
        self.bufs: List[torch.Tensor] = []
        self._h_bufs = []
        for _ in range(num_bufs):
            b = symm_mem.empty(max_rows, width, dtype=torch.bfloat16, device=dev)
            b.zero_()
            self.bufs.append(b)
            self._h_bufs.append(symm_mem.rendezvous(b, group=gname))
        words = int(self.lib.dptb_tp_flag_words(self.max_tiles))
        self.flags = symm_mem.empty(words, dtype=torch.int32, device=dev)
        self.flags.zero_()
        self._h_flags = symm_mem.rendezvous(self.flags, group=gname)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.exit_counter = torch.zeros(1, dtype=torch.int32, device=dev)
        # "shard ready" flags of the all-gather GEMM (one word per source rank) and this rank's publication counter
        self.ready = symm_mem.empty(MAX_RANKS, dtype=torch.int32, device=dev)
        self.ready.zero_()
        self._h_ready = symm_mem.rendezvous(self.ready, group=gname)
        self.ag_epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self._ag_side, self._ag_events, self._ag_stage = None, None, None   # staged all-gather GEMM (made on first use)
        mc_ok = all(int(getattr(h, "multicast_ptr", 0) or 0) != 0 for h in [self._h_partial] + self._h_bufs)
        want = mc_ok if use_nvls is None else use_nvls
        env = os.environ.get("DPTB200_TP_NVLS")
        if env is not None:
            want = env not in ("0", "false", "False")
        self.use_nvls = bool(want and mc_ok)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)          # every rank's flags are zero before anyone signals
        self._ar = []
        for i in range(num_bufs):
            a = TpArArgs()
            a.world, a.rank, a.use_nvls, a.max_tiles = self.world, self.rank, int(self.use_nvls), self.max_tiles
            a.partial, a.partial_elems = self.partial.data_ptr(), self.partial.numel()
            for r in range(MAX_RANKS):
                a.peer_partial[r] = int(self._h_partial.buffer_ptrs[r]) if r < self.world else None
                a.out_peer[r] = int(self._h_bufs[i].buffer_ptrs[r]) if r < self.world else None
                a.flags_peer[r] = int(self._h_flags.buffer_ptrs[r]) if r < self.world else None
            a.mc_partial = int(self._h_partial.multicast_ptr) if self.use_nvls else None
            a.mc_out = int(self._h_bufs[i].multicast_ptr) if self.use_nvls else None
            a.epoch, a.exit_counter = self.epoch.data_ptr(), self.exit_counter.data_ptr()
            a.mode = 0
            self._ar.append(a)
        self._rs = []
        for a in self._ar:
            b = TpArArgs()
            ctypes.memmove(ctypes.byref(b), ctypes.byref(a), ctypes.sizeof(TpArArgs))
            b.mode = 1
            self._rs.append(b)
        self._sig = TpSignalArgs()
        self._sig.world, self._sig.rank = self.world, self.rank
        for r in range(MAX_RANKS):
            self._sig.ready_peer[r] = int(self._h_ready.buffer_ptrs[r]) if r < self.world else None
        self._sig.epoch = self.ag_epoch.data_ptr()
        # One-shot all-reduce of decode-sized outputs (csrc/gemm_skinny.cu): per-rank tile slots on every rank, one
        # 8-byte word {fp32 bits, launch number} per value, two halves alternating by launch parity, and the local
        # launch counter (starts at 0, so zeroed slots never look valid).
        # Every rank receives (world - 1) tiles as 16-byte NVLink packets, so the scheme pays off for small groups:
        # measured on the Llama-3-8B TP shapes, 3.70 vs 5.08 ms per decode step with 2 ranks, but 6.65 vs 5.85 ms with
        # 8 ranks, where the gather + broadcast epilogue moves 1/8 of the bytes.  DPTB200_TP_ONESHOT=1 / 0 forces it.
        self._os = None
        want_os = os.environ.get("DPTB200_TP_ONESHOT")
        if (want_os == "1") or (want_os is None and self.world <= 4):
            os_tiles = (width + 127) // 128
            self.os_slots = symm_mem.empty(2 * MAX_RANKS * os_tiles * 64 * 128, dtype=torch.int64, device=dev)
            self.os_slots.zero_()
            self._h_os_slots = symm_mem.rendezvous(self.os_slots, group=gname)
            self.os_epoch = torch.zeros(1, dtype=torch.int32, device=dev)
            self.os_exit = torch.zeros(1, dtype=torch.int32, device=dev)
            o = TpOneShotArgs()
            o.world, o.rank, o.max_tiles = self.world, self.rank, os_tiles
            for r in range(MAX_RANKS):
                o.slots_peer[r] = int(self._h_os_slots.buffer_ptrs[r]) if r < self.world else None
            o.epoch, o.exit_counter = self.os_epoch.data_ptr(), self.os_exit.data_ptr()
            torch.cuda.synchronize()
            dist.barrier(group=self.group)      # every rank's slots are zero before anyone stores into them
            self._os = o

    def buffer(self, index: int, rows: int) -> torch.Tensor:
        """First ``rows`` rows of activation buffer ``index`` (this rank's copy)."""
        if rows > self.max_rows:
            raise ValueError(f"TpComm: {rows} rows exceed the buffer's {self.max_rows}")
        return self.bufs[index][:rows]

    def gemm_allreduce(self, x: torch.Tensor, w_shard: torch.Tensor, out_index: int,
                       residual: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                       scatter: bool = False) -> torch.Tensor:
        """``out = sum_over_ranks(x_r @ w_r^T) (+ bias) (+ residual)`` written into activation buffer ``out_index`` of
        EVERY rank.  ``x``: ``[M, K/world]`` bf16 (this rank's slice of the features), ``w_shard``: ``[N, K/world]``.
        ``residual`` (the same on all ranks) must not alias the output buffer."""
        M, Kr = x.shape
        Nn = w_shard.shape[0]
        if w_shard.shape[1] != Kr:
            raise ValueError(f"gemm_allreduce: inner dimensions differ ({Kr} vs {w_shard.shape[1]})")
        if Nn != self.width:
            raise ValueError(f"gemm_allreduce: output width {Nn} != buffer width {self.width}")
        rows_out = M
        if scatter:
            if M % (self.world * 128):
                raise ValueError(f"gemm_reduce_scatter: {M} rows do not split into whole 128-row tiles per rank")
            rows_out = M // self.world
        out = self.buffer(out_index, rows_out)
        if residual is not None and residual.data_ptr() == out.data_ptr():
            raise ValueError("gemm_allreduce: residual must live in a different buffer than the output")
        for t in (x, w_shard):
            if t.dtype != torch.bfloat16 or t.stride(-1) != 1:
                raise TypeError("gemm_allreduce: operands must be bfloat16 with a contiguous last axis")
        g = N.GemmArgs()
        g.A, g.B, g.C = x.data_ptr(), w_shard.data_ptr(), out.data_ptr()
        g.lda, g.ldb, g.ldc = x.stride(0), w_shard.stride(0), out.stride(0)
        g.M, g.N, g.K = M, Nn, Kr
        g.trans_a, g.trans_b = 0, 1
        g.alpha, g.splits = 1.0, 1
        if bias is not None:
            g.bias, g.bias_f32 = bias.data_ptr(), int(bias.dtype == torch.float32)
        if residual is not None:
            if residual.dtype != torch.bfloat16 or residual.shape[0] != rows_out or residual.shape[1] < Nn:
                raise ValueError("gemm_allreduce: residual has the wrong shape or dtype")
            g.residual, g.ldr = residual.data_ptr(), residual.stride(0)
        args = self._rs[out_index] if scatter else self._ar[out_index]
        if M <= K.SKINNY_MAX_ROWS and not scatter and K._SKINNY_ON:
            # decode-sized rows: the weight-streaming kernel with the same fused all-reduce (split-K needs scratch)
            ws, counters = K.splitk_workspace(x.device)
            g.splits = 0
            g.ws, g.ws_bytes = ws.data_ptr(), ws.numel()
            g.counters, g.num_counters = counters.data_ptr(), counters.numel()
            if self._os is not None:
                # one-shot all-reduce: every rank multicasts its tile and sums all tiles itself (one NVLink hop)
                rc = self.lib.dptb_gemm_skinny_oneshot(ctypes.byref(g), ctypes.byref(self._os), N.stream_ptr())
            else:
                rc = self.lib.dptb_gemm_skinny(ctypes.byref(g), ctypes.byref(args), N.stream_ptr())
            if rc != K.ERR_UNSUPPORTED:
                N.check(rc, "gemm_skinny_allreduce")
                return out
            g.splits = 1
        N.check(self.lib.dptb_gemm_allreduce(ctypes.byref(g), ctypes.byref(args), N.stream_ptr()),
                "gemm_reduce_scatter" if scatter else "gemm_allreduce")
        return out

    def gemm_reduce_scatter(self, x: torch.Tensor, w_shard: torch.Tensor, out_index: int,
                            residual: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sequence-parallel form of ``gemm_allreduce``: this rank keeps rows ``[rank * M / world, (rank + 1) * M /
        world)`` of the sum, as the first ``M / world`` rows of its activation buffer ``out_index``; ``residual`` is
        this rank's ``[M / world, N]`` shard."""
        return self.gemm_allreduce(x, w_shard, out_index, residual=residual, bias=bias, scatter=True)

    def publish_shard(self) -> None:
        """Tell every peer that this rank's row shard (written by kernels launched so far on the current stream) is
        complete.  Every rank calls it once before each ``allgather_gemm``."""
        N.check(self.lib.dptb_tp_signal(ctypes.byref(self._sig), N.stream_ptr()), "tp_signal")

    def allgather_gemm(self, in_index: int, rows_per_rank: int, w_shard: torch.Tensor, out: torch.Tensor,
                       bias: Optional[torch.Tensor] = None, act=None, staged: Optional[bool] = None) -> torch.Tensor:
        """``out[world * rows_per_rank, N] = concat_over_ranks(shard_r) @ w_shard^T``: column-parallel Linear whose
        input is row-sharded.  Rank r's shard is the first ``rows_per_rank`` rows of ITS activation buffer
        ``in_index`` (``publish_shard`` first).

        ``staged`` (the default; ``DPTB200_TP_AG_STAGED=0`` turns it off): every peer shard crosses NVLink once, copied
        into local memory on a side stream while the GEMM of the shard before it runs, own shard first.  Otherwise one
        kernel reads the peers' shards in place with its tile loads, which moves every remote tile once per column
        tile of the output (measured 4-5 times slower at the Llama-3-8B shapes)."""
        if rows_per_rank % 128 or rows_per_rank > self.max_rows:
            raise ValueError("allgather_gemm: rows_per_rank must be a multiple of 128 within the buffer")
        Nn, Kd = w_shard.shape
        if Kd != self.width:
            raise ValueError(f"allgather_gemm: inner dimension {Kd} != buffer width {self.width}")
        M = rows_per_rank * self.world
        if out.shape[0] != M or out.shape[1] < Nn or out.dtype != torch.bfloat16 or out.stride(-1) != 1:
            raise ValueError("allgather_gemm: output must be bf16 [world * rows_per_rank, >= N]")
        if staged is None:
            staged = os.environ.get("DPTB200_TP_AG_STAGED", "1") != "0"
        if staged and self.world > 1:
            return self._allgather_gemm_staged(in_index, rows_per_rank, w_shard, out, bias, act)
        g = N.GemmArgs()
        src = self.bufs[in_index]
        g.A, g.B, g.C = src.data_ptr(), w_shard.data_ptr(), out.data_ptr()
        g.lda, g.ldb, g.ldc = src.stride(0), w_shard.stride(0), out.stride(0)
        g.M, g.N, g.K = M, Nn, Kd
        g.trans_a, g.trans_b = 0, 1
        g.alpha, g.splits = 1.0, 1
        if bias is not None:
            g.bias, g.bias_f32 = bias.data_ptr(), int(bias.dtype == torch.float32)
        if act is not None:
            g.act = K.ACT_CODES[act]
        ag = TpAgArgs()
        ag.world, ag.rank, ag.rows_per_rank = self.world, self.rank, rows_per_rank
        for r in range(MAX_RANKS):
            ag.a_peer[r] = int(self._h_bufs[in_index].buffer_ptrs[r]) if r < self.world else None
        ag.ready, ag.epoch = self.ready.data_ptr(), self.ag_epoch.data_ptr()
        N.check(self.lib.dptb_allgather_gemm(ctypes.byref(g), ctypes.byref(ag), N.stream_ptr()), "allgather_gemm")
        return out

    def _allgather_gemm_staged(self, in_index, rows, w_shard, out, bias, act):
        """Gather by copy, GEMM by shard: the side stream waits (bounded, on the device) for the peers' "shard ready"
        flags, then copies shard after shard into a local staging matrix; the launching stream multiplies this rank's
        own shard at once and each staged shard as soon as its copy has finished."""
        if self._ag_side is None:
            self._ag_side = torch.cuda.Stream(device=self.device)
            self._ag_events = [torch.cuda.Event() for _ in range(self.world + 1)]
        need = self.world * rows
        if self._ag_stage is None or self._ag_stage.shape[0] < need:
            self._ag_stage = torch.empty(need, self.width, dtype=torch.bfloat16, device=self.device)
        stage, side, evs = self._ag_stage, self._ag_side, self._ag_events
        main = torch.cuda.current_stream(self.device)
        order = [(self.rank + i) % self.world for i in range(1, self.world)]
        evs[self.world].record(main)          # after publish_shard, and after the previous consumers of the staging rows
        with torch.cuda.stream(side):
            side.wait_event(evs[self.world])
            N.check(self.lib.dptb_tp_wait_ready(self.ready.data_ptr(), self.ag_epoch.data_ptr(), self.world, self.rank,
                                                N.stream_ptr()), "tp_wait_ready")
            for s in order:
                N.check(self.lib.dptb_copy_async(stage[s * rows:(s + 1) * rows].data_ptr(),
                                                 int(self._h_bufs[in_index].buffer_ptrs[s]),
                                                 rows * self.width * 2, N.stream_ptr()), "copy_async")
                evs[s].record(side)
        b = None if bias is None else bias.view(-1)
        K.gemm(self.bufs[in_index][:rows], w_shard, out[self.rank * rows:(self.rank + 1) * rows], trans_b=True, bias=b,
               act=act, n_cols=w_shard.shape[0])
        for s in order:
            main.wait_event(evs[s])
            K.gemm(stage[s * rows:(s + 1) * rows], w_shard, out[s * rows:(s + 1) * rows], trans_b=True, bias=b, act=act,
                   n_cols=w_shard.shape[0])
        return out


def reference_row_parallel(x_full: torch.Tensor, w_full: torch.Tensor, residual=None, bias=None) -> torch.Tensor:
    """fp32 oracle of what ``gemm_allreduce`` leaves on every rank."""
    y = x_full.float() @ w_full.float().t()
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y
