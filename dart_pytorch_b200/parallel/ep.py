"""Expert parallelism: host side of ``csrc/moe_ep.cu``.

The reference runs every expert on one device (lib/core/nn/moe.dart:364-536).  Here the experts of a layer are sharded
over the ranks of a group and token rows travel to their experts and back through symmetric memory, written by the
dispatch / return kernels themselves (peer stores over NVLink; no collective library on the data path).

Forward of one layer on a rank with local tokens ``x [T, D]``::

    logits = x Wg^T;  (probs, idx, w) = route(logits)          softmax, top-k (optionally renormalised)
    slot, count = slots(idx)                                   position inside the (source, expert) quota of C rows
    rows_in  = dispatch(x, idx, slot)                          [El * world * C, D] on every expert's rank
    rows_out = experts(rows_in)                                SwiGLU MLP per local expert (tensor-core GEMMs)
    y = combine(return(rows_out), idx, slot, w)                rows come home, weighted sum over the k choices
    aux = E * sum_e f_e * mean_t probs[t, e]                   load-balance loss (f_e: fraction of routed pairs)

Rows beyond a quota are dropped (their weight contributes nothing), which is the capacity-factor rule applied per
source rank.  ``EpDispatchFn`` / ``EpCombineFn`` are each other's adjoints, so the backward pass is the same kernels run
in the opposite direction; the expert MLP in between is ordinary differentiable ops.
"""
from __future__ import annotations

import ctypes
import math
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _native as N
from .. import ops as F
from ..nn.layers import Linear
from ..nn.module import Module, make_param, normal_, uniform_
from .tp import MAX_RANKS

c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


class EpArgs(ctypes.Structure):
    _fields_ = [("world", c_int), ("rank", c_int), ("El", c_int), ("C", c_int), ("D", c_int), ("E", c_int),
                ("recv_peer", c_void_p * MAX_RANKS), ("ret_peer", c_void_p * MAX_RANKS),
                ("counts_peer", c_void_p * MAX_RANKS), ("flags_peer", c_void_p * MAX_RANKS),
                ("epoch", c_void_p), ("exit_counter", c_void_p)]


_declared = False


def _lib():
    global _declared
    lib = N.load()
    if not _declared:
        P, I, L, Fl = c_void_p, c_int, c_ll, c_float
        EP = ctypes.POINTER(EpArgs)
        for name, args in (("dptb_moe_route", [P, L, I, P, P, P, I, I, I, I, Fl, I, P, I, I, P]),
                           ("dptb_moe_slots", [P, P, P, I, I, I, P]),
                           ("dptb_moe_dispatch", [EP, P, L, P, P, P, P, I, I, P]),
                           ("dptb_moe_zero_tail", [P, P, I, I, I, I, P]),
                           ("dptb_moe_return", [EP, P, P, P]),
                           ("dptb_moe_combine", [P, P, P, P, P, L, I, I, I, I, P]),
                           ("dptb_moe_combine_dot", [P, P, P, P, L, P, I, I, I, I, P])):
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, c_int
        _declared = True
    return lib


def capacity(tokens: int, top_k: int, num_experts: int, capacity_factor: float) -> int:
    """Rows per (source rank, expert) quota, rounded up to a multiple of 8."""
    c = int(math.ceil(capacity_factor * tokens * top_k / num_experts))
    return max(8, (c + 7) // 8 * 8)


class EpComm:
    """Symmetric buffers of one expert-parallel group for rows of width ``D`` and quota ``C``."""

    def __init__(self, num_experts: int, C: int, D: int, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.lib = _lib()
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if num_experts % self.world:
            raise ValueError("EpComm: the number of experts must divide by the group size")
        if D % 8:
            raise ValueError("EpComm: row width must be a multiple of 8")
        self.E, self.El, self.C, self.D = num_experts, num_experts // self.world, C, D
        dev = torch.device("cuda", torch.cuda.current_device())
        self.device = dev
        gname = self.group.group_name
        self.recv = symm_mem.empty(self.El * self.world * C, D, dtype=torch.bfloat16, device=dev)
        self.ret = symm_mem.empty(self.E * C, D, dtype=torch.bfloat16, device=dev)
        self.counts = symm_mem.empty(self.El * self.world, dtype=torch.int32, device=dev)
        self.flags = symm_mem.empty(2 * MAX_RANKS, dtype=torch.int32, device=dev)
        for t in (self.recv, self.ret, self.counts, self.flags):
            t.zero_()
        hs = [symm_mem.rendezvous(t, group=gname) for t in (self.recv, self.ret, self.counts, self.flags)]
        self._handles = hs
        self.epoch = torch.zeros(2, dtype=torch.int32, device=dev)
        self.exit_counter = torch.zeros(2, dtype=torch.int32, device=dev)
        a = EpArgs()
        a.world, a.rank, a.El, a.C, a.D, a.E = self.world, self.rank, self.El, C, D, self.E
        for r in range(MAX_RANKS):
            ok = r < self.world
            a.recv_peer[r] = int(hs[0].buffer_ptrs[r]) if ok else None
            a.ret_peer[r] = int(hs[1].buffer_ptrs[r]) if ok else None
            a.counts_peer[r] = int(hs[2].buffer_ptrs[r]) if ok else None
            a.flags_peer[r] = int(hs[3].buffer_ptrs[r]) if ok else None
        a.epoch, a.exit_counter = self.epoch.data_ptr(), self.exit_counter.data_ptr()
        self.args = a
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    # ---- kernels --------------------------------------------------------------------------------------
    def dispatch(self, x: torch.Tensor, idx: torch.Tensor, slot: torch.Tensor, count: torch.Tensor,
                 scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Send rows to their experts; returns a fresh copy of what arrived here ``[El * world * C, D]`` (unused
        quota rows zeroed)."""
        T, k = idx.shape
        N.check(self.lib.dptb_moe_dispatch(ctypes.byref(self.args), x.data_ptr(), x.stride(0), idx.data_ptr(),
                                           slot.data_ptr(), N.ptr(scale), count.data_ptr(), T, k, N.stream_ptr()),
                "moe_dispatch")
        counts_here = self.counts.clone()
        N.check(self.lib.dptb_moe_zero_tail(self.recv.data_ptr(), counts_here.data_ptr(), self.El, self.world, self.C,
                                            self.D, N.stream_ptr()), "moe_zero_tail")
        return self.recv.clone(), counts_here

    def give_back(self, rows: torch.Tensor, counts_here: torch.Tensor) -> torch.Tensor:
        """Return expert-side rows to their sources; returns a fresh copy of ``ret [E * C, D]`` of this rank."""
        N.check(self.lib.dptb_moe_return(ctypes.byref(self.args), rows.data_ptr(), counts_here.data_ptr(),
                                         N.stream_ptr()), "moe_return")
        return self.ret.clone()

    def combine(self, ret: torch.Tensor, idx: torch.Tensor, slot: torch.Tensor, w: Optional[torch.Tensor]):
        T, k = idx.shape
        y = torch.empty(T, self.D, dtype=torch.bfloat16, device=ret.device)
        N.check(self.lib.dptb_moe_combine(ret.data_ptr(), idx.data_ptr(), slot.data_ptr(), N.ptr(w), y.data_ptr(),
                                          y.stride(0), T, k, self.C, self.D, N.stream_ptr()), "moe_combine")
        return y

    def combine_dot(self, ret: torch.Tensor, idx: torch.Tensor, slot: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
        T, k = idx.shape
        dw = torch.empty(T, k, dtype=torch.float32, device=ret.device)
        N.check(self.lib.dptb_moe_combine_dot(ret.data_ptr(), idx.data_ptr(), slot.data_ptr(), dy.data_ptr(),
                                              dy.stride(0), dw.data_ptr(), T, k, self.C, self.D, N.stream_ptr()),
                "moe_combine_dot")
        return dw


def route(logits: torch.Tensor, top_k: int, renorm: bool = False, route_scale: float = 1.0, gate: str = "softmax",
          bias: Optional[torch.Tensor] = None, groups: int = 1, top_groups: Optional[int] = None):
    """``(probs [T, E] fp32, idx [T, k] int32, w [T, k] fp32)`` of router logits ``[T, E]`` (fp32 or bf16).
    ``gate``: "softmax" or "sigmoid"; ``bias [E]`` fp32 is added to the scores for the choice only; ``groups`` /
    ``top_groups``: grouped top-k (reference: lib/core/nn/moe.dart:379-472)."""
    lib = _lib()
    T, E = logits.shape
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != E or not bias.is_contiguous()):
        raise ValueError("route: bias must be a contiguous fp32 vector with one entry per expert")
    probs = torch.empty(T, E, dtype=torch.float32, device=logits.device)
    idx = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    N.check(lib.dptb_moe_route(logits.data_ptr(), logits.stride(0), int(logits.dtype == torch.float32),
                               probs.data_ptr(), idx.data_ptr(), w.data_ptr(), T, E, top_k, int(renorm),
                               float(route_scale), {"softmax": 0, "sigmoid": 1}[gate], N.ptr(bias), int(groups),
                               int(groups if top_groups is None else top_groups), N.stream_ptr()), "moe_route")
    return probs, idx, w


def slots(idx: torch.Tensor, num_experts: int, C: int):
    """``(slot [T, k] int32 (-1 = dropped), count [E] int32)``: token order inside every expert's quota."""
    lib = _lib()
    slot = torch.empty_like(idx)
    count = torch.empty(num_experts, dtype=torch.int32, device=idx.device)
    N.check(lib.dptb_moe_slots(idx.data_ptr(), slot.data_ptr(), count.data_ptr(), idx.numel(), num_experts, C,
                               N.stream_ptr()), "moe_slots")
    return slot, count


class EpDispatchFn(torch.autograd.Function):
    """rows_in = dispatch(x); adjoint: dx[t] = sum_j returned(d_rows_in)[e_j][slot_j]."""

    @staticmethod
    def forward(ctx, x, comm: EpComm, idx, slot, count):
        rows, counts_here = comm.dispatch(x, idx, slot, count)
        ctx.comm, ctx.meta = comm, (idx, slot, counts_here)
        ctx.mark_non_differentiable(counts_here)
        return rows, counts_here

    @staticmethod
    def backward(ctx, d_rows, _):
        idx, slot, counts_here = ctx.meta
        d_rows = d_rows if d_rows.is_contiguous() else d_rows.contiguous()
        ret = ctx.comm.give_back(d_rows, counts_here)
        return ctx.comm.combine(ret, idx, slot, None), None, None, None, None


class EpCombineFn(torch.autograd.Function):
    """y = combine(returned(rows_out), w); adjoints: d_rows_out = dispatch(w * dy), dw = <dy, returned rows>."""

    @staticmethod
    def forward(ctx, rows_out, w, comm: EpComm, idx, slot, count, counts_here):
        rows_out = rows_out if rows_out.is_contiguous() else rows_out.contiguous()
        ret = comm.give_back(rows_out, counts_here)
        ctx.comm, ctx.meta = comm, (idx, slot, count)
        ctx.save_for_backward(ret, w)
        return comm.combine(ret, idx, slot, w)

    @staticmethod
    def backward(ctx, dy):
        ret, w = ctx.saved_tensors
        idx, slot, count = ctx.meta
        dy = dy if dy.is_contiguous() else dy.contiguous()
        dw = ctx.comm.combine_dot(ret, idx, slot, dy)
        d_rows, _ = ctx.comm.dispatch(dy, idx, slot, count, scale=w)
        return d_rows, dw, None, None, None, None, None


class RouteFn(torch.autograd.Function):
    """Gate (softmax or sigmoid) + (grouped, biased) top-k on the device; gradients flow to the logits through the
    selected probabilities (and through all probabilities for the auxiliary loss)."""

    @staticmethod
    def forward(ctx, logits, top_k, renorm, route_scale, gate="softmax", bias=None, groups=1, top_groups=None):
        probs, idx, w = route(logits, top_k, renorm, route_scale, gate, bias, groups, top_groups)
        ctx.save_for_backward(probs, idx, w)
        ctx.cfg = (top_k, renorm, route_scale, logits.dtype, gate)
        ctx.mark_non_differentiable(idx)
        return probs, idx, w

    @staticmethod
    def backward(ctx, d_probs, _, d_w):
        probs, idx, w = ctx.saved_tensors
        top_k, renorm, route_scale, dtype, gate = ctx.cfg
        dp = torch.zeros_like(probs) if d_probs is None else d_probs.float().clone()
        if d_w is not None:
            li = idx.long()
            sel = torch.gather(probs, 1, li)
            g = d_w.float() * route_scale
            if renorm:
                s = sel.sum(1, keepdim=True) + 1e-9
                g = (g - (g * sel).sum(1, keepdim=True) / s) / s
            dp.scatter_add_(1, li, g)
        if gate == "sigmoid":
            dlogits = dp * probs * (1.0 - probs)
        else:
            dlogits = probs * (dp - (dp * probs).sum(1, keepdim=True))
        return dlogits.to(dtype), None, None, None, None, None, None, None


class ExpertParallelMoE(Module):
    """SwiGLU experts sharded over an expert-parallel group, softmax top-k routing with a per-source capacity quota and
    a load-balance auxiliary loss (``self.aux_loss`` after every forward)."""

    def __init__(self, dim: int, hidden: int, num_experts: int, top_k: int = 2, capacity_factor: float = 1.25,
                 aux_loss_coef: float = 0.01, tokens_per_rank: int = 0, group=None, renormalize_top_k: bool = False,
                 route_scale: float = 1.0, device=None, seed: int = 0, dtype=torch.bfloat16,
                 init_std: Optional[float] = None, gate_function: str = "softmax", num_expert_groups: int = 1,
                 top_k_groups: Optional[int] = None, bias_update_rate: float = 0.001):
        """``gate_function``: "softmax" or "sigmoid"; ``num_expert_groups`` / ``top_k_groups``: grouped top-k;
        ``bias_update_rate``: step of the aux-loss-free balancing bias (``update_routing_bias``), all as in the
        single-device layer (reference: lib/core/nn/moe.dart:379-472, 550-569)."""
        super().__init__()
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if num_experts % self.world:
            raise ValueError("ExpertParallelMoE: num_experts must divide by the group size")
        self.dim, self.hidden, self.E, self.k = dim, hidden, num_experts, top_k
        self.El = num_experts // self.world
        self.capacity_factor, self.aux_loss_coef = capacity_factor, aux_loss_coef
        self.renorm, self.route_scale = renormalize_top_k, route_scale
        if gate_function not in ("softmax", "sigmoid"):
            raise ValueError("ExpertParallelMoE: gate_function must be 'softmax' or 'sigmoid'")
        if num_expert_groups < 1 or num_experts % num_expert_groups:
            raise ValueError("ExpertParallelMoE: num_experts must divide into num_expert_groups groups")
        self.gate_function, self.groups = gate_function, num_expert_groups
        self.top_groups = num_expert_groups if top_k_groups is None else top_k_groups
        if not 1 <= self.top_groups <= self.groups or top_k > self.top_groups * (num_experts // self.groups):
            raise ValueError("ExpertParallelMoE: top_k_groups out of range for top_k")
        self.bias_update_rate = bias_update_rate
        self.routing_bias = torch.zeros(num_experts, dtype=torch.float32, device=device)
        self._expert_load = torch.zeros(num_experts, dtype=torch.float32, device=device)
        # router weights are replicated (same seed on every rank); expert weights are seeded by global expert id
        self.gate = make_param(normal_((num_experts, dim), init_std or 0.02, seed, device, dtype))
        self.w_gate_up: List[torch.Tensor] = []
        self.w_down: List[torch.Tensor] = []
        for le in range(self.El):
            ge = self.rank * self.El + le
            std1 = init_std or 1.0 / math.sqrt(dim)
            std2 = init_std or 1.0 / math.sqrt(hidden)
            self.w_gate_up.append(make_param(normal_((2 * hidden, dim), std1, seed + 1000 + 10 * ge, device, dtype)))
            self.w_down.append(make_param(normal_((dim, hidden), std2, seed + 1005 + 10 * ge, device, dtype)))
        self._comm: Optional[EpComm] = None
        self._tokens = tokens_per_rank
        self.aux_loss = None
        self._dropped = None

    def own_parameters(self):
        return [self.gate] + self.w_gate_up + self.w_down

    def expert_parameters(self):
        """Parameters that differ between ranks (they must not be averaged by data-parallel reduction)."""
        return self.w_gate_up + self.w_down

    @property
    def last_aux_loss(self):
        return self.aux_loss if self.aux_loss_coef else None

    def update_routing_bias(self) -> None:
        """Aux-loss-free balancing over the whole group: the routed-pair counts of every rank since the last call are
        summed, the bias of under-loaded experts rises by ``bias_update_rate`` and that of over-loaded ones falls
        (sign rule), then the counters reset (reference: lib/core/nn/moe.dart:550-569)."""
        load = self._expert_load.clone()
        if self.world > 1:
            dist.all_reduce(load, group=self.group)
        if float(load.sum()) > 0:
            self.routing_bias += self.bias_update_rate * torch.sign(load.mean() - load)
        self._expert_load.zero_()

    def _comm_for(self, T: int) -> EpComm:
        C = capacity(T, self.k, self.E, self.capacity_factor)
        if self._comm is None or self._comm.C != C:
            self._comm = EpComm(self.E, C, self.dim, self.group)
        return self._comm

    @property
    def last_dropped(self):
        """Routed (token, expert) pairs of the last forward that did not fit their expert's quota (synchronises)."""
        return None if self._dropped is None else int(self._dropped.item())

    def forward(self, x):
        shape = x.shape
        x2 = x.reshape(-1, self.dim)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        T = x2.shape[0]
        comm = self._comm_for(T)
        logits = F.linear(x2, self.gate)
        if self.routing_bias.device != x2.device:
            self.routing_bias = self.routing_bias.to(x2.device)
            self._expert_load = self._expert_load.to(x2.device)
        probs, idx, w = RouteFn.apply(logits, self.k, self.renorm, self.route_scale, self.gate_function,
                                      self.routing_bias, self.groups, self.top_groups)
        slot, count = slots(idx, self.E, comm.C)
        rows_in, counts_here = EpDispatchFn.apply(x2, comm, idx, slot, count)
        per = self.world * comm.C
        outs = []
        for le in range(self.El):
            r = rows_in[le * per:(le + 1) * per]
            h = F.swiglu(F.linear(r, self.w_gate_up[le]))
            outs.append(F.linear(h, self.w_down[le]))
        rows_out = outs[0] if self.El == 1 else torch.cat(outs, 0)
        y = EpCombineFn.apply(rows_out, w, comm, idx, slot, count, counts_here)
        # load-balance auxiliary loss: E * sum_e f_e * P_e, f_e from the routed (not yet capacity-clipped) pairs
        with torch.no_grad():
            flat = idx.reshape(-1).long()
            # (scatter_add, not bincount: bincount reads its output size back to the host, a synchronisation per layer)
            counts = torch.zeros(self.E, dtype=torch.float32, device=flat.device).scatter_add_(
                0, flat, torch.ones(flat.numel(), dtype=torch.float32, device=flat.device))
            self._expert_load += counts
            f = counts / float(T * self.k)
            self._dropped = (slot < 0).sum()      # read lazily (``last_dropped``): no host synchronisation per layer
        self.aux_loss = self.aux_loss_coef * self.E * (f * probs.mean(0)).sum()
        return y.reshape(shape)
