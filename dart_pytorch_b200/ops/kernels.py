"""Thin, allocation-explicit wrappers over the native kernels: torch tensors in, launch on the current stream.

No autograd here (see ``ops/cuda.py``); these are the calls the autograd functions, the optimizers and the
parallel layer share.  Every wrapper validates shapes on the host and raises on a non-zero return code.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .. import _native as N

# "gelu_tanh_d" applies the same GELU but writes the activation's derivative (not the pre-activation) to ``aux_out``;
# the matching backward code "mul" multiplies by ``aux_in`` as it is.  One tanh per element instead of two per step.
ACT_CODES = {None: 0, "none": 0, "relu": 1, "gelu_tanh": 2, "quick_gelu": 3, "silu": 4, "gelu_tanh_d": 5}
ACT_BWD_CODES = {"relu": 11, "gelu_tanh": 12, "quick_gelu": 13, "silu": 14, "mul": 15}


def _lead(t: torch.Tensor) -> int:
    """Leading dimension (elements) of a 2-D tensor whose last axis is contiguous."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise ValueError("expected a 2-D tensor with a contiguous last axis")
    return t.stride(0) if t.shape[0] > 1 else max(t.shape[1], t.stride(0))


_SPLITK_WS = {}
SPLITK_WS_BYTES = 64 << 20
SKINNY_MAX_ROWS = 64      # rows up to which x @ W^T takes the weight-streaming kernel (csrc/gemm_skinny.cu)
_SKINNY_ON = os.environ.get("DPTB200_SKINNY_GEMM", "1") != "0"
ERR_UNSUPPORTED = -5
SPLITK_COUNTERS = 4096


def splitk_workspace(device: torch.device):
    """Scratch of the split-K GEMM path, one per (device, stream): an fp32 partial-tile buffer and zeroed per-tile
    counters.  Launches on one stream reuse it in order (the counters return to zero at the end of every launch);
    GEMMs launched on another stream (weight gradients beside the data-gradient chain) get their own."""
    dev = device.index if device.index is not None else torch.cuda.current_device()
    key = (dev, torch.cuda.current_stream(dev).cuda_stream)
    ws = _SPLITK_WS.get(key)
    if ws is None:
        ws = (torch.empty(SPLITK_WS_BYTES, dtype=torch.uint8, device=device),
              torch.zeros(SPLITK_COUNTERS, dtype=torch.int32, device=device))
        _SPLITK_WS[key] = ws
    return ws


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
         bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
         aux_out: Optional[torch.Tensor] = None, aux_in: Optional[torch.Tensor] = None, act=None,
         act_bwd=None, accumulate: bool = False, alpha: float = 1.0, force_simt: bool = False, bn: int = 0,
         n_cols: Optional[int] = None, splits: int = 0) -> torch.Tensor:
    """``out[M,N] = epilogue(op(a) @ op(b))``.

    ``a`` is stored ``[M,K]`` (or ``[K,M]`` with ``trans_a``); ``b`` is stored ``[K,N]`` (or ``[N,K]`` with ``trans_b``,
    the layout of an ``nn.Linear`` weight).  All operands are 2-D with a contiguous last axis; row strides may exceed
    the row length (padded buffers).  ``n_cols`` restricts N below ``out.shape[1]``.
    Epilogue order: ``*alpha, +bias, aux_out<-value (or act'(value) with "gelu_tanh_d"), act, *act'(aux_in), +residual,
    (+out)``.
    """
    lib = N.load()
    if trans_a:
        K, M = a.shape
    else:
        M, K = a.shape
    if trans_b:
        Nn, Kb = b.shape
    else:
        Kb, Nn = b.shape
    if n_cols is not None:
        Nn = n_cols
    if Kb != K:
        raise ValueError(f"gemm: inner dimensions differ ({K} vs {Kb})")
    if out.shape[0] != M or out.shape[1] < Nn:
        raise ValueError(f"gemm: output is {tuple(out.shape)}, need [{M}, >={Nn}]")
    args = N.GemmArgs()
    args.A, args.B, args.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.lda, args.ldb, args.ldc = _lead(a), _lead(b), _lead(out)
    args.M, args.N, args.K = M, Nn, K
    args.trans_a, args.trans_b = int(trans_a), int(trans_b)
    args.a_f32 = int(a.dtype == torch.float32)
    args.b_f32 = int(b.dtype == torch.float32)
    for t in (a, b):
        if t.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError("gemm: inputs must be float32 or bfloat16")
    args.out_f32 = int(out.dtype == torch.float32)
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("gemm: output must be float32 or bfloat16")
    if bias is not None:
        if bias.numel() < Nn:
            raise ValueError("gemm: bias shorter than N")
        args.bias = bias.data_ptr()
        args.bias_f32 = int(bias.dtype == torch.float32)
    for name, t in (("residual", residual), ("aux_out", aux_out), ("aux_in", aux_in)):
        if t is not None:
            if t.dtype != torch.bfloat16:
                raise TypeError(f"gemm: {name} must be bfloat16")
            if t.shape[0] != M or t.shape[1] < Nn:
                raise ValueError(f"gemm: {name} has the wrong shape")
    if residual is not None:
        args.residual, args.ldr = residual.data_ptr(), _lead(residual)
    if aux_out is not None:
        args.aux_out, args.ld_aux_out = aux_out.data_ptr(), _lead(aux_out)
    if aux_in is not None:
        args.aux_in, args.ld_aux_in = aux_in.data_ptr(), _lead(aux_in)
    args.act = ACT_BWD_CODES[act_bwd] if act_bwd else ACT_CODES[act]
    args.accumulate = int(accumulate)
    args.alpha = alpha
    args.force_simt = int(force_simt)
    args.bn = bn
    args.splits = splits
    if splits != 1 and not force_simt:
        ws, counters = splitk_workspace(a.device)
        args.ws, args.ws_bytes = ws.data_ptr(), ws.numel()
        args.counters, args.num_counters = counters.data_ptr(), counters.numel()
    if M <= SKINNY_MAX_ROWS and trans_b and not trans_a and not force_simt and bn == 0 and _SKINNY_ON:
        # decode-sized rows: the weight-streaming kernel (declines, with "unsupported", what it does not cover)
        rc = lib.dptb_gemm_skinny(ctypes.byref(args), None, N.stream_ptr())
        if rc != ERR_UNSUPPORTED:
            N.check(rc, "gemm_skinny")
            return out
    N.check(lib.dptb_gemm(ctypes.byref(args), N.stream_ptr()), "gemm")
    return out


def norm_partial_rows() -> int:
    """Rows of the ``[rows, 2, D]`` fp32 scratch the norm backward kernels need."""
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count * 2


def layernorm_fwd(x, gamma, beta, eps):
    lib = N.load()
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    rows = x2.shape[0]
    y = torch.empty_like(x2)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    N.check(lib.dptb_layernorm_fwd(x2.data_ptr(), gamma.data_ptr(), N.ptr(beta), y.data_ptr(), mean.data_ptr(),
                                   rstd.data_ptr(), rows, D, eps, N.dtype_code(x2), N.stream_ptr()), "layernorm_fwd")
    return y.view(x.shape), mean, rstd


def layernorm_bwd(x, dy, gamma, mean, rstd, dres=None, dgamma=None, dbeta=None, accumulate=False, defer_reduce=False):
    """``defer_reduce``: launch only the kernel that writes ``dx`` and the per-CTA partials of the parameter gradients,
    and return a fourth value, a callable that launches their reduction into ``dgamma`` / ``dbeta`` on whatever stream
    is current when it is called (it keeps the partials alive; the caller orders that stream after this call)."""
    lib = N.load()
    D = x.shape[-1]
    x2, dy2 = x.reshape(-1, D), dy.reshape(-1, D)
    rows = x2.shape[0]
    dx = torch.empty_like(x2)
    if dgamma is None:
        dgamma = torch.empty_like(gamma)
        accumulate = False
    if dbeta is None:
        dbeta = torch.empty_like(gamma)
    prow = norm_partial_rows()
    partial = torch.empty(prow * 2 * D, dtype=torch.float32, device=x.device)
    nparts = ctypes.c_int(0)
    N.check(lib.dptb_layernorm_bwd(x2.data_ptr(), dy2.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                   N.ptr(None if dres is None else dres.reshape(-1, D)), dx.data_ptr(),
                                   dgamma.data_ptr(), dbeta.data_ptr(), partial.data_ptr(), prow, int(accumulate), rows,
                                   D, N.dtype_code(x2), N.stream_ptr(), int(defer_reduce), ctypes.byref(nparts)),
            "layernorm_bwd")
    if not defer_reduce:
        return dx.view(x.shape), dgamma, dbeta
    code = N.dtype_code(x2)

    def finish():
        N.check(lib.dptb_norm_param_grad_reduce(partial.data_ptr(), nparts.value, D, dgamma.data_ptr(), dbeta.data_ptr(),
                                                int(accumulate), code, N.stream_ptr()), "norm_param_grad_reduce")
    return dx.view(x.shape), dgamma, dbeta, finish


def rmsnorm_fwd(x, gamma, eps, out=None):
    lib = N.load()
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    rows = x2.shape[0]
    y = torch.empty_like(x2) if out is None else out.reshape(-1, D)
    if y.shape != x2.shape or y.dtype != x2.dtype or not y.is_contiguous():
        raise ValueError("rmsnorm_fwd: `out` must be a contiguous tensor of the input's shape and dtype")
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    N.check(lib.dptb_rmsnorm_fwd(x2.data_ptr(), gamma.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, D, eps,
                                 N.dtype_code(x2), N.stream_ptr()), "rmsnorm_fwd")
    return y.view(x.shape), rstd


def rmsnorm_bwd(x, dy, gamma, rstd, dres=None, dgamma=None, accumulate=False):
    lib = N.load()
    D = x.shape[-1]
    x2, dy2 = x.reshape(-1, D), dy.reshape(-1, D)
    rows = x2.shape[0]
    dx = torch.empty_like(x2)
    if dgamma is None:
        dgamma = torch.empty_like(gamma)
        accumulate = False
    prow = norm_partial_rows()
    partial = torch.empty(prow * 2 * D, dtype=torch.float32, device=x.device)
    N.check(lib.dptb_rmsnorm_bwd(x2.data_ptr(), dy2.data_ptr(), gamma.data_ptr(), rstd.data_ptr(),
                                 N.ptr(None if dres is None else dres.reshape(-1, D)), dx.data_ptr(), dgamma.data_ptr(),
                                 partial.data_ptr(), prow, int(accumulate), rows, D, N.dtype_code(x2), N.stream_ptr(),
                                 0, None),
            "rmsnorm_bwd")
    return dx.view(x.shape), dgamma


def ce_fwd(logits2d: torch.Tensor, targets: torch.Tensor, vocab: int):
    """Per-row loss and log-sum-exp over the first ``vocab`` columns of a (possibly padded) 2-D logits buffer."""
    lib = N.load()
    rows = logits2d.shape[0]
    loss = torch.empty(rows, dtype=torch.float32, device=logits2d.device)
    lse = torch.empty(rows, dtype=torch.float32, device=logits2d.device)
    N.check(lib.dptb_ce_fwd(logits2d.data_ptr(), _lead(logits2d), targets.data_ptr(), loss.data_ptr(), lse.data_ptr(),
                            rows, vocab, N.dtype_code(logits2d), N.stream_ptr()), "ce_fwd")
    return loss, lse


def ce_bwd(logits2d, targets, lse, g, scale: float, vocab: int, out=None, pad_to: Optional[int] = None):
    """``(softmax - onehot) * g[row] * scale`` written to ``out`` (default: in place over ``logits2d``)."""
    lib = N.load()
    rows = logits2d.shape[0]
    out = logits2d if out is None else out
    pad_to = vocab if pad_to is None else pad_to
    g_stride = 0 if g.numel() == 1 else 1
    N.check(lib.dptb_ce_bwd(logits2d.data_ptr(), _lead(logits2d), targets.data_ptr(), lse.data_ptr(), g.data_ptr(),
                            g_stride, scale, out.data_ptr(), _lead(out), rows, vocab, pad_to,
                            N.dtype_code(logits2d), N.stream_ptr()), "ce_bwd")
    return out


def softmax_fwd(x):
    lib = N.load()
    D = x.shape[-1]
    x2 = x.reshape(-1, D).contiguous()
    y = torch.empty_like(x2)
    N.check(lib.dptb_softmax_fwd(x2.data_ptr(), y.data_ptr(), x2.shape[0], D, N.dtype_code(x2), N.stream_ptr()),
            "softmax_fwd")
    return y.view(x.shape)


def softmax_bwd(y, dy):
    lib = N.load()
    D = y.shape[-1]
    y2, dy2 = y.reshape(-1, D).contiguous(), dy.reshape(-1, D).contiguous()
    dx = torch.empty_like(y2)
    N.check(lib.dptb_softmax_bwd(y2.data_ptr(), dy2.data_ptr(), dx.data_ptr(), y2.shape[0], D, N.dtype_code(y2),
                                 N.stream_ptr()), "softmax_bwd")
    return dx.view(y.shape)


def mean_f32(x: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    lib = N.load()
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    n = x.numel()
    N.check(lib.dptb_mean_f32(x.data_ptr(), n, out.data_ptr(), (1.0 / n) if scale is None else scale, N.stream_ptr()),
            "mean_f32")
    return out


def embedding_fwd(table, idx, pos_table=None, pos_start: int = 0, seq_len: int = 0):
    lib = N.load()
    idx = idx.contiguous()
    n, D = idx.numel(), table.shape[1]
    out = torch.empty(n, D, dtype=table.dtype, device=table.device)
    N.check(lib.dptb_embedding_fwd(table.data_ptr(), table.shape[0], idx.data_ptr(), N.ptr(pos_table),
                                   0 if pos_table is None else pos_table.shape[0], pos_start, seq_len, out.data_ptr(),
                                   n, D, N.dtype_code(table), N.stream_ptr()), "embedding_fwd")
    return out.view(*idx.shape, D)


def embedding_bwd(dtable, idx, dout, deterministic: bool = True):
    """``dtable[idx[n]] += dout[n]`` in place."""
    lib = N.load()
    idx = idx.reshape(-1).contiguous()
    n, D = idx.numel(), dtable.shape[1]
    dout2 = dout.reshape(n, D).contiguous()
    sidx = perm = None
    if deterministic:
        sidx, perm = torch.sort(idx, stable=True)
    N.check(lib.dptb_embedding_bwd(dtable.data_ptr(), dtable.shape[0], idx.data_ptr(), N.ptr(sidx), N.ptr(perm),
                                   dout2.data_ptr(), n, D, N.dtype_code(dtable), N.stream_ptr()), "embedding_bwd")
    return dtable


def pos_embedding_bwd(dpos, dout, pos_start: int, seq_len: int, batch: int):
    lib = N.load()
    D = dpos.shape[1]
    dout2 = dout.reshape(-1, D).contiguous()
    N.check(lib.dptb_pos_embedding_bwd(dpos.data_ptr(), dpos.shape[0], pos_start, seq_len, batch, dout2.data_ptr(), D,
                                       N.dtype_code(dpos), N.stream_ptr()), "pos_embedding_bwd")
    return dpos


def grad_norm(g_flat: torch.Tensor, ctrl: torch.Tensor, max_norm: float, partial: Optional[torch.Tensor] = None,
              add_previous: bool = False):
    """Global L2 norm of a flat gradient range into ``ctrl = [norm, scale, finite, sumsq]`` (fp32, device)."""
    lib = N.load()
    n = g_flat.numel()
    parts = lib.dptb_sqnorm_parts(n)
    if partial is None or partial.numel() < parts:
        partial = torch.empty(parts, dtype=torch.float32, device=g_flat.device)
    N.check(lib.dptb_grad_norm(g_flat.data_ptr(), n, N.dtype_code(g_flat), partial.data_ptr(), ctrl.data_ptr(),
                               float(max_norm), int(add_previous), N.stream_ptr()), "grad_norm")
    return ctrl


def scale_by_ctrl(g_flat, ctrl):
    lib = N.load()
    N.check(lib.dptb_scale_by_ctrl(g_flat.data_ptr(), g_flat.numel(), N.dtype_code(g_flat), ctrl.data_ptr(),
                                   N.stream_ptr()), "scale_by_ctrl")


def adam_flat(p, shadow, g, m, v, ctrl, lr, beta1, beta2, eps, weight_decay, bc1, bc2, skip_if_nonfinite=False,
              hyper=None):
    """``p`` is the fp32 master range, ``shadow`` the optional bf16 working copy written alongside."""
    lib = N.load()
    n = p.numel()
    if p.dtype != torch.float32 or m.dtype != torch.float32 or v.dtype != torch.float32:
        raise TypeError("adam_flat: p, m and v must be float32")
    if shadow is not None and (shadow.dtype != torch.bfloat16 or shadow.numel() != n):
        raise TypeError("adam_flat: shadow must be bfloat16 with p's length")
    if g.numel() != n or m.numel() != n or v.numel() != n:
        raise ValueError("adam_flat: g, m and v must have p's length")
    N.check(lib.dptb_adam_flat(p.data_ptr(), N.ptr(shadow), g.data_ptr(), N.dtype_code(g), m.data_ptr(), v.data_ptr(),
                               p.numel(), N.ptr(ctrl), lr, beta1, beta2, eps, weight_decay, bc1, bc2,
                               int(skip_if_nonfinite), N.ptr(hyper), N.stream_ptr()), "adam_flat")


def sgd_flat(p, shadow, g, buf, ctrl, lr, momentum, weight_decay, first_step):
    if p.dtype != torch.float32 or g.numel() != p.numel():
        raise TypeError("sgd_flat: p must be float32 and g must have p's length")
    if shadow is not None and (shadow.dtype != torch.bfloat16 or shadow.numel() != p.numel()):
        raise TypeError("sgd_flat: shadow must be bfloat16 with p's length")
    if buf is not None and (buf.dtype != torch.float32 or buf.numel() != p.numel()):
        raise TypeError("sgd_flat: buf must be float32 with p's length")
    lib = N.load()
    N.check(lib.dptb_sgd_flat(p.data_ptr(), N.ptr(shadow), g.data_ptr(), N.dtype_code(g), N.ptr(buf), p.numel(),
                              N.ptr(ctrl), lr, momentum, weight_decay, int(first_step), N.stream_ptr()), "sgd_flat")


# --------------------------------------------------------------------------- elementwise / reductions / misc
BINARY_OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3}
UNARY_OPS = {"relu": 0, "sigmoid": 1, "tanh": 2, "abs": 3, "log": 4, "pow": 5, "gelu_tanh": 6, "quick_gelu": 7,
             "silu": 8, "scale": 9, "exp": 10, "neg": 11, "sqrt": 12, "add_scalar": 13}


def binary(a: torch.Tensor, b: torch.Tensor, op: str) -> torch.Tensor:
    """Same-shape, scalar (either side) or ``[M,N] op [N]`` row broadcast
    (reference broadcast rules: lib/core/tensor/ops.dart:207-254)."""
    lib = N.load()
    a, b = a.contiguous(), b.contiguous()
    if a.numel() == b.numel():
        mode, big, cols = 0, a, 1
    elif b.numel() == 1:
        mode, big, cols = 1, a, 1
    elif a.numel() == 1:
        mode, big, cols = 3, b, 1
    elif a.dim() >= 2 and b.numel() == a.shape[-1]:
        mode, big, cols = 2, a, a.shape[-1]
    else:
        raise ValueError(f"binary {op}: shapes {tuple(a.shape)} and {tuple(b.shape)} do not broadcast")
    out = torch.empty_like(big)
    N.check(lib.dptb_binary(a.data_ptr(), b.data_ptr(), out.data_ptr(), big.numel(), cols, BINARY_OPS[op], mode,
                            N.dtype_code(big), N.stream_ptr()), f"binary_{op}")
    return out


def unary(x: torch.Tensor, op: str, param: float = 0.0) -> torch.Tensor:
    lib = N.load()
    x = x.contiguous()
    out = torch.empty_like(x)
    N.check(lib.dptb_unary(x.data_ptr(), out.data_ptr(), x.numel(), UNARY_OPS[op], float(param), N.dtype_code(x),
                           N.stream_ptr()), f"unary_{op}")
    return out


def unary_bwd(x: torch.Tensor, dy: torch.Tensor, op: str, param: float = 0.0) -> torch.Tensor:
    lib = N.load()
    x, dy = x.contiguous(), dy.contiguous()
    dx = torch.empty_like(x)
    N.check(lib.dptb_unary_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.numel(), UNARY_OPS[op], float(param),
                               N.dtype_code(x), N.stream_ptr()), f"unary_bwd_{op}")
    return dx


def colsum(x2d: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False, n_cols=None):
    """Column sums of a 2-D tensor (bias gradients), deterministic: fixed row slices, folded in slice order."""
    lib = N.load()
    rows = x2d.shape[0]
    cols = x2d.shape[1] if n_cols is None else n_cols
    if out is None:
        out = torch.empty(cols, dtype=x2d.dtype, device=x2d.device)
        accumulate = False
    if x2d.dtype == torch.bfloat16 and cols % 8 == 0:
        # 16-byte path: about four 256-column CTAs per SM, at least 32 rows each
        nparts = max(1, min(256, 592 // ((cols + 255) // 256), (rows + 31) // 32))
    else:
        nparts = max(1, min(48, (rows + 255) // 256))
    partial = torch.empty(nparts * cols, dtype=torch.float32, device=x2d.device)
    N.check(lib.dptb_colsum(x2d.data_ptr(), _lead(x2d), out.data_ptr(), partial.data_ptr(), rows, cols, nparts,
                            int(accumulate), N.dtype_code(x2d), N.stream_ptr()), "colsum")
    return out


def sum_all(x: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    lib = N.load()
    x = x.contiguous()
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    partial = torch.empty(148 * 16 * 2, dtype=torch.float32, device=x.device)
    N.check(lib.dptb_sum_all(x.data_ptr(), x.numel(), out.data_ptr(), partial.data_ptr(), float(scale),
                             N.dtype_code(x), N.stream_ptr()), "sum_all")
    return out


def transpose2d(x: torch.Tensor) -> torch.Tensor:
    lib = N.load()
    x = x.contiguous()
    rows, cols = x.shape
    out = torch.empty(cols, rows, dtype=x.dtype, device=x.device)
    N.check(lib.dptb_transpose2d(x.data_ptr(), out.data_ptr(), rows, cols, N.dtype_code(x), N.stream_ptr()),
            "transpose2d")
    return out


def copy2d(src: torch.Tensor, dst: torch.Tensor, rows: int, cols: int):
    lib = N.load()
    N.check(lib.dptb_copy2d(src.data_ptr(), _lead(src), dst.data_ptr(), _lead(dst), rows, cols, N.dtype_code(src),
                            N.stream_ptr()), "copy2d")
    return dst


def copy_flat(src: torch.Tensor, dst: torch.Tensor, grid: int = 0):
    """``dst[:] = src[:]`` for contiguous tensors of equal byte size (a multiple of 16), by a kernel that keeps eight
    16-byte loads in flight per thread; either side may be another GPU's memory mapped into this process."""
    lib = N.load()
    nbytes = src.numel() * src.element_size()
    if nbytes != dst.numel() * dst.element_size() or not (src.is_contiguous() and dst.is_contiguous()):
        raise ValueError("copy_flat: contiguous tensors of equal byte size")
    lib.dptb_copy_flat.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p]
    lib.dptb_copy_flat.restype = ctypes.c_int
    N.check(lib.dptb_copy_flat(src.data_ptr(), dst.data_ptr(), nbytes, grid, N.stream_ptr()), "copy_flat")
    return dst


def rope(x2d: torch.Tensor, heads: int, head_dim: int, rotary_dim: int, seq_len: int, pos_start: int, base: float,
         inverse: bool = False, out: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None,
         col_offset: int = 0):
    """Rotate ``heads`` consecutive heads starting at column ``col_offset`` of every row of ``x2d`` (row = token)."""
    lib = N.load()
    out = x2d if out is None else out
    esz = x2d.element_size()
    N.check(lib.dptb_rope(x2d.data_ptr() + col_offset * esz, out.data_ptr() + col_offset * esz, x2d.shape[0], heads,
                          head_dim, rotary_dim, seq_len, pos_start, float(base), int(inverse), N.dtype_code(x2d),
                          _lead(x2d), _lead(out), N.ptr(positions), N.stream_ptr()), "rope")
    return out


def dropout(x: torch.Tensor, p: float, seed: int, offset: int) -> torch.Tensor:
    lib = N.load()
    x = x.contiguous()
    out = torch.empty_like(x)
    N.check(lib.dptb_dropout(x.data_ptr(), out.data_ptr(), x.numel(), float(p), seed, offset, N.dtype_code(x),
                             N.stream_ptr()), "dropout")
    return out


def swiglu_fwd(g: torch.Tensor, u: torch.Tensor, out: Optional[torch.Tensor] = None):
    lib = N.load()
    rows, cols = g.shape
    if out is None:
        out = torch.empty(rows, cols, dtype=g.dtype, device=g.device)
    N.check(lib.dptb_swiglu_fwd(g.data_ptr(), _lead(g), u.data_ptr(), _lead(u), out.data_ptr(), _lead(out), rows, cols,
                                N.dtype_code(g), N.stream_ptr()), "swiglu_fwd")
    return out


def swiglu_bwd(g, u, dout, dg, du):
    lib = N.load()
    rows, cols = g.shape
    N.check(lib.dptb_swiglu_bwd(g.data_ptr(), _lead(g), u.data_ptr(), _lead(u), dout.data_ptr(), _lead(dout),
                                dg.data_ptr(), _lead(dg), du.data_ptr(), _lead(du), rows, cols, N.dtype_code(g),
                                N.stream_ptr()), "swiglu_bwd")
    return dg, du


def argmax_rows(x2d: torch.Tensor, n_cols: Optional[int] = None) -> torch.Tensor:
    lib = N.load()
    rows = x2d.shape[0]
    cols = x2d.shape[1] if n_cols is None else n_cols
    out = torch.empty(rows, dtype=torch.long, device=x2d.device)
    N.check(lib.dptb_argmax_rows(x2d.data_ptr(), _lead(x2d), out.data_ptr(), rows, cols, N.dtype_code(x2d),
                                 N.stream_ptr()), "argmax_rows")
    return out


def topk_sample(x2d: torch.Tensor, u: torch.Tensor, k: int, temperature: float, n_cols: Optional[int] = None):
    lib = N.load()
    rows = x2d.shape[0]
    cols = x2d.shape[1] if n_cols is None else n_cols
    out = torch.empty(rows, dtype=torch.long, device=x2d.device)
    N.check(lib.dptb_topk_sample(x2d.data_ptr(), _lead(x2d), u.data_ptr(), out.data_ptr(), rows, cols, k,
                                 float(temperature), N.dtype_code(x2d), 0, N.stream_ptr()), "topk_sample")
    return out


def im2col_nhwc(x: torch.Tensor, batch: int, channels: int, ksize: int, board: int = 8):
    lib = N.load()
    x = x.contiguous()
    out = torch.empty(batch * board * board, channels * ksize * ksize, dtype=x.dtype, device=x.device)
    N.check(lib.dptb_im2col_nhwc(x.data_ptr(), out.data_ptr(), batch, channels, ksize, board, N.dtype_code(x),
                                 N.stream_ptr()), "im2col_nhwc")
    return out


def conv_out_size(size: int, k: int, stride: int, pad: int) -> int:
    return (size + 2 * pad - k) // stride + 1


def im2col_nchw(x: torch.Tensor, kh: int, kw: int, stride: int, pad: int) -> torch.Tensor:
    """``[B, C, H, W]`` -> ``[B*Ho*Wo, C*kh*kw]`` rows, column order ``(c, ky, kx)``, zero padding."""
    lib = N.load()
    x = x.contiguous()
    B, C, H, W = x.shape
    ho, wo = conv_out_size(H, kh, stride, pad), conv_out_size(W, kw, stride, pad)
    out = torch.empty(B * ho * wo, C * kh * kw, dtype=x.dtype, device=x.device)
    N.check(lib.dptb_conv_lower(x.data_ptr(), out.data_ptr(), B, C, H, W, kh, kw, stride, pad, 0, N.dtype_code(x),
                                N.stream_ptr()), "im2col_nchw")
    return out


def col2im_nchw(cols: torch.Tensor, shape, kh: int, kw: int, stride: int, pad: int) -> torch.Tensor:
    """Adjoint of :func:`im2col_nchw`: scatter-sums column gradients back to a ``[B, C, H, W]`` image gradient."""
    lib = N.load()
    cols = cols.contiguous()
    B, C, H, W = shape
    out = torch.empty(B, C, H, W, dtype=cols.dtype, device=cols.device)
    N.check(lib.dptb_conv_lower(cols.data_ptr(), out.data_ptr(), B, C, H, W, kh, kw, stride, pad, 1,
                                N.dtype_code(cols), N.stream_ptr()), "col2im_nchw")
    return out


def patchify(img: torch.Tensor, patch: int, out_dtype=None) -> torch.Tensor:
    """``[B, C, H, W]`` image -> ``[B * (H/P) * (W/P), P*P*C]`` rows with per-patch order ``(dy, dx, c)``."""
    lib = N.load()
    img = img.contiguous()
    B, C, H, W = img.shape
    out_dtype = out_dtype or img.dtype
    out = torch.empty(B * (H // patch) * (W // patch), patch * patch * C, dtype=out_dtype, device=img.device)
    code = int(img.dtype == torch.bfloat16) + 2 * int(out_dtype == torch.bfloat16)
    N.check(lib.dptb_patchify(img.data_ptr(), out.data_ptr(), B, C, H, W, patch, code, N.stream_ptr()), "patchify")
    return out
