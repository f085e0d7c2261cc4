"""Autograd functions whose forward and backward are the native sm_100a kernels.

Each function is the device counterpart of a reference tensor op (lib/core/tensor/*.dart); where the reference
composes a backward from many forward ops, the backward here is one or two fused kernels.  Parameter gradients
can be written straight into a preallocated ``.grad`` (see ``utils/arena.py``): the weight-gradient GEMM then
accumulates in its epilogue and autograd receives ``None`` for that input.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from . import kernels as K

VOCAB_PAD = 128  # logits buffers are padded to a multiple of this many columns

_rng_state = {"seed": 0x5EED, "offset": 0}


def manual_seed(seed: int) -> None:
    _rng_state["seed"] = int(seed) & 0xFFFFFFFFFFFFFFFF
    _rng_state["offset"] = 0


_grad_listener = None


def set_grad_listener(listener) -> None:
    """``listener.touch(p)`` is called whenever a backward kernel is about to accumulate into ``p``'s arena gradient
    (data-parallel overlap uses it to learn when a bucket is final)."""
    global _grad_listener
    _grad_listener = listener


def _direct_grad(p: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """The preallocated gradient buffer of ``p`` if it takes in-kernel accumulation, else None."""
    if p is None or not getattr(p, "_dptb_direct_grad", False):
        return None
    if _grad_listener is not None:
        _grad_listener.touch(p)
    return p.grad


def _as2d(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    return x2 if x2.is_contiguous() else x2.contiguous()


def _is_bf16(*ts) -> bool:
    return all(t is None or t.dtype == torch.bfloat16 for t in ts)


# --------------------------------------------------------------------------- linear / mlp
def _weight_grad(dy2: torch.Tensor, x2: torch.Tensor, w: torch.Tensor, needs: bool):
    """dW[N,K] = dy2^T @ x2, into the direct-grad buffer when there is one."""
    if not needs:
        return None
    tgt = _direct_grad(w)
    if tgt is not None:
        K.gemm(dy2, x2, tgt, trans_a=True, accumulate=True)
        return None
    dw = torch.empty_like(w)
    K.gemm(dy2, x2, dw, trans_a=True)
    return dw


# Parameter-gradient tails on a side stream.  The column sums of an upstream gradient (bias gradients) and the reduction
# of the norm layers' per-CTA partials into dgamma / dbeta are memory-bound and nothing in the backward pass waits for
# them, while the GEMMs beside them are compute-bound.  They are launched on a side stream forked from the current one:
# the bias sums are joined after the GEMMs of their own autograd node, the norm reductions at the next such join or at
# the end of the backward pass (engine callback), so both run on the SMs that a GEMM's last wave leaves idle.  Measured on
# the GPT-2 step, same box: 20.83 -> 20.79 ms with the bias sums alone (within noise), -> 20.53 ms with the norm
# reductions as well; on 2 GPUs 21.55 -> 21.0 ms.  Only gradients accumulated straight into an optimizer arena take this
# path (no tensor changes streams).  Moving the weight-gradient GEMMs there too gained less: two persistent GEMMs then
# compete for the same SMs.  DPTB200_GRAD_SIDE_STREAM=0 turns all of it off, DPTB200_NORM_DEFER=0 the norm part.
_GRAD_SIDE = os.environ.get("DPTB200_GRAD_SIDE_STREAM", "1") != "0"
_NORM_DEFER = os.environ.get("DPTB200_NORM_DEFER", "1") != "0"      # the norm parameter-gradient reduction as well
_side_streams = {}


class _ParamGradFork:
    """``with`` block whose body runs on the side stream, after everything queued on the current stream so far;
    ``join()`` makes the current stream wait for it."""

    def __init__(self, device):
        self.cur = torch.cuda.current_stream(device)
        key = device.index
        side = _side_streams.get(key)
        if side is None:
            side = _side_streams[key] = torch.cuda.Stream(device=device)
        self.side = side
        self.used = False

    def __enter__(self):
        self.side.wait_stream(self.cur)
        self.used = True
        self._ctx = torch.cuda.stream(self.side)
        self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        return self._ctx.__exit__(*exc)

    def join(self):
        if self.used:
            self.cur.wait_stream(self.side)


_deferred = {"gen": 0, "forks": {}, "keep": []}


def _defer_to_side(device, launch) -> None:
    """Runs ``launch()`` on the side stream, ordered after everything queued on the current stream, WITHOUT joining:
    the side stream runs in order, so the next ``_ParamGradFork.join()`` on this device covers it, and a callback at the
    end of the backward pass joins whatever is still open (the optimizer and a graph capture see one stream again).
    ``launch`` is kept alive until that join: it owns the scratch its kernel reads."""
    fork = _ParamGradFork(device)
    with fork:
        launch()
    _deferred["forks"][device.index] = fork
    _deferred["keep"].append(launch)
    gen = _deferred["gen"]
    torch.autograd.Variable._execution_engine.queue_callback(lambda: _join_deferred(gen))


def _join_deferred(gen: int) -> None:
    if gen != _deferred["gen"]:
        return                       # an earlier callback of this backward pass has joined already
    _deferred["gen"] += 1
    for fork in _deferred["forks"].values():
        fork.join()
    _deferred["forks"].clear()
    _deferred["keep"].clear()


def param_side_stream(device) -> Optional["torch.cuda.Stream"]:
    """The side stream parameter-gradient kernels of ``device`` may be running on (None if none was made yet): a
    consumer of gradients that runs before the end of the backward pass orders itself after it."""
    return _side_streams.get(device.index if device.index is not None else torch.cuda.current_device())


def _bias_grad_fork(dy2, b, needs: bool, fork: Optional[_ParamGradFork]):
    """The bias gradient, on the fork's side stream when it accumulates straight into an arena (returns None then, as
    ``_bias_grad`` does for such a parameter)."""
    if fork is None or b is None or not needs or _direct_grad(b) is None:
        return _bias_grad(dy2, b, needs)
    with fork:
        _bias_grad(dy2, b, needs)
    return None


def _bias_grad(dy2: torch.Tensor, b: Optional[torch.Tensor], needs: bool):
    if b is None or not needs:
        return None
    tgt = _direct_grad(b)
    if tgt is not None:
        K.colsum(dy2, out=tgt.view(-1), accumulate=True)
        return None
    return K.colsum(dy2).to(b.dtype).view(b.shape)


class LinearFn(torch.autograd.Function):
    """``act(x @ w.T + b) + residual`` with everything after the GEMM done in its epilogue (bf16)."""

    @staticmethod
    def forward(ctx, x, w, b, act, residual):
        x2 = _as2d(x)
        M, Nn = x2.shape[0], w.shape[0]
        out = torch.empty(M, Nn, dtype=x.dtype, device=x.device)
        fused = _is_bf16(x2, w, residual)
        pre = None
        if fused:
            pre = torch.empty_like(out) if act else None
            K.gemm(x2, w, out, trans_b=True, bias=None if b is None else b.view(-1), act=act, aux_out=pre,
                   residual=None if residual is None else _as2d(residual))
        else:
            K.gemm(x2, w, out, trans_b=True, bias=None if b is None else b.view(-1))
            if act:
                pre = out
                out = K.unary(pre, act)
            if residual is not None:
                out = K.binary(out, _as2d(residual), "add")
        ctx.save_for_backward(x2, pre)
        ctx.w, ctx.b, ctx.act = w, b, act
        ctx.has_res = residual is not None
        ctx.xshape = x.shape
        # A 2-D input gets the fresh buffer itself, not a view of it: in-place consumers (the rotary embedding of the
        # fused QKV output) may not modify a view created inside a custom Function.
        return out if x.dim() == 2 else out.view(*x.shape[:-1], Nn)

    @staticmethod
    def backward(ctx, dy):
        x2, pre = ctx.saved_tensors
        w, b, act = ctx.w, ctx.b, ctx.act
        dy2 = _as2d(dy)
        dpre = K.unary_bwd(pre, dy2, act) if act else dy2
        fork = _ParamGradFork(dy2.device) if (_GRAD_SIDE and dy2.is_cuda) else None
        db = _bias_grad_fork(dpre, b, ctx.needs_input_grad[2], fork)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x2)
            K.gemm(dpre, w, dx)
            dx = dx.view(ctx.xshape)
        dw = _weight_grad(dpre, x2, w, ctx.needs_input_grad[1])
        if fork is not None:
            fork.join()
        dres = dy if ctx.has_res and ctx.needs_input_grad[4] else None
        return dx, dw, db, None, dres


class MLPFn(torch.autograd.Function):
    """``act(x @ w1.T + b1) @ w2.T + b2 (+ residual)`` as two GEMMs forward and four backward.

    The activation derivative rides in the epilogue of the second layer's data-gradient GEMM, so no standalone
    elementwise kernel runs in either direction.
    """

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, act, residual):
        x2 = _as2d(x)
        M, F, D = x2.shape[0], w1.shape[0], w2.shape[0]
        # For GELU the saved tensor is the derivative at the pre-activation (computed beside the activation from the
        # same tanh), so the backward epilogue is one multiply; other activations save the pre-activation itself.
        pre = torch.empty(M, F, dtype=x.dtype, device=x.device)
        a = torch.empty_like(pre)
        fwd_act = "gelu_tanh_d" if act == "gelu_tanh" else act
        K.gemm(x2, w1, a, trans_b=True, bias=None if b1 is None else b1.view(-1), act=fwd_act, aux_out=pre)
        out = torch.empty(M, D, dtype=x.dtype, device=x.device)
        K.gemm(a, w2, out, trans_b=True, bias=None if b2 is None else b2.view(-1),
               residual=None if residual is None else _as2d(residual))
        ctx.save_for_backward(x2, pre, a)
        ctx.params = (w1, b1, w2, b2)
        ctx.act = act
        ctx.has_res = residual is not None
        ctx.xshape = x.shape
        return out.view(*x.shape[:-1], D)

    @staticmethod
    def backward(ctx, dy):
        x2, pre, a = ctx.saved_tensors
        w1, b1, w2, b2 = ctx.params
        dy2 = _as2d(dy)
        dpre = torch.empty_like(pre)
        fork = _ParamGradFork(dy2.device) if (_GRAD_SIDE and dy2.is_cuda) else None
        db2 = _bias_grad_fork(dy2, b2, ctx.needs_input_grad[4], fork)       # beside the next two GEMMs
        K.gemm(dy2, w2, dpre, aux_in=pre, act_bwd="mul" if ctx.act == "gelu_tanh" else ctx.act)
        dw2 = _weight_grad(dy2, a, w2, ctx.needs_input_grad[3])
        if fork is not None:
            fork.join()
        db1 = _bias_grad_fork(dpre, b1, ctx.needs_input_grad[2], fork)      # dpre is complete: beside the last two
        dw1 = _weight_grad(dpre, x2, w1, ctx.needs_input_grad[1])
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x2)
            K.gemm(dpre, w1, dx)
            dx = dx.view(ctx.xshape)
        if fork is not None:
            fork.join()
        dres = dy if ctx.has_res and ctx.needs_input_grad[6] else None
        return dx, dw1, db1, dw2, db2, None, dres


class MatmulFn(torch.autograd.Function):
    """``a[M,K] @ b[K,N]`` (reference: lib/core/tensor/mat_mul.dart:12-93)."""

    @staticmethod
    def forward(ctx, a, b):
        a2 = _as2d(a)
        b2 = b if b.is_contiguous() else b.contiguous()
        out = torch.empty(a2.shape[0], b2.shape[1], dtype=a.dtype, device=a.device)
        K.gemm(a2, b2, out)
        ctx.save_for_backward(a2, b2)
        ctx.ashape = a.shape
        return out.view(*a.shape[:-1], b2.shape[1])

    @staticmethod
    def backward(ctx, dy):
        a2, b2 = ctx.saved_tensors
        dy2 = _as2d(dy)
        da = db = None
        if ctx.needs_input_grad[0]:
            da = torch.empty_like(a2)
            K.gemm(dy2, b2, da, trans_b=True)  # dy @ b^T : b stored [K,N] = [N', K'] with N'=K
            da = da.view(ctx.ashape)
        if ctx.needs_input_grad[1]:
            db = torch.empty_like(b2)
            K.gemm(a2, dy2, db, trans_a=True)  # a^T @ dy
        return da, db


# --------------------------------------------------------------------------- norms
class LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, passthrough):
        xc = x if x.is_contiguous() else x.contiguous()
        y, mean, rstd = K.layernorm_fwd(xc, gamma, beta, eps)
        ctx.save_for_backward(xc, mean, rstd)
        ctx.gamma, ctx.beta = gamma, beta
        ctx.passthrough = passthrough
        if passthrough:
            return x.view_as(x), y
        return y

    @staticmethod
    def backward(ctx, *grads):
        xc, mean, rstd = ctx.saved_tensors
        gamma, beta = ctx.gamma, ctx.beta
        if ctx.passthrough:
            dres, dy = grads
        else:
            dres, dy = None, grads[0]
        if dy is None:
            return dres, None, None, None, None
        dy = dy if dy.is_contiguous() else dy.contiguous()
        if dres is not None and not dres.is_contiguous():
            dres = dres.contiguous()
        tg, tb = _direct_grad(gamma), _direct_grad(beta)
        if tg is not None and (beta is None or tb is not None):
            if _GRAD_SIDE and _NORM_DEFER and tb is not None:
                # dx is what the backward pass waits for; the reduction of the parameter-gradient partials goes to
                # the side stream, beside the GEMMs of the autograd node that follows
                dx, _, _, finish = K.layernorm_bwd(xc, dy, gamma, mean, rstd, dres=dres, dgamma=tg, dbeta=tb,
                                                   accumulate=True, defer_reduce=True)
                _defer_to_side(dy.device, finish)
                return dx, None, None, None, None
            dx, _, _ = K.layernorm_bwd(xc, dy, gamma, mean, rstd, dres=dres, dgamma=tg, dbeta=tb, accumulate=True)
            return dx, None, None, None, None
        dx, dg, db = K.layernorm_bwd(xc, dy, gamma, mean, rstd, dres=dres)
        return dx, dg, (db if beta is not None else None), None, None


class RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, eps, passthrough):
        xc = x if x.is_contiguous() else x.contiguous()
        y, rstd = K.rmsnorm_fwd(xc, gamma, eps)
        ctx.save_for_backward(xc, rstd)
        ctx.gamma = gamma
        ctx.passthrough = passthrough
        if passthrough:
            return x.view_as(x), y
        return y

    @staticmethod
    def backward(ctx, *grads):
        xc, rstd = ctx.saved_tensors
        gamma = ctx.gamma
        if ctx.passthrough:
            dres, dy = grads
        else:
            dres, dy = None, grads[0]
        if dy is None:
            return dres, None, None, None
        dy = dy if dy.is_contiguous() else dy.contiguous()
        if dres is not None and not dres.is_contiguous():
            dres = dres.contiguous()
        tg = _direct_grad(gamma)
        if tg is not None:
            dx, _ = K.rmsnorm_bwd(xc, dy, gamma, rstd, dres=dres, dgamma=tg, accumulate=True)
            return dx, None, None, None
        dx, dg = K.rmsnorm_bwd(xc, dy, gamma, rstd, dres=dres)
        return dx, dg, None, None


# --------------------------------------------------------------------------- softmax / cross-entropy
class SoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        y = K.softmax_fwd(x)
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        return K.softmax_bwd(y, dy)


class CrossEntropyFn(torch.autograd.Function):
    """Per-row loss ``[R, 1]`` (fp32) from logits ``[R, V]``; the backward never materialises probabilities."""

    @staticmethod
    def forward(ctx, logits, targets):
        V = logits.shape[-1]
        l2 = _as2d(logits)
        tgt = targets.reshape(-1).to(torch.long)
        loss, lse = K.ce_fwd(l2, tgt, V)
        ctx.save_for_backward(l2, tgt, lse)
        ctx.lshape = logits.shape
        return loss.view(-1, 1)

    @staticmethod
    def backward(ctx, dloss):
        l2, tgt, lse = ctx.saved_tensors
        g = dloss.reshape(-1).float().contiguous()
        d = torch.empty_like(l2)
        K.ce_bwd(l2, tgt, lse, g, 1.0, l2.shape[1], out=d)
        return d.view(ctx.lshape), None


class LMHeadLossFn(torch.autograd.Function):
    """Mean cross-entropy of ``h @ w.T`` against ``targets`` without keeping logits for the backward in a second
    buffer: the (padded) logits buffer is overwritten in place by its own gradient, which then feeds the two
    gradient GEMMs."""

    @staticmethod
    def forward(ctx, h, w, targets):
        h2 = _as2d(h)
        M, V = h2.shape[0], w.shape[0]
        vpad = (V + VOCAB_PAD - 1) // VOCAB_PAD * VOCAB_PAD
        logits = torch.empty(M, vpad, dtype=h.dtype, device=h.device)
        K.gemm(h2, w, logits, trans_b=True, n_cols=V)
        tgt = targets.reshape(-1).to(torch.long)
        loss_rows, lse = K.ce_fwd(logits, tgt, V)
        loss = K.mean_f32(loss_rows)
        ctx.save_for_backward(h2, logits, tgt, lse)
        ctx.w = w
        ctx.hshape = h.shape
        return loss.view(())

    @staticmethod
    def backward(ctx, g):
        h2, logits, tgt, lse = ctx.saved_tensors
        w = ctx.w
        M, V = h2.shape[0], w.shape[0]
        gg = g.reshape(1).float().contiguous()
        K.ce_bwd(logits, tgt, lse, gg, 1.0 / M, V, pad_to=logits.shape[1])  # in place
        dl = logits[:, :V]
        dh = None
        if ctx.needs_input_grad[0]:
            dh = torch.empty_like(h2)
            K.gemm(dl, w, dh)
            dh = dh.view(ctx.hshape)
        dw = _weight_grad(dl, h2, w, ctx.needs_input_grad[1])
        return dh, dw, None


# --------------------------------------------------------------------------- embedding
class EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, idx, pos_table, pos_start):
        idx = idx.to(torch.long) if not idx.is_floating_point() else torch.floor(idx + 0.5).to(torch.long)
        seq_len = idx.shape[-1] if idx.dim() >= 1 else 1
        out = K.embedding_fwd(table, idx, pos_table=pos_table, pos_start=pos_start, seq_len=seq_len)
        ctx.save_for_backward(idx)
        ctx.table, ctx.pos_table, ctx.pos_start, ctx.seq_len = table, pos_table, pos_start, seq_len
        return out

    @staticmethod
    def backward(ctx, dout):
        (idx,) = ctx.saved_tensors
        table, pos_table = ctx.table, ctx.pos_table
        dout = dout if dout.is_contiguous() else dout.contiguous()
        dt = dp = None
        if ctx.needs_input_grad[0]:
            tgt = _direct_grad(table)
            if tgt is not None:
                K.embedding_bwd(tgt, idx, dout)
            else:
                dt = torch.zeros_like(table)
                K.embedding_bwd(dt, idx, dout)
        if pos_table is not None and ctx.needs_input_grad[2]:
            batch = idx.numel() // max(1, ctx.seq_len)
            tgt = _direct_grad(pos_table)
            if tgt is not None:
                K.pos_embedding_bwd(tgt, dout, ctx.pos_start, ctx.seq_len, batch)
            else:
                dp = torch.zeros_like(pos_table)
                K.pos_embedding_bwd(dp, dout, ctx.pos_start, ctx.seq_len, batch)
        return dt, None, dp, None


class ScatterRowsAddFn(torch.autograd.Function):
    """``out[idx[n]] += rows[n]`` into zeros ``[total, D]``; the backward is a gather (reference: scatter.dart:20-85)."""

    @staticmethod
    def forward(ctx, rows, idx, total):
        idx = idx.to(torch.long) if not idx.is_floating_point() else torch.floor(idx + 0.5).to(torch.long)
        out = torch.zeros(total, rows.shape[-1], dtype=rows.dtype, device=rows.device)
        K.embedding_bwd(out, idx, rows)
        ctx.save_for_backward(idx)
        return out

    @staticmethod
    def backward(ctx, dout):
        (idx,) = ctx.saved_tensors
        return K.embedding_fwd(dout.contiguous(), idx.reshape(-1)), None, None


# --------------------------------------------------------------------------- elementwise
class UnaryFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op, param):
        ctx.save_for_backward(x)
        ctx.op, ctx.param = op, param
        return K.unary(x, op, param).view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return K.unary_bwd(x, dy, ctx.op, ctx.param).view(x.shape), None, None


def _reduce_like(g: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    """Sum a broadcast gradient back to the operand's shape (scalar, or a row broadcast over rows)."""
    if g.shape == like.shape:
        return g
    if like.numel() == 1:
        return K.sum_all(g).to(g.dtype).view(like.shape)
    return K.colsum(_as2d(g)).view(like.shape)


class BinaryFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, op):
        ctx.save_for_backward(a, b)
        ctx.op = op
        return K.binary(a, b, op)

    @staticmethod
    def backward(ctx, dy):
        a, b = ctx.saved_tensors
        op = ctx.op
        da = db = None
        if op == "add":
            da, db = dy, dy
        elif op == "sub":
            da, db = dy, K.unary(dy, "neg")
        elif op == "mul":
            da, db = K.binary(dy, b, "mul"), K.binary(dy, a, "mul")
        else:  # a / b
            da = K.binary(dy, b, "div")
            db = K.unary(K.binary(K.binary(da, a, "mul"), b, "div"), "neg")
        if ctx.needs_input_grad[0]:
            da = _reduce_like(da, a)
        else:
            da = None
        if ctx.needs_input_grad[1]:
            db = _reduce_like(db, b)
        else:
            db = None
        return da, db, None


class SumFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mean):
        ctx.xshape, ctx.n, ctx.mean, ctx.dtype = x.shape, x.numel(), mean, x.dtype
        return K.sum_all(x, 1.0 / x.numel() if mean else 1.0).to(x.dtype).view(1, 1)

    @staticmethod
    def backward(ctx, g):
        scale = 1.0 / ctx.n if ctx.mean else 1.0
        return (g.reshape(1).to(ctx.dtype) * scale).expand(ctx.n).reshape(ctx.xshape).contiguous(), None


class TransposeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return K.transpose2d(x)

    @staticmethod
    def backward(ctx, dy):
        return K.transpose2d(dy)


class DropoutFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p):
        ctx.p, ctx.seed, ctx.offset = p, _rng_state["seed"], _rng_state["offset"]
        _rng_state["offset"] += x.numel()
        return K.dropout(x, p, ctx.seed, ctx.offset).view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        return K.dropout(dy, ctx.p, ctx.seed, ctx.offset).view(dy.shape), None


class RopeFn(torch.autograd.Function):
    """Rotary embedding over ``[..., N, heads*hd]`` rows (token-major); the backward is the inverse rotation."""

    @staticmethod
    def forward(ctx, x, heads, head_dim, rotary_dim, seq_len, pos_start, base):
        x2 = _as2d(x)
        out = torch.empty_like(x2)
        K.rope(x2, heads, head_dim, rotary_dim, seq_len, pos_start, base, out=out)
        ctx.cfg = (heads, head_dim, rotary_dim, seq_len, pos_start, base)
        return out.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        heads, head_dim, rotary_dim, seq_len, pos_start, base = ctx.cfg
        d2 = _as2d(dy)
        out = torch.empty_like(d2)
        K.rope(d2, heads, head_dim, rotary_dim, seq_len, pos_start, base, inverse=True, out=out)
        return out.view(dy.shape), None, None, None, None, None, None


class SwiGLUFn(torch.autograd.Function):
    """``silu(gu[:, :F]) * gu[:, F:]`` for a fused gate/up projection output ``[M, 2F]``."""

    @staticmethod
    def forward(ctx, gu):
        gu2 = _as2d(gu)
        F = gu2.shape[1] // 2
        out = K.swiglu_fwd(gu2[:, :F], gu2[:, F:])
        ctx.save_for_backward(gu2)
        ctx.shape = gu.shape
        return out.view(*gu.shape[:-1], F)

    @staticmethod
    def backward(ctx, dout):
        (gu2,) = ctx.saved_tensors
        F = gu2.shape[1] // 2
        d = torch.empty_like(gu2)
        K.swiglu_bwd(gu2[:, :F], gu2[:, F:], _as2d(dout), d[:, :F], d[:, F:])
        return d.view(ctx.shape)


class RopeColsFn(torch.autograd.Function):
    """In-place rotary embedding of the first ``heads`` head blocks of every row of a fused projection output
    (the Q and K columns of ``[rows, (H + 2 Hkv) hd]``); the V columns are untouched.  The backward applies the inverse
    rotation to the same columns of the incoming gradient, also in place (that gradient is produced by the attention
    backward and has no other consumer)."""

    @staticmethod
    def forward(ctx, qkv, heads, head_dim, rotary_dim, seq_len, pos_start, base):
        K.rope(qkv, heads, head_dim, rotary_dim, seq_len, pos_start, base)
        ctx.mark_dirty(qkv)
        ctx.cfg = (heads, head_dim, rotary_dim, seq_len, pos_start, base)
        return qkv

    @staticmethod
    def backward(ctx, dy):
        heads, head_dim, rotary_dim, seq_len, pos_start, base = ctx.cfg
        d = dy if dy.is_contiguous() else dy.contiguous()
        K.rope(d, heads, head_dim, rotary_dim, seq_len, pos_start, base, inverse=True)
        return d, None, None, None, None, None, None
