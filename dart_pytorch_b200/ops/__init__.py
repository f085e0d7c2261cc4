"""Functional tensor ops.  CPU tensors take the pure-PyTorch reference formulas (``ops/reference.py``, the hot ones
through their single-call restatements in ``ops/cpu_fast.py``); CUDA tensors
take the native sm_100a kernels through the autograd functions of ``ops/cuda.py``.  There is one code path per
device: a CUDA tensor never falls back to a library kernel, and a missing native library raises.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from . import cpu_fast as fast
from . import reference as ref
from .reference import causal_mask, sample_from_logits  # noqa: F401  (re-exported)


def _cuda(*ts) -> bool:
    return any(t is not None and isinstance(t, torch.Tensor) and t.is_cuda for t in ts)


def _cu():
    from . import cuda
    return cuda


def _match(x: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    return x if x.dtype == like.dtype else x.to(like.dtype)


def _decode_half(w, like: torch.Tensor):
    """CPU half-precision *storage* operands (weights kept as fp16 to halve memory) are widened where they are used
    (reference: fp16 right-hand sides are decoded on the fly, lib/core/tensor/mat_mul.dart:51-76)."""
    if w is not None and w.dtype == torch.float16 and like.dtype != torch.float16 and not w.is_cuda:
        return w.to(like.dtype)
    return w


# --------------------------------------------------------------------------- matmul / linear
def matmul(a, b):
    if b.dim() != 2:
        raise ValueError("matmul: right operand must be 2-D [K, N]")
    if a.shape[-1] != b.shape[0]:
        raise ValueError(f"matmul: inner dims differ: {tuple(a.shape)} @ {tuple(b.shape)}")
    if a.device != b.device:
        raise ValueError("matmul: operands live on different devices")
    if _cuda(a, b):
        return _cu().MatmulFn.apply(a, _match(b, a))
    return ref.matmul(a, _decode_half(b, a))


def linear(x, weight, bias=None, activation=None, residual=None):
    if activation in ("none",):
        activation = None
    if _cuda(x):
        x = _match(x, weight)
        if residual is not None:
            residual = _match(residual, weight)
        return _cu().LinearFn.apply(x, weight, bias, activation, residual)
    return fast.linear(x, _decode_half(weight, x), _decode_half(bias, x), activation, residual)


def mlp(x, w1, b1, w2, b2, activation="relu", residual=None):
    """Two-layer feed-forward ``act(x w1^T + b1) w2^T + b2 (+ residual)``."""
    if _cuda(x) and w1.dtype == torch.bfloat16 and activation not in (None, "none"):
        x = _match(x, w1)
        if residual is not None:
            residual = _match(residual, w1)
        return _cu().MLPFn.apply(x, w1, b1, w2, b2, activation, residual)
    h = linear(x, w1, b1, activation)
    return linear(h, w2, b2, None, residual)


# --------------------------------------------------------------------------- norms
def layer_norm(x, gamma, beta=None, eps: float = 1e-5):
    if _cuda(x):
        return _cu().LayerNormFn.apply(_match(x, gamma), gamma, beta, eps, False)
    return fast.layer_norm(x, gamma, beta, eps)


def rms_norm(x, gamma, eps: float = 1e-6):
    if _cuda(x):
        return _cu().RMSNormFn.apply(_match(x, gamma), gamma, eps, False)
    return ref.rms_norm(x, gamma, eps)


def layer_norm_residual(x, gamma, beta=None, eps: float = 1e-5):
    """``(x, layer_norm(x))`` where the first output carries the residual stream: in the backward the gradient of the
    residual branch is added inside the norm's kernel instead of by a separate add."""
    if _cuda(x):
        return _cu().LayerNormFn.apply(_match(x, gamma), gamma, beta, eps, True)
    return x, fast.layer_norm(x, gamma, beta, eps)


def rms_norm_residual(x, gamma, eps: float = 1e-6):
    if _cuda(x):
        return _cu().RMSNormFn.apply(_match(x, gamma), gamma, eps, True)
    return x, ref.rms_norm(x, gamma, eps)


# --------------------------------------------------------------------------- softmax / losses
def softmax(x):
    if _cuda(x):
        return _cu().SoftmaxFn.apply(x)
    return fast.softmax(x)


def cross_entropy(logits, targets):
    """Per-row loss ``[R, 1]``; call ``.mean()`` on it for the scalar (the reference's contract)."""
    if _cuda(logits):
        rows = logits.numel() // logits.shape[-1]
        if targets.numel() != rows:
            raise ValueError("cross_entropy: number of targets must equal number of rows")
        return _cu().CrossEntropyFn.apply(logits, ref._round_index(targets))
    return fast.cross_entropy(logits, targets)


def lm_head_loss(h, weight, targets):
    """Scalar mean cross-entropy of ``h @ weight.T`` (the tied or untied LM head) against ``targets``."""
    if _cuda(h):
        return _cu().LMHeadLossFn.apply(_match(h, weight), weight, ref._round_index(targets))
    logits = h @ weight.t()
    return fast.cross_entropy(logits, targets).mean()


# --------------------------------------------------------------------------- embedding
def embedding(table, indices, pos_table=None, pos_start: int = 0):
    """Row gather (out-of-range -> zero row).  With ``pos_table`` the learned position rows
    ``pos_start + arange(indices.shape[-1])`` are added in the same kernel."""
    if _cuda(table):
        return _cu().EmbeddingFn.apply(table, indices, pos_table, pos_start)
    out = fast.embedding(table, indices)
    if pos_table is not None:
        n = indices.shape[-1]
        out = out + pos_table[pos_start:pos_start + n]
    return out


def scatter_rows_add(rows, indices, total_rows: int):
    if _cuda(rows):
        return _cu().ScatterRowsAddFn.apply(rows.reshape(-1, rows.shape[-1]), indices.reshape(-1), total_rows)
    return ref.scatter_rows_add(rows, indices, total_rows)


# --------------------------------------------------------------------------- attention
def attention(q, k, v, causal: bool = False, mask=None, q_offset: int = 0):
    """``[B, Hq, Sq, hd]`` x ``[B, Hkv, Sk, hd]`` grouped-query attention."""
    if _cuda(q):
        from . import flash as attn
        return attn.attention_bhsd(q, k, v, causal=causal, mask=mask, q_offset=q_offset)
    return fast.attention(q, k, v, causal=causal, mask=mask, q_offset=q_offset)


def attention_packed(qkv, batch: int, seq: int, heads: int, kv_heads: int, head_dim: int, causal: bool = True):
    """Attention straight from a fused projection output ``[B*S, (H + 2*Hkv) * hd]`` (columns: all Q heads, all K
    heads, all V heads) to ``[B*S, H*hd]`` with heads concatenated, ready for the output projection."""
    if _cuda(qkv):
        from . import flash as attn
        return attn.attention_packed(qkv, batch, seq, heads, kv_heads, head_dim, causal)
    d_q, d_kv = heads * head_dim, kv_heads * head_dim
    x = qkv.reshape(batch, seq, d_q + 2 * d_kv)
    q = x[..., :d_q].reshape(batch, seq, heads, head_dim).transpose(1, 2)
    k = x[..., d_q:d_q + d_kv].reshape(batch, seq, kv_heads, head_dim).transpose(1, 2)
    v = x[..., d_q + d_kv:].reshape(batch, seq, kv_heads, head_dim).transpose(1, 2)
    o = fast.attention(q, k, v, causal=causal)
    return o.transpose(1, 2).reshape(batch * seq, d_q)


def sdpa(q, k, v, mask=None):
    """The reference's single-head 2-D attention (lib/core/tensor/attention.dart:17-55)."""
    if _cuda(q):
        o = attention(q[None, None], k[None, None], v[None, None], causal=False, mask=mask)
        return o[0, 0]
    return ref.sdpa(q, k, v, mask)


# --------------------------------------------------------------------------- rope / dropout / swiglu
def rope(x, start_pos: int = 0, base: float = 10000.0, rotary_dim: Optional[int] = None, heads: int = 1):
    """Half-split rotary embedding.  ``x`` is ``[..., N, heads*hd]`` (token-major rows, heads side by side)."""
    if _cuda(x):
        hd = x.shape[-1] // heads
        rd = hd if rotary_dim is None else rotary_dim
        return _cu().RopeFn.apply(x, heads, hd, rd, x.shape[-2], start_pos, base)
    if heads == 1:
        return ref.rope(x, start_pos, base, rotary_dim)
    hd = x.shape[-1] // heads
    xs = x.reshape(*x.shape[:-1], heads, hd).transpose(-2, -3)  # [..., heads, N, hd]
    out = ref.rope(xs, start_pos, base, rotary_dim)
    return out.transpose(-2, -3).reshape(x.shape)


def dropout(x, p: float, training: bool, generator=None):
    if not (0.0 <= p < 1.0):
        raise ValueError("dropout: p must be in [0, 1)")
    if not training or p == 0.0:
        return x
    if _cuda(x):
        return _cu().DropoutFn.apply(x, p)
    return fast.dropout(x, p, training, generator)


def swiglu(gate_up):
    """``silu(gate) * up`` for ``gate_up = [gate | up]`` along the last axis."""
    if _cuda(gate_up):
        return _cu().SwiGLUFn.apply(gate_up)
    f = gate_up.shape[-1] // 2
    return ref.silu(gate_up[..., :f]) * gate_up[..., f:]


# --------------------------------------------------------------------------- elementwise / reductions
def _unary(x, op, param=0.0, cpu=None):
    if _cuda(x):
        return _cu().UnaryFn.apply(x, op, float(param))
    return cpu(x)


def relu(x):
    return _unary(x, "relu", cpu=ref.relu)


def sigmoid(x):
    return _unary(x, "sigmoid", cpu=ref.sigmoid)


def tanh(x):
    return _unary(x, "tanh", cpu=ref.tanh)


def abs(x):  # noqa: A001
    return _unary(x, "abs", cpu=torch.abs)


def log(x):
    """Natural log.  On the device ``1e-7`` is added first, as the reference's kernel does; on the CPU it is not."""
    return _unary(x, "log", 1e-7, cpu=ref.log_eps)


def pow(x, e: float):  # noqa: A001
    return _unary(x, "pow", e, cpu=lambda t: ref.safe_pow(t, e))


def exp(x):
    return _unary(x, "exp", cpu=torch.exp)


def sqrt(x):
    return _unary(x, "sqrt", cpu=torch.sqrt)


def gelu_tanh(x):
    return _unary(x, "gelu_tanh", cpu=fast.gelu_tanh)


def quick_gelu(x):
    return _unary(x, "quick_gelu", cpu=ref.quick_gelu)


def silu(x):
    return _unary(x, "silu", cpu=ref.silu)


ACTIVATION_FNS = {None: lambda x: x, "none": lambda x: x, "relu": relu, "gelu_tanh": gelu_tanh,
                  "quick_gelu": quick_gelu, "silu": silu, "sigmoid": sigmoid, "tanh": tanh}


def _binary(a, b, op, cpu):
    if isinstance(b, (int, float)):
        if _cuda(a):
            if op == "add":
                return _cu().UnaryFn.apply(a, "add_scalar", float(b))
            if op == "sub":
                return _cu().UnaryFn.apply(a, "add_scalar", -float(b))
            if op == "mul":
                return _cu().UnaryFn.apply(a, "scale", float(b))
            b = torch.full((1,), float(b), dtype=a.dtype, device=a.device)
        else:
            return cpu(a, torch.tensor(float(b), dtype=a.dtype))
    if isinstance(a, (int, float)):
        a = torch.full((1,), float(a), dtype=b.dtype, device=b.device)
    if a.device != b.device:
        raise ValueError(f"{op}: operands live on different devices")
    if _cuda(a, b):
        return _cu().BinaryFn.apply(a, _match(b, a), op)
    return cpu(a, b)


def _bcast_ok(a, b):
    if a.shape == b.shape or a.numel() == 1 or b.numel() == 1:
        return
    if a.numel() == b.numel():
        return
    if a.dim() >= 2 and b.numel() == a.shape[-1]:
        return
    raise ValueError(f"shapes {tuple(a.shape)} and {tuple(b.shape)} do not broadcast")


def _cpu_bin(fn):
    def run(a, b):
        _bcast_ok(a, b)
        if a.dim() >= 2 and b.dim() >= 1 and b.numel() == a.shape[-1] and b.shape != a.shape:
            b = b.reshape(-1)
        elif a.numel() == b.numel() and a.shape != b.shape:
            b = b.reshape(a.shape)
        return fn(a, b)
    return run


def add(a, b):
    return _binary(a, b, "add", _cpu_bin(torch.add))


def sub(a, b):
    return _binary(a, b, "sub", _cpu_bin(torch.sub))


def mul(a, b):
    return _binary(a, b, "mul", _cpu_bin(torch.mul))


def div(a, b):
    """Division; on the device the denominator magnitude is floored at 1e-20 (the reference kernel's rule)."""
    return _binary(a, b, "div", _cpu_bin(torch.div))


def sum(x):  # noqa: A001
    """Sum of all elements as ``[1, 1]`` (reference: lib/core/tensor/ops.dart:524-547)."""
    if _cuda(x):
        return _cu().SumFn.apply(x, False)
    return x.sum().reshape(1, 1)


def mean(x):
    if _cuda(x):
        return _cu().SumFn.apply(x, True)
    return x.mean().reshape(1, 1)


def transpose(x):
    if x.dim() != 2:
        raise ValueError("transpose: 2-D tensors only")
    if _cuda(x):
        return _cu().TransposeFn.apply(x)
    return x.t().contiguous()


def concat(tensors: Sequence[torch.Tensor], axis: int = 0):
    return ref.concat(tensors, axis)


def split_rows(t, chunk: int):
    return ref.split_rows(t, chunk)


def slice_top_left(t, rows: int, cols: int):
    return ref.slice_top_left(t, rows, cols)


def aft_full(q, k, v, w, causal: bool = True):
    if _cuda(q):
        from . import aft
        return aft.aft_full_cuda(q, k, v, w, causal)
    return ref.aft_full(q, k, v, w, causal)


def im2col_nhwc(x, batch: int, channels: int, ksize: int, board: int = 8):
    if _cuda(x):
        from . import kernels as K
        return K.im2col_nhwc(x, batch, channels, ksize, board)
    return ref.im2col_nhwc(x, batch, channels, ksize, board)
