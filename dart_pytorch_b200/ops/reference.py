"""Pure-PyTorch fp32 restatement of every tensor op: the CPU path and the numerical oracle.

Each function states the formula that the reference library's CPU loops compute
(reference: lib/core/tensor/*.dart).  They run on any device, are differentiable through
torch autograd, and are what every CUDA kernel in ``csrc/`` is tested against.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

SQRT_2_OVER_PI = 0.7978845608028654


# --------------------------------------------------------------------------- elementwise
def safe_div(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a / b`` with ``|b|`` floored at 1e-20, sign preserved (reference GPU path:
    lib/native/src/kernels/elementwise.cuh:211-224)."""
    mag = b.abs().clamp_min(1e-20)
    sign = torch.where(b < 0, -torch.ones_like(b), torch.ones_like(b))
    return a / (mag * sign)


def safe_pow(x: torch.Tensor, e: float) -> torch.Tensor:
    """NaN-free power: integer exponents by exact repeated multiplication semantics (negatives
    allowed, ``0**neg -> 0``); fractional exponents give ``x**e`` for ``x > 0`` else 0
    (reference: lib/native/src/kernels/elementwise.cuh:255-298)."""
    if abs(e - round(e)) < 1e-6:
        n = int(round(e))
        if n >= 0:
            return x.pow(n)
        inv = x.pow(-n)
        return torch.where(inv == 0, torch.zeros_like(x), 1.0 / torch.where(inv == 0, torch.ones_like(inv), inv))
    pos = x > 0
    return torch.where(pos, torch.where(pos, x, torch.ones_like(x)).pow(e), torch.zeros_like(x))


def log_eps(x: torch.Tensor, eps: float = 0.0) -> torch.Tensor:
    """Natural log; the reference's GPU kernel adds 1e-7 before the log, its CPU loop does not
    (lib/native/src/kernels/elementwise.cuh:390-398 vs lib/core/tensor/ops.dart:376)."""
    return torch.log(x + eps) if eps else torch.log(x)


def relu(x):
    return torch.relu(x)


def sigmoid(x):
    return torch.sigmoid(x)


def tanh(x):
    return torch.tanh(x)


def silu(x):
    return x * torch.sigmoid(x)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """``0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))`` (reference: lib/core/nn/transformer.dart:97-102)."""
    inner = (x + 0.044715 * x * x * x) * SQRT_2_OVER_PI
    return 0.5 * x * (1.0 + torch.tanh(inner))


def quick_gelu(x: torch.Tensor) -> torch.Tensor:
    """``x * sigmoid(1.702 x)`` (reference: lib/core/nn/transformer.dart:104-109)."""
    return x * torch.sigmoid(1.702 * x)


ACTIVATIONS = {
    None: lambda x: x,
    "none": lambda x: x,
    "relu": relu,
    "gelu_tanh": gelu_tanh,
    "quick_gelu": quick_gelu,
    "silu": silu,
    "sigmoid": sigmoid,
    "tanh": tanh,
}


# --------------------------------------------------------------------------- matmul / linear
def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """2-D x 2-D, or ``[..., K] @ [K, N]`` by flattening the leading axes
    (reference: lib/core/tensor/mat_mul.dart:12-93)."""
    if b.dim() != 2:
        raise ValueError("matmul: right operand must be 2-D [K, N]")
    if a.shape[-1] != b.shape[0]:
        raise ValueError(f"matmul: inner dims differ: {tuple(a.shape)} @ {tuple(b.shape)}")
    return a @ b


def linear(x, weight, bias=None, activation=None, residual=None):
    """``act(x @ weight.T + bias) + residual`` with weight ``[out, in]`` (reference: lib/core/nn/linear.dart:67-96)."""
    y = x @ weight.t()
    if bias is not None:
        y = y + bias.reshape(-1)
    y = ACTIVATIONS[activation](y)
    if residual is not None:
        y = y + residual
    return y


# --------------------------------------------------------------------------- norms
def layer_norm(x, gamma, beta, eps: float = 1e-5):
    """Row-wise centred two-pass mean/variance, ``(x-mean) * rsqrt(var+eps) * gamma + beta``
    (reference: lib/core/tensor/layer_norm.dart:15-200)."""
    mean = x.mean(dim=-1, keepdim=True)
    xc = x - mean
    var = (xc * xc).mean(dim=-1, keepdim=True)
    y = xc * torch.rsqrt(var + eps) * gamma
    return y + beta if beta is not None else y


def rms_norm(x, gamma, eps: float = 1e-6):
    """``x * rsqrt(mean(x^2) + eps) * gamma`` (reference: lib/core/tensor/rms_norm.dart:18-148)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * gamma


# --------------------------------------------------------------------------- softmax / CE
def softmax(x):
    """Last-axis softmax with max subtraction (reference: lib/core/tensor/softmax.dart:10-98)."""
    m = x.max(dim=-1, keepdim=True).values
    e = torch.exp(x - m)
    return e / e.sum(dim=-1, keepdim=True)


def _round_index(t: torch.Tensor) -> torch.Tensor:
    """Indices may arrive as floats (the reference has no integer tensors): ``floor(t + 0.5)``."""
    if t.is_floating_point():
        return torch.floor(t + 0.5).to(torch.long)
    return t.to(torch.long)


def cross_entropy(logits, targets):
    """Per-row ``logsumexp(x) - x[target]`` returned as ``[R, 1]``; accepts ``[B,S,V]`` + ``[B,S]`` by
    flattening; only logits receive a gradient (reference: lib/core/tensor/softmax.dart:100-212)."""
    v = logits.shape[-1]
    flat = logits.reshape(-1, v)
    tgt = _round_index(targets).reshape(-1)
    if tgt.numel() != flat.shape[0]:
        raise ValueError("cross_entropy: number of targets must equal number of rows")
    lse = torch.logsumexp(flat.float(), dim=-1)
    picked = flat.float().gather(1, tgt.unsqueeze(1)).squeeze(1)
    return (lse - picked).unsqueeze(1)


# --------------------------------------------------------------------------- embedding / scatter
def embedding(table, indices):
    """Row gather; out-of-range indices give a zero row (reference: lib/core/tensor/embedding.dart:16-115,
    lib/native/src/kernels/embedding.cuh:19-34)."""
    idx = _round_index(indices)
    v = table.shape[0]
    ok = (idx >= 0) & (idx < v)
    safe = torch.where(ok, idx, torch.zeros_like(idx))
    out = table[safe.reshape(-1)].reshape(*idx.shape, table.shape[1])
    return out * ok.unsqueeze(-1).to(out.dtype)


def scatter_rows_add(rows, indices, total_rows: int):
    """Adjoint of ``embedding``: ``out[idx[n], :] += rows[n, :]`` into zeros ``[total_rows, D]``; out-of-range
    indices are skipped (reference: lib/core/tensor/scatter.dart:20-85)."""
    idx = _round_index(indices).reshape(-1)
    d = rows.shape[-1]
    flat = rows.reshape(-1, d)
    ok = (idx >= 0) & (idx < total_rows)
    safe = torch.where(ok, idx, torch.zeros_like(idx))
    out = torch.zeros(total_rows, d, dtype=rows.dtype, device=rows.device)
    return out.index_add(0, safe, flat * ok.unsqueeze(-1).to(flat.dtype))


# --------------------------------------------------------------------------- attention
def sdpa(q, k, v, mask=None):
    """Single-head 2-D attention ``softmax(q k^T / sqrt(dk) + mask) v``
    (reference: lib/core/tensor/attention.dart:17-55)."""
    scale = 1.0 / math.sqrt(q.shape[-1])
    s = (q @ k.transpose(-1, -2)) * scale
    if mask is not None:
        s = s + mask
    return softmax(s) @ v


def attention(q, k, v, causal: bool = False, mask=None, q_offset: int = 0):
    """Batched multi-head attention with grouped-query sharing.

    ``q``: ``[B, Hq, Sq, hd]``, ``k``/``v``: ``[B, Hkv, Sk, hd]`` with ``Hq % Hkv == 0``; query head ``h`` reads
    KV head ``h // (Hq/Hkv)`` (reference: lib/core/nn/attention/multi_head_attention.dart:181-189).  ``causal``
    forbids key ``j`` for query ``i`` when ``j > i + q_offset`` using the reference's additive ``-1e9``.
    """
    b, hq, sq, hd = q.shape
    hkv = k.shape[1]
    if hq % hkv:
        raise ValueError("attention: numHeads must be a multiple of numKvHeads")
    g = hq // hkv
    if g > 1:
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
    s = (q.float() @ k.float().transpose(-1, -2)) * (1.0 / math.sqrt(hd))
    if causal:
        sk = k.shape[2]
        i = torch.arange(sq, device=q.device).unsqueeze(1) + q_offset
        j = torch.arange(sk, device=q.device).unsqueeze(0)
        s = s + torch.where(j > i, -1e9, 0.0).to(s.dtype)
    if mask is not None:
        s = s + mask
    return (softmax(s) @ v.float()).to(q.dtype)


def causal_mask(n: int, block_value: float = -1e9, device=None, dtype=torch.float32):
    """Additive ``[n, n]`` mask, ``j > i -> block_value`` (reference: lib/core/nn/masks.dart:16-28)."""
    i = torch.arange(n, device=device).unsqueeze(1)
    j = torch.arange(n, device=device).unsqueeze(0)
    return torch.where(j > i, block_value, 0.0).to(dtype)


# --------------------------------------------------------------------------- RoPE
def rope_tables(positions: torch.Tensor, head_dim: int, rotary_dim: Optional[int], base: float):
    """cos/sin ``[N, head_dim]`` for half-split rotation; dims past ``rotary_dim`` get cos=1, sin=0
    (reference: lib/core/nn/rotary.dart:95-131)."""
    rd = head_dim if rotary_dim is None else rotary_dim
    half = rd // 2
    i = torch.arange(half, device=positions.device, dtype=torch.float64)
    inv = base ** (-2.0 * i / rd)
    ang = positions.to(torch.float64).unsqueeze(1) * inv.unsqueeze(0)  # [N, half]
    cos = torch.ones(positions.numel(), head_dim, dtype=torch.float64, device=positions.device)
    sin = torch.zeros_like(cos)
    cos[:, :half] = torch.cos(ang)
    cos[:, half:rd] = torch.cos(ang)
    sin[:, :half] = torch.sin(ang)
    sin[:, half:rd] = torch.sin(ang)
    return cos.float(), sin.float()


def rope(x, start_pos: int = 0, base: float = 10000.0, rotary_dim: Optional[int] = None, positions=None):
    """Half-split (NeoX/Llama) rotary embedding on the last axis; the second-to-last axis is the position axis.
    ``out = x*cos + rotate_half(x)*sin`` with ``rotate_half([a, b]) = [-b, a]`` on the first ``rotary_dim`` dims
    (reference: lib/core/nn/rotary.dart:133-201)."""
    n, hd = x.shape[-2], x.shape[-1]
    rd = hd if rotary_dim is None else rotary_dim
    if positions is None:
        positions = torch.arange(start_pos, start_pos + n, device=x.device)
    cos, sin = rope_tables(positions, hd, rd, base)
    half = rd // 2
    rot = torch.zeros_like(x, dtype=torch.float32)
    xf = x.float()
    rot[..., :half] = -xf[..., half:rd]
    rot[..., half:rd] = xf[..., :half]
    return (xf * cos + rot * sin).to(x.dtype)


# --------------------------------------------------------------------------- dropout / concat / slicing
def dropout(x, p: float, training: bool, generator: Optional[torch.Generator] = None):
    """Inverted dropout with a ``{0, 1/(1-p)}`` mask (reference: lib/core/tensor/dropout.dart:13-31)."""
    if not (0.0 <= p < 1.0):
        raise ValueError("dropout: p must be in [0, 1)")
    if not training or p == 0.0:
        return x
    keep = torch.rand(x.shape, device=x.device, generator=generator) >= p
    return x * (keep.to(x.dtype) / (1.0 - p))


def concat(tensors: Sequence[torch.Tensor], axis: int = 0):
    """2-D concat along axis 0 or 1 (reference: lib/core/tensor/concat.dart:14-142)."""
    if axis not in (0, 1):
        raise ValueError("concat: axis must be 0 or 1")
    if not tensors:
        raise ValueError("concat: empty list")
    return torch.cat(list(tensors), dim=axis)


def split_rows(t: torch.Tensor, chunk: int):
    """Equal row chunks (reference: lib/core/tensor/concat.dart:151-203)."""
    if chunk <= 0 or t.shape[0] % chunk:
        raise ValueError("split_rows: rows must divide evenly by chunk")
    return list(torch.split(t, chunk, dim=0))


def slice_top_left(t: torch.Tensor, rows: int, cols: int):
    """Top-left sub-matrix; the backward zero-pads (reference: lib/core/tensor/aft.dart:230-294)."""
    if rows > t.shape[0] or cols > t.shape[1]:
        raise ValueError("slice_top_left: slice exceeds source")
    return t[:rows, :cols]


# --------------------------------------------------------------------------- AFT-full
def aft_full(q, k, v, w, causal: bool = True):
    """Attention-free transformer (full): ``out[t,d] = sigmoid(q[t,d]) * sum_t' softmax_t'(k[t',d] + w[t,t']) v[t',d]``
    with ``1e-6`` added to the denominator and an optional causal limit ``t' <= t``
    (reference: lib/native/src/kernels/attention.cuh:17-49, lib/core/tensor/aft.dart:34-228)."""
    t, d = q.shape
    logits = k.unsqueeze(0) + w[:t, :t].unsqueeze(-1)  # [t, t', d]
    if causal:
        i = torch.arange(t, device=q.device).unsqueeze(1)
        j = torch.arange(t, device=q.device).unsqueeze(0)
        allowed = (j <= i).unsqueeze(-1)
        logits = torch.where(allowed, logits, torch.full_like(logits, float("-inf")))
    m = logits.max(dim=1, keepdim=True).values
    e = torch.exp(logits - m)
    num = (e * v.unsqueeze(0)).sum(dim=1)
    den = e.sum(dim=1) + 1e-6
    return torch.sigmoid(q) * num / den


# --------------------------------------------------------------------------- im2col (8x8 board, NHWC-flat)
def im2col_nhwc(x, batch: int, channels: int, ksize: int, board: int = 8):
    """Unfold ``[B*board*board, C]`` into ``[B*board*board, C*k*k]`` with zero padding ``k//2``; column order is
    ``(c, ky, kx)`` (reference: lib/native/src/kernels/im2col.cuh:17-50)."""
    pad = ksize // 2
    img = x.reshape(batch, board, board, channels)
    padded = torch.nn.functional.pad(img, (0, 0, pad, pad, pad, pad))
    cols = []
    for ky in range(ksize):
        for kx in range(ksize):
            cols.append(padded[:, ky:ky + board, kx:kx + board, :])  # [B, 8, 8, C]
    stacked = torch.stack(cols, dim=-1)  # [B, 8, 8, C, k*k]
    return stacked.reshape(batch * board * board, channels * ksize * ksize)


# --------------------------------------------------------------------------- sampling
def sample_from_logits(row: torch.Tensor, temperature: float, top_k: Optional[int], rng) -> int:
    """Greedy when ``temperature <= 0`` or ``top_k <= 1``; otherwise temperature scale, keep the top-k, softmax,
    and draw by walking the CDF with one uniform from ``rng.random()`` (reference: lib/core/nn/gpt.dart:288-342)."""
    v = row.numel()
    if temperature <= 0.0 or (top_k is not None and top_k <= 1):
        return int(torch.argmax(row).item())
    scaled = row.double() / temperature
    if top_k is not None and top_k < v:
        kth = torch.topk(scaled, top_k).indices
        keep = torch.zeros(v, dtype=torch.bool, device=row.device)
        keep[kth] = True
        scaled = torch.where(keep, scaled, torch.full_like(scaled, float("-inf")))
    e = torch.exp(scaled - scaled.max())
    total = float(e.sum().item())
    u = rng.random() * total
    cdf = torch.cumsum(e, 0)
    idx = int(torch.searchsorted(cdf, torch.tensor(u, dtype=cdf.dtype, device=cdf.device)).item())
    return min(idx, v - 1)
