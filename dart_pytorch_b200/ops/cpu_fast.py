"""Fused restatements of the hot CPU ops.

``ops/reference.py`` spells every formula out op by op; it stays the oracle of the test-suite.  The functions here
compute the same formulas through single ATen calls (``F.linear``, ``F.layer_norm``, ``torch.softmax``,
``torch.native_dropout`` ...), which removes most of the per-op autograd bookkeeping that dominates small CPU models.
They are used for CPU tensors whose operands share one floating dtype and fall back to the reference otherwise;
``tests/test_ops_cpu.py`` checks values and gradients of both against each other.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

from . import reference as ref

_FAST_ACT = {
    None: None,
    "none": None,
    "relu": torch.relu,
    "gelu_tanh": lambda y: F.gelu(y, approximate="tanh"),
    "silu": F.silu,
    "sigmoid": torch.sigmoid,
    "tanh": torch.tanh,
}


def _same_float(*ts) -> bool:
    dt = None
    for t in ts:
        if t is None:
            continue
        if not t.is_floating_point() or (dt is not None and t.dtype != dt):
            return False
        dt = t.dtype
    return dt in (torch.float32, torch.float64)


def linear(x, weight, bias=None, activation=None, residual=None):
    if activation not in _FAST_ACT or not _same_float(x, weight, bias, residual):
        return ref.linear(x, weight, bias, activation, residual)
    y = F.linear(x, weight, None if bias is None else bias.reshape(-1))
    act = _FAST_ACT[activation]
    if act is not None:
        y = act(y)
    if residual is not None:
        y = y + residual
    return y


def gelu_tanh(x):
    return F.gelu(x, approximate="tanh") if _same_float(x) else ref.gelu_tanh(x)


def layer_norm(x, gamma, beta=None, eps: float = 1e-5):
    if not _same_float(x, gamma, beta) or gamma.numel() != x.shape[-1]:
        return ref.layer_norm(x, gamma, beta, eps)
    return F.layer_norm(x, (x.shape[-1],), gamma.reshape(-1), None if beta is None else beta.reshape(-1), eps)


def softmax(x):
    return torch.softmax(x, dim=-1) if _same_float(x) else ref.softmax(x)


_MASKS: Dict[Tuple[int, int, int, str, torch.dtype], torch.Tensor] = {}


def _causal_bias(sq: int, sk: int, q_offset: int, device, dtype) -> torch.Tensor:
    key = (sq, sk, q_offset, str(device), dtype)
    m = _MASKS.get(key)
    if m is None:
        if len(_MASKS) > 64:
            _MASKS.clear()
        i = torch.arange(sq, device=device).unsqueeze(1) + q_offset
        j = torch.arange(sk, device=device).unsqueeze(0)
        m = torch.where(j > i, -1e9, 0.0).to(dtype)
        _MASKS[key] = m
    return m


def attention(q, k, v, causal: bool = False, mask=None, q_offset: int = 0):
    """Same contract as ``reference.attention`` (grouped-query sharing, additive ``-1e9`` causal bias)."""
    if not _same_float(q, k, v) or (mask is not None and mask.dtype != q.dtype):
        return ref.attention(q, k, v, causal=causal, mask=mask, q_offset=q_offset)
    b, hq, sq, hd = q.shape
    hkv = k.shape[1]
    if hq % hkv:
        raise ValueError("attention: numHeads must be a multiple of numKvHeads")
    g = hq // hkv
    if g > 1:
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
    sk = k.shape[2]
    if mask is None:
        # One fused ATen call (forward and backward three times cheaper than the op chain below on a small model).
        # Its own causal mask is aligned to the top-left corner, which is this function's rule only for q_offset 0 and
        # equal lengths; a query block that sees every key needs no mask; other offsets pass the additive bias.
        if not causal or q_offset >= sk - 1:
            return F.scaled_dot_product_attention(q, k, v)
        if q_offset == 0 and sq == sk:
            return F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return F.scaled_dot_product_attention(q, k, v, attn_mask=_causal_bias(sq, sk, q_offset, q.device, q.dtype))
    s = torch.matmul(q, k.transpose(-1, -2)) * (1.0 / math.sqrt(hd))
    if causal:
        s = s + _causal_bias(sq, sk, q_offset, q.device, s.dtype)
    s = s + mask
    return torch.matmul(torch.softmax(s, dim=-1), v)


def dropout(x, p: float, training: bool, generator: Optional[torch.Generator] = None):
    if generator is not None or not _same_float(x):
        return ref.dropout(x, p, training, generator)
    if not (0.0 <= p < 1.0):
        raise ValueError("dropout: p must be in [0, 1)")
    if not training or p == 0.0:
        return x
    # Inverted dropout with the mask drawn 16 bits per element: one call fills n / 4 64-bit words from the default
    # generator (so ``torch.manual_seed`` governs it), viewed as int16 and compared with the threshold for ``p``
    # (resolution 2^-16).  Three times cheaper than ``torch.native_dropout`` on the tensors of a small CPU model,
    # whose cost is the generator's bernoulli path; autograd sees a plain multiply by the scaled mask.
    if p < 2e-3 or p > 1.0 - 2e-3:
        return torch.native_dropout(x, p, True)[0]      # beyond what 16 bits resolve: the generator's bernoulli path
    n = x.numel()
    words = torch.empty((n + 3) // 4, dtype=torch.int64, device=x.device).random_(-2 ** 63, None)
    keep = words.view(torch.int16)[:n].view(x.shape) >= (-32768 + int(round(p * 65536.0)))
    return x * keep.to(x.dtype).mul_(1.0 / (1.0 - p))


def embedding(table, indices):
    """Row gather; a batch with an out-of-range index takes the reference path (zero rows for those)."""
    idx = ref._round_index(indices)
    if idx.numel() == 0 or int(idx.min()) < 0 or int(idx.max()) >= table.shape[0]:
        return ref.embedding(table, indices)
    return F.embedding(idx, table)


def cross_entropy(logits, targets):
    """``[R, 1]`` per-row losses, as ``reference.cross_entropy``."""
    if logits.dtype != torch.float32:           # the reference works (and answers) in fp32 whatever comes in
        return ref.cross_entropy(logits, targets)
    v = logits.shape[-1]
    flat = logits.reshape(-1, v)
    tgt = ref._round_index(targets).reshape(-1)
    if tgt.numel() != flat.shape[0]:
        raise ValueError("cross_entropy: number of targets must equal number of rows")
    if tgt.numel() and (int(tgt.min()) < 0 or int(tgt.max()) >= v):
        return ref.cross_entropy(logits, targets)
    return F.cross_entropy(flat, tgt, reduction="none").unsqueeze(1)
