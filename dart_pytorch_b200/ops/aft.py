"""AFT-full on the GPU as two tensor-core GEMMs (reference kernel: lib/native/src/kernels/attention.cuh:17-49, one
thread per output element looping over every position; autograd: lib/core/tensor/aft.dart:34-228).

``exp(k[t', d] + w[t, t'])`` factors into ``exp(w[t, t']) * exp(k[t', d])``, so

    num = EW @ (EK * v),   den = EW @ EK,   out = sigmoid(q) * num / den

with ``EW = exp(w - rowmax(w)) * causal_mask`` (``[T, T]``) and ``EK = exp(k - colmax(k))`` (``[T, D]``): the row / column
shifts cancel between numerator and denominator and keep every exponential <= 1.  Both products are one GEMM against
the concatenated ``[EK * v | EK]`` operand.  Everything is composed from the framework's differentiable kernel ops, so
the backward pass is the corresponding GEMMs and elementwise kernels.  (The reference adds 1e-6 to its denominator,
whose terms sum to at least 1 there; the shifted denominator here can be smaller, so the guard is 1e-30.)
"""
from __future__ import annotations

import torch


def aft_full_cuda(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, causal: bool = True):
    from . import add, div, exp, matmul, mul, sigmoid, sub
    t, d = q.shape
    wt = w[:t, :t]
    if causal:
        allowed = torch.tril(torch.ones(t, t, dtype=torch.bool, device=q.device))
        row_max = torch.where(allowed, wt.detach(), torch.full_like(wt, float("-inf"))).max(dim=1, keepdim=True).values
    else:
        allowed = None
        row_max = wt.detach().max(dim=1, keepdim=True).values
    col_max = k.detach().max(dim=0, keepdim=True).values
    ew = exp(sub(wt.contiguous(), row_max.expand(t, t).contiguous()))
    if allowed is not None:
        ew = mul(ew, allowed.to(ew.dtype))
    ek = exp(sub(k, col_max.expand(t, d).contiguous()))
    both = matmul(ew, torch.cat([mul(ek, v), ek], dim=1))        # [T, 2D] = [num | den]
    num, den = both[:, :d], both[:, d:]
    return mul(sigmoid(q), div(num.contiguous(), add(den.contiguous(), 1e-30)))
