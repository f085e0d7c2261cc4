"""Core layers: Linear, LayerNorm, RMSNorm, Embedding, Dropout, positional encodings, SwiGLU, projector.

Constructor signatures and parameter order follow the reference modules (cited per class); the forward passes call the
fused functional ops, so on a CUDA device each layer is one kernel (bias / activation / residual live in the GEMM
epilogue).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import ops as F
from .module import Module, make_param, normal_, uniform_

_ACT_NAMES = {"relu": "relu", "geluTanh": "gelu_tanh", "gelu_tanh": "gelu_tanh", "quickGelu": "quick_gelu",
              "quick_gelu": "quick_gelu", "silu": "silu", None: None, "none": None}


def activation_name(a) -> Optional[str]:
    name = getattr(a, "value", a)
    if name not in _ACT_NAMES:
        raise ValueError(f"unknown activation {a!r}")
    return _ACT_NAMES[name]


class Linear(Module):
    """``y = x W^T + b`` with ``W [out, in]`` ~ U(+-1/sqrt(in)); bias stored ``[out]`` and exported ``[1, out]``
    (reference: lib/core/nn/linear.dart:17-100)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, seed: int = 0,
                 dtype=torch.float32, init_std: Optional[float] = None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        bound = 1.0 / math.sqrt(in_features)
        if init_std is None:
            w = uniform_((out_features, in_features), bound, seed, device, dtype)
        else:
            w = normal_((out_features, in_features), init_std, seed, device, dtype)
        self.weight = make_param(w)
        self.bias = None
        if bias:
            b = uniform_((out_features,), bound, seed + 1, device, dtype) if init_std is None else \
                torch.zeros(out_features, device=device, dtype=dtype)
            self.bias = make_param(b)

    def own_parameters(self):
        return [self.weight] + ([self.bias] if self.bias is not None else [])

    def own_reference_parameters(self):
        out = [self.weight.data]
        if self.bias is not None:
            out.append(self.bias.data.view(1, -1))
        return out

    def forward(self, x, activation=None, residual=None):
        if x.dim() < 2:
            raise ValueError("Linear: input must have rank >= 2")
        if x.shape[-1] != self.in_features:
            raise ValueError(f"Linear: expected last dim {self.in_features}, got {x.shape[-1]}")
        return F.linear(x, self.weight, self.bias, activation_name(activation), residual)


class LayerNorm(Module):
    """(reference: lib/core/nn/layer_norm.dart:7-21)"""

    def __init__(self, dim: int, eps: float = 1e-5, device=None, dtype=torch.float32):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.gamma = make_param(torch.ones(dim, device=device, dtype=dtype))
        self.beta = make_param(torch.zeros(dim, device=device, dtype=dtype))

    def own_parameters(self):
        return [self.gamma, self.beta]

    def forward(self, x):
        if x.shape[-1] != self.dim:
            raise ValueError(f"LayerNorm: expected last dim {self.dim}, got {x.shape[-1]}")
        return F.layer_norm(x, self.gamma, self.beta, self.eps)

    def with_residual(self, x):
        """``(x, norm(x))``: see ``ops.layer_norm_residual``."""
        return F.layer_norm_residual(x, self.gamma, self.beta, self.eps)


class RMSNorm(Module):
    """(reference: lib/core/nn/rms_norm.dart:10-22)"""

    def __init__(self, dim: int, eps: float = 1e-6, device=None, dtype=torch.float32):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.gamma = make_param(torch.ones(dim, device=device, dtype=dtype))

    def own_parameters(self):
        return [self.gamma]

    def forward(self, x):
        if x.shape[-1] != self.dim:
            raise ValueError(f"RMSNorm: expected last dim {self.dim}, got {x.shape[-1]}")
        return F.rms_norm(x, self.gamma, self.eps)

    def with_residual(self, x):
        return F.rms_norm_residual(x, self.gamma, self.eps)


class Embedding(Module):
    """Table ``[V, D]`` ~ N(0, 1/D) (reference: lib/core/nn/embedding.dart:9-43)."""

    def __init__(self, num_embeddings: int, dim: int, device=None, seed: int = 0, dtype=torch.float32,
                 init_std: Optional[float] = None):
        super().__init__()
        self.num_embeddings, self.dim = num_embeddings, dim
        std = (1.0 / math.sqrt(dim)) if init_std is None else init_std
        self.weight = make_param(normal_((num_embeddings, dim), std, seed, device, dtype))

    def own_parameters(self):
        return [self.weight]

    def forward(self, indices):
        return F.embedding(self.weight, indices)


class Dropout(Module):
    """Inverted dropout active only in training mode (reference: lib/core/nn/dropout.dart:12-30)."""

    def __init__(self, p: float = 0.0, rng: Optional[torch.Generator] = None):
        super().__init__()
        if not (0.0 <= p < 1.0):
            raise ValueError("Dropout: p must be in [0, 1)")
        self.p, self.rng = p, rng

    def forward(self, x):
        return F.dropout(x, self.p, self.training, self.rng)


class SinusoidalPositionalEncoding(Module):
    """``pe[p, 2k] = sin(p w_k)``, ``pe[p, 2k+1] = cos(p w_k)``, ``w_k = 10000^(-2k/D)``; added to the input
    (reference: lib/core/nn/positional.dart:27-100)."""

    def __init__(self, dim: int):
        super().__init__()
        self.dim = dim

    def table(self, n: int, start_pos: int, device, dtype):
        pos = torch.arange(start_pos, start_pos + n, dtype=torch.float64, device=device).unsqueeze(1)
        i = torch.arange(self.dim, dtype=torch.float64, device=device)
        freq = torch.pow(10000.0, -2.0 * torch.floor(i / 2.0) / self.dim)
        ang = pos * freq
        pe = torch.where((torch.arange(self.dim, device=device) % 2 == 0), torch.sin(ang), torch.cos(ang))
        return pe.to(dtype)

    def forward(self, x, start_pos: int = 0):
        if x.dim() not in (2, 3):
            raise ValueError("SinusoidalPositionalEncoding: input must be [N, D] or [B, N, D]")
        return F.add(x, self.table(x.shape[-2], start_pos, x.device, x.dtype).expand_as(x).contiguous())


class LearnedPositionalEmbedding(Module):
    """Learned table ``[maxLen, D]`` added to the input (reference: lib/core/nn/positional.dart:102-159)."""

    def __init__(self, max_len: int, dim: int, device=None, seed: int = 0, dtype=torch.float32,
                 init_std: Optional[float] = None):
        super().__init__()
        self.max_len, self.dim = max_len, dim
        self.table = Embedding(max_len, dim, device=device, seed=seed, dtype=dtype, init_std=init_std)

    def submodules(self):
        return [self.table]

    def forward(self, x, start_pos: int = 0):
        n = x.shape[-2]
        if start_pos + n > self.max_len:
            raise ValueError(f"LearnedPositionalEmbedding: positions {start_pos}..{start_pos + n} exceed {self.max_len}")
        idx = torch.arange(start_pos, start_pos + n, device=x.device)
        pe = F.embedding(self.table.weight, idx)
        return F.add(x, pe.expand_as(x).contiguous()) if x.dim() == 3 else F.add(x, pe)


class SwiGluFfn(Module):
    """``down(silu(gate(x)) * up(x))``, three bias-free projections.  Gate and up share one ``[2*hidden, dim]`` weight so
    they are one GEMM; exported as gate, up, down (reference: lib/core/nn/ffn/swiglu.dart:26-73)."""

    def __init__(self, dim: int, hidden: int, device=None, seed: int = 0, dtype=torch.float32,
                 init_std: Optional[float] = None):
        super().__init__()
        self.dim, self.hidden = dim, hidden
        gate = Linear(dim, hidden, bias=False, device=device, seed=seed, dtype=dtype, init_std=init_std)
        up = Linear(dim, hidden, bias=False, device=device, seed=seed + 1000, dtype=dtype, init_std=init_std)
        self.w_gate_up = make_param(torch.cat([gate.weight.data, up.weight.data], 0))
        self.down = Linear(hidden, dim, bias=False, device=device, seed=seed + 2000, dtype=dtype, init_std=init_std)

    def own_parameters(self):
        return [self.w_gate_up]

    def own_reference_parameters(self):
        return [self.w_gate_up.data[:self.hidden], self.w_gate_up.data[self.hidden:]]

    def submodules(self):
        return [self.down]

    def forward(self, x, residual=None):
        gu = F.linear(x, self.w_gate_up)
        return self.down(F.swiglu(gu), residual=residual)


class VisionProjector(Module):
    """``down(silu(up(x)))`` (reference: lib/core/nn/vision_projector.dart:23-73)."""

    def __init__(self, in_dim: int, out_dim: int, hidden: Optional[int] = None, device=None, seed: int = 0,
                 dtype=torch.float32):
        super().__init__()
        hidden = hidden or out_dim
        self.in_dim, self.out_dim, self.hidden_dim = in_dim, out_dim, hidden
        self.up = Linear(in_dim, hidden, device=device, seed=seed, dtype=dtype)
        self.down = Linear(hidden, out_dim, device=device, seed=seed + 1000, dtype=dtype)

    def submodules(self):
        return [self.up, self.down]

    def forward(self, x):
        return self.down(self.up(x, activation="silu"))


def causal_mask(n: int, block_value: float = -1e9, device=None, dtype=torch.float32):
    """Additive ``[n, n]`` mask with ``block_value`` above the diagonal (reference: lib/core/nn/masks.dart:16-28)."""
    return F.causal_mask(n, block_value, device, dtype)
