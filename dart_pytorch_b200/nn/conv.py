"""2-D convolution as lowering + GEMM (reference: lib/core/nn/conv2d.dart:22-208).

NCHW in and out; weight ``[Cout, Cin, Kh, Kw]`` ~ U(+-1/sqrt(Cin*Kh*Kw)), bias ``[Cout]`` zeros.  The reference lowers
on the host and differentiates only through the matmul (weight / bias); here the lowering is a device kernel with its
adjoint, so the input gradient flows too and the output stays on the input's device.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops as F
from .module import Module, make_param, uniform_


class _Im2ColFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kh, kw, stride, pad):
        from ..ops import kernels as K
        ctx.geom = (tuple(x.shape), kh, kw, stride, pad)
        return K.im2col_nchw(x, kh, kw, stride, pad)

    @staticmethod
    def backward(ctx, dcols):
        from ..ops import kernels as K
        shape, kh, kw, stride, pad = ctx.geom
        return K.col2im_nchw(dcols, shape, kh, kw, stride, pad), None, None, None, None


def im2col(x, kh: int, kw: int, stride: int = 1, pad: int = 0):
    """``[B, C, H, W] -> [B*Ho*Wo, C*kh*kw]`` (column order ``(c, ky, kx)``), differentiable."""
    if x.is_cuda:
        return _Im2ColFn.apply(x, kh, kw, stride, pad)
    cols = torch.nn.functional.unfold(x, (kh, kw), padding=pad, stride=stride)       # [B, C*kh*kw, L]
    return cols.transpose(1, 2).reshape(-1, cols.shape[1])


class Conv2d(Module):
    def __init__(self, in_channels: int, out_channels: int, kernel: int = 3, kernel_h: Optional[int] = None,
                 kernel_w: Optional[int] = None, stride: int = 1, padding: int = 0, bias: bool = True, device=None,
                 seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_h, self.kernel_w = kernel_h or kernel, kernel_w or kernel
        self.stride, self.padding = stride, padding
        fan_in = in_channels * self.kernel_h * self.kernel_w
        self.weight = make_param(uniform_((out_channels, in_channels, self.kernel_h, self.kernel_w),
                                          1.0 / math.sqrt(fan_in), seed, device, dtype))
        self.bias = make_param(torch.zeros(out_channels, device=device, dtype=dtype)) if bias else None

    def own_parameters(self):
        return [self.weight] + ([self.bias] if self.bias is not None else [])

    def out_size(self, h: int, w: int):
        ho = (h + 2 * self.padding - self.kernel_h) // self.stride + 1
        wo = (w + 2 * self.padding - self.kernel_w) // self.stride + 1
        return ho, wo

    def forward(self, x):
        squeeze = x.dim() == 3
        if squeeze:
            x = x.unsqueeze(0)
        if x.dim() != 4 or x.shape[1] != self.in_channels:
            raise ValueError(f"Conv2d: expected [B, {self.in_channels}, H, W]; got {list(x.shape)}")
        B, _, H, W = x.shape
        ho, wo = self.out_size(H, W)
        if ho <= 0 or wo <= 0:
            raise ValueError(f"Conv2d: kernel {self.kernel_h}x{self.kernel_w} larger than padded input {H}x{W}")
        cols = im2col(x, self.kernel_h, self.kernel_w, self.stride, self.padding)    # [B*ho*wo, Cin*kh*kw]
        y = F.linear(cols, self.weight.reshape(self.out_channels, -1), self.bias)    # [B*ho*wo, Cout]
        y = y.reshape(B, ho, wo, self.out_channels).permute(0, 3, 1, 2).contiguous()
        return y[0] if squeeze else y
