"""Device attention: autograd wrappers over the tcgen05 flash-attention kernels (``csrc/attention_*.cu``).

Tensors are token-major: element ``(b, s, head, d)`` of Q lives at row ``b*S + s``, column ``head*hd + d`` of a 2-D
matrix, which is exactly what a fused QKV projection writes and what the output projection reads, so no
split / permute / concat kernels run around the attention kernel (the reference concatenates per-head results on the
host: lib/core/nn/attention/multi_head_attention.dart:167-196).
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional

import torch

from .. import _native as N
from . import reference as ref

c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


class AttnFwdArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("o", c_void_p), ("lse", c_void_p),
                ("ldq", c_ll), ("ldk", c_ll), ("ldv", c_ll), ("ldo", c_ll),
                ("B", c_int), ("Sq", c_int), ("Sk", c_int), ("Hq", c_int), ("Hkv", c_int), ("head_dim", c_int),
                ("causal", c_int), ("q_offset", c_int), ("scale", c_float), ("kv_batch_rows", c_ll)]


class AttnBwdArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("o", c_void_p), ("do", c_void_p),
                ("lse", c_void_p), ("delta", c_void_p), ("dq_acc", c_void_p), ("dq", c_void_p), ("dk", c_void_p),
                ("dv", c_void_p),
                ("ldq", c_ll), ("ldk", c_ll), ("ldv", c_ll), ("ldo", c_ll), ("lddo", c_ll), ("lddq", c_ll),
                ("lddk", c_ll), ("lddv", c_ll),
                ("B", c_int), ("Sq", c_int), ("Sk", c_int), ("Hq", c_int), ("Hkv", c_int), ("head_dim", c_int),
                ("causal", c_int), ("q_offset", c_int), ("scale", c_float)]


def kernel_head_dim(hd: int, backward: bool = False) -> Optional[int]:
    """Head size the tensor-core kernels run a head of ``hd`` features at: 64 and 128 directly (the backward kernel
    exists for 64 only), smaller sizes that are a multiple of 8 zero-padded to 64 (zeros add nothing to the scores and
    give zero output columns), sizes between 64 and 128 padded to 128 in forward.  ``None`` = no kernel for it."""
    if hd <= 0 or hd % 8:
        return None
    if backward and deterministic():
        return None          # the backward kernel sums dQ with fp32 atomics: run-to-run order is not fixed
    if hd <= 64:
        return 64
    if hd <= 128 and not backward:
        return 128
    return None


def deterministic() -> bool:
    """``DPTB200_DETERMINISTIC=1``: bit-identical results from run to run.  Every reduction in this package is ordered
    (two-stage column sums, split-K folded in split order, sorted embedding scatter, fixed rank order in the collective
    kernels) except the flash attention backward, whose dQ tiles from different key tiles meet in fp32 ``red.add``; with
    the flag, attention that needs gradients takes the composed GEMM + softmax path instead."""
    return os.environ.get("DPTB200_DETERMINISTIC", "0") not in ("0", "", "false", "False")


def supported_head_dim(hd: int, backward: bool = False) -> bool:
    return kernel_head_dim(hd, backward) is not None


def _wants_grad(*tensors) -> bool:
    return torch.is_grad_enabled() and any(t.requires_grad for t in tensors)


def _pad_heads(x2: torch.Tensor, heads: int, hd: int, to: int) -> torch.Tensor:
    """Token-major ``[rows, heads*hd]`` -> ``[rows, heads*to]`` with zeros behind every head's features."""
    return torch.nn.functional.pad(x2.reshape(x2.shape[0], heads, hd), (0, to - hd)).reshape(x2.shape[0], heads * to)


def _to_bhsd(x2: torch.Tensor, batch: int, seq: int, heads: int, hd: int) -> torch.Tensor:
    return x2.reshape(batch, seq, heads, hd).transpose(1, 2)


def _ld(t: torch.Tensor) -> int:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError("attention operands must be 2-D with a contiguous last axis")
    return t.stride(0)


def attn_fwd(q2, k2, v2, B, Sq, Sk, Hq, Hkv, hd, causal, q_offset=0, scale=None, need_lse=True, out=None,
             kv_batch_rows=0):
    """Forward kernel call on token-major 2-D views (``q2``: ``[B*Sq, >= Hq*hd]`` etc.).  Returns ``(o, lse)``."""
    lib = N.load()
    if out is None:
        out = torch.empty(B * Sq, Hq * hd, dtype=torch.bfloat16, device=q2.device)
    lse = torch.empty(B, Hq, Sq, dtype=torch.float32, device=q2.device) if need_lse else None
    a = AttnFwdArgs()
    a.q, a.k, a.v, a.o, a.lse = q2.data_ptr(), k2.data_ptr(), v2.data_ptr(), out.data_ptr(), N.ptr(lse)
    a.ldq, a.ldk, a.ldv, a.ldo = _ld(q2), _ld(k2), _ld(v2), _ld(out)
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.head_dim = B, Sq, Sk, Hq, Hkv, hd
    a.causal, a.q_offset = int(causal), int(q_offset)
    a.scale = (1.0 / math.sqrt(hd)) if scale is None else scale
    a.kv_batch_rows = kv_batch_rows
    N.check(lib.dptb_attn_fwd(ctypes.byref(a), N.stream_ptr()), "attn_fwd")
    return out, lse


def attn_bwd(q2, k2, v2, o2, do2, lse, dq2, dk2, dv2, B, Sq, Sk, Hq, Hkv, hd, causal, q_offset=0, scale=None):
    """Backward kernel call; writes dQ / dK / dV into the given token-major 2-D views."""
    lib = N.load()
    delta = torch.empty(B, Hq, Sq, dtype=torch.float32, device=q2.device)
    dq_acc = torch.zeros(B * Sq, Hq * hd, dtype=torch.float32, device=q2.device)
    a = AttnBwdArgs()
    a.q, a.k, a.v, a.o, a.do = q2.data_ptr(), k2.data_ptr(), v2.data_ptr(), o2.data_ptr(), do2.data_ptr()
    a.lse, a.delta, a.dq_acc = lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr()
    a.dq, a.dk, a.dv = dq2.data_ptr(), dk2.data_ptr(), dv2.data_ptr()
    a.ldq, a.ldk, a.ldv, a.ldo, a.lddo = _ld(q2), _ld(k2), _ld(v2), _ld(o2), _ld(do2)
    a.lddq, a.lddk, a.lddv = _ld(dq2), _ld(dk2), _ld(dv2)
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.head_dim = B, Sq, Sk, Hq, Hkv, hd
    a.causal, a.q_offset = int(causal), int(q_offset)
    a.scale = (1.0 / math.sqrt(hd)) if scale is None else scale
    N.check(lib.dptb_attn_bwd(ctypes.byref(a), N.stream_ptr()), "attn_bwd")


class PackedAttentionFn(torch.autograd.Function):
    """Attention over a fused projection output ``qkv`` ``[B*S, (H + 2 Hkv) hd]`` -> ``[B*S, H hd]``."""

    @staticmethod
    def forward(ctx, qkv, B, S, H, Hkv, hd, causal):
        dq, dkv = H * hd, Hkv * hd
        q2, k2, v2 = qkv[:, :dq], qkv[:, dq:dq + dkv], qkv[:, dq + dkv:]
        o, lse = attn_fwd(q2, k2, v2, B, S, S, H, Hkv, hd, causal, need_lse=True)
        ctx.save_for_backward(qkv, o, lse)
        ctx.cfg = (B, S, H, Hkv, hd, causal)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse = ctx.saved_tensors
        B, S, H, Hkv, hd, causal = ctx.cfg
        dq, dkv = H * hd, Hkv * hd
        do = do if do.is_contiguous() else do.contiguous()
        dqkv = torch.empty_like(qkv)
        attn_bwd(qkv[:, :dq], qkv[:, dq:dq + dkv], qkv[:, dq + dkv:], o, do, lse,
                 dqkv[:, :dq], dqkv[:, dq:dq + dkv], dqkv[:, dq + dkv:], B, S, S, H, Hkv, hd, causal)
        return dqkv, None, None, None, None, None, None


class SeparateAttentionFn(torch.autograd.Function):
    """Attention over separate token-major ``q [B*Sq, H hd]``, ``k``/``v`` ``[B*Sk, Hkv hd]``."""

    @staticmethod
    def forward(ctx, q2, k2, v2, B, Sq, Sk, H, Hkv, hd, causal, q_offset, scale=None):
        o, lse = attn_fwd(q2, k2, v2, B, Sq, Sk, H, Hkv, hd, causal, q_offset=q_offset, scale=scale, need_lse=True)
        ctx.save_for_backward(q2, k2, v2, o, lse)
        ctx.cfg = (B, Sq, Sk, H, Hkv, hd, causal, q_offset, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        q2, k2, v2, o, lse = ctx.saved_tensors
        B, Sq, Sk, H, Hkv, hd, causal, q_offset, scale = ctx.cfg
        do = do if do.is_contiguous() else do.contiguous()
        dq, dk, dv = torch.empty_like(q2), torch.empty_like(k2), torch.empty_like(v2)
        attn_bwd(q2, k2, v2, o, do, lse, dq, dk, dv, B, Sq, Sk, H, Hkv, hd, causal, q_offset=q_offset, scale=scale)
        return dq, dk, dv, None, None, None, None, None, None, None, None, None


def attention_packed(qkv, batch, seq, heads, kv_heads, head_dim, causal=True):
    """Attention over a fused projection output ``[B*S, (H + 2 Hkv) hd]`` -> ``[B*S, H hd]``."""
    d_q, d_kv = heads * head_dim, kv_heads * head_dim
    hd_k = kernel_head_dim(head_dim, backward=_wants_grad(qkv)) if qkv.dtype == torch.bfloat16 else None
    if hd_k == head_dim:
        return PackedAttentionFn.apply(qkv, batch, seq, heads, kv_heads, head_dim, causal)
    return attention_tokens(qkv[:, :d_q], qkv[:, d_q:d_q + d_kv], qkv[:, d_q + d_kv:], batch, seq, seq, heads, kv_heads,
                            head_dim, causal)


def attention_tokens(q2, k2, v2, batch, sq, sk, heads, kv_heads, head_dim, causal=True, q_offset=0):
    """Token-major separate operands ``q2 [B*Sq, H hd]``, ``k2`` / ``v2`` ``[B*Sk, Hkv hd]`` (with a KV cache: cache
    views) -> ``[B*Sq, H hd]``.  bf16 heads of 64 / 128 features run the tensor-core kernels as they are, other sizes
    zero-padded to the next of the two; what the kernels do not cover (see ``kernel_head_dim``) runs the composed path."""
    hd_k = kernel_head_dim(head_dim, backward=_wants_grad(q2, k2, v2)) if q2.dtype == torch.bfloat16 else None
    if hd_k is None:
        o = _attention_composed(_to_bhsd(q2, batch, sq, heads, head_dim), _to_bhsd(k2, batch, sk, kv_heads, head_dim),
                                _to_bhsd(v2, batch, sk, kv_heads, head_dim), causal, None, q_offset)
        return o.transpose(1, 2).reshape(batch * sq, heads * head_dim)
    if hd_k == head_dim:
        return SeparateAttentionFn.apply(q2, k2, v2, batch, sq, sk, heads, kv_heads, head_dim, causal, q_offset)
    o = SeparateAttentionFn.apply(_pad_heads(q2, heads, head_dim, hd_k), _pad_heads(k2, kv_heads, head_dim, hd_k),
                                  _pad_heads(v2, kv_heads, head_dim, hd_k), batch, sq, sk, heads, kv_heads, hd_k, causal,
                                  q_offset, 1.0 / math.sqrt(head_dim))
    return o.reshape(batch * sq, heads, hd_k)[:, :, :head_dim].reshape(batch * sq, heads * head_dim)


def attention_bhsd(q, k, v, causal=False, mask=None, q_offset=0):
    """``[B, H, S, hd]`` operands.  bf16 with a supported head size runs the tensor-core kernel (after a
    token-major relayout); anything else (fp32, odd head sizes, an additive mask) runs the composed
    device path: score GEMMs on the SIMT kernel, row softmax kernel."""
    B, H, Sq, hd = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    if q.dtype == torch.bfloat16 and mask is None and supported_head_dim(hd, backward=_wants_grad(q, k, v)):
        q2 = q.transpose(1, 2).reshape(B * Sq, H * hd)
        k2 = k.transpose(1, 2).reshape(B * Sk, Hkv * hd)
        v2 = v.transpose(1, 2).reshape(B * Sk, Hkv * hd)
        o = attention_tokens(q2, k2, v2, B, Sq, Sk, H, Hkv, hd, causal, q_offset)
        return o.reshape(B, Sq, H, hd).transpose(1, 2)
    return _attention_composed(q, k, v, causal, mask, q_offset)


def _attention_composed(q, k, v, causal, mask, q_offset):
    """Generic path built from the library's own GEMM / softmax ops, one (batch, head) at a time."""
    from . import matmul, softmax, transpose
    from . import cuda as C
    B, H, Sq, hd = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    g = H // Hkv
    scale = 1.0 / math.sqrt(hd)
    add = None
    if causal:
        i = torch.arange(Sq, device=q.device).unsqueeze(1) + q_offset
        j = torch.arange(Sk, device=q.device).unsqueeze(0)
        add = torch.where(j > i, -1e9, 0.0).to(q.dtype)
    if mask is not None:
        add = mask.to(q.dtype) if add is None else add + mask.to(q.dtype)
    outs = []
    for b in range(B):
        heads = []
        for h in range(H):
            qh, kh, vh = q[b, h].contiguous(), k[b, h // g].contiguous(), v[b, h // g].contiguous()
            s = C.UnaryFn.apply(matmul(qh, transpose(kh)), "scale", scale)
            if add is not None:
                s = C.BinaryFn.apply(s, add.expand(Sq, Sk).contiguous(), "add")
            heads.append(matmul(softmax(s), vh))
        outs.append(torch.stack(heads, 0))
    return torch.stack(outs, 0)
