"""Decode-path kernels: attention over a KV cache for a few new query tokens, and the fused rotary + cache append
(``csrc/attention_decode.cu``).  CPU tensors run reference formulas with the same contracts."""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from .. import _native as N

c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


class DecodeArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("o", c_void_p), ("ws", c_void_p),
                ("ws_floats", c_ll), ("ldq", c_ll), ("ldkv", c_ll), ("ldo", c_ll), ("kv_batch_stride", c_ll),
                ("B", c_int), ("Sq", c_int), ("Sk", c_int), ("Hq", c_int), ("Hkv", c_int), ("head_dim", c_int),
                ("splits", c_int), ("q_offset", c_int), ("scale", c_float), ("pos_ptr", c_void_p), ("cap", c_int)]


_declared = False


def _lib():
    global _declared
    lib = N.load()
    if not _declared:
        lib.dptb_attn_decode.argtypes = [ctypes.POINTER(DecodeArgs), c_void_p]
        lib.dptb_attn_decode.restype = c_int
        lib.dptb_attn_decode_ws_floats.argtypes = [c_int] * 5
        lib.dptb_attn_decode_ws_floats.restype = c_ll
        lib.dptb_attn_decode_splits.argtypes = [c_int] * 4
        lib.dptb_attn_decode_splits.restype = c_int
        lib.dptb_attn_decode_splits_hd.argtypes = [c_int] * 5
        lib.dptb_attn_decode_splits_hd.restype = c_int
        lib.dptb_rope_kv_append.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_ll] + [c_int] * 7 + \
            [c_float, c_int, c_void_p, c_void_p]
        lib.dptb_rope_kv_append.restype = c_int
        _declared = True
    return lib


def attn_decode_reference(q2, k_cache, v_cache, B, Sq, Sk, Hq, Hkv, hd, q_offset, scale=None):
    """fp32 formulas: ``q2 [B*Sq, >= Hq*hd]``, caches ``[B, cap, >= Hkv*hd]``; query row ``i`` sees keys
    ``<= q_offset + i``."""
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    q = q2[:, :Hq * hd].float().reshape(B, Sq, Hq, hd).permute(0, 2, 1, 3)
    k = k_cache[:, :Sk, :Hkv * hd].float().reshape(B, Sk, Hkv, hd).permute(0, 2, 1, 3)
    v = v_cache[:, :Sk, :Hkv * hd].float().reshape(B, Sk, Hkv, hd).permute(0, 2, 1, 3)
    g = Hq // Hkv
    k, v = k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1)
    s = q @ k.transpose(-1, -2) * scale
    qi = torch.arange(Sq, device=s.device).view(Sq, 1) + q_offset
    kj = torch.arange(Sk, device=s.device).view(1, Sk)
    s = s.masked_fill(kj > qi, float("-inf"))
    o = torch.softmax(s, -1) @ v
    return o.permute(0, 2, 1, 3).reshape(B * Sq, Hq * hd)


def attn_decode(q2: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, B: int, Sq: int, Sk: int, Hq: int,
                Hkv: int, hd: int, q_offset: int, scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
                splits: int = 0, workspace: Optional[torch.Tensor] = None,
                pos: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of ``Sq`` new query rows per sequence over the first ``Sk`` cache rows (which already include the
    new tokens).  ``q2``: ``[B*Sq, >= Hq*hd]`` bf16; caches ``[B, cap, Hkv*hd]`` bf16.  Returns ``[B*Sq, Hq*hd]``.
    With ``pos`` (an int32 device scalar) the kernel takes ``q_offset = pos`` and ``Sk = pos + Sq`` from the device;
    ``Sk`` then only sizes the split of the keys (pass the largest context that will be reached)."""
    if not q2.is_cuda:
        o = attn_decode_reference(q2, k_cache, v_cache, B, Sq, Sk, Hq, Hkv, hd, q_offset, scale).to(q2.dtype)
        if out is not None:
            out.copy_(o)
            return out
        return o
    lib = _lib()
    for t in (q2, k_cache, v_cache):
        if t.dtype != torch.bfloat16 or t.stride(-1) != 1:
            raise TypeError("attn_decode: q / k / v must be bfloat16 with a contiguous last axis")
    if k_cache.dim() != 3 or k_cache.shape != v_cache.shape or k_cache.stride() != v_cache.stride():
        raise ValueError("attn_decode: caches must be [B, cap, Hkv*hd] with equal layouts")
    if Sk > k_cache.shape[1] or B > k_cache.shape[0]:
        raise ValueError("attn_decode: Sk / B exceed the cache")
    if out is None:
        out = torch.empty(B * Sq, Hq * hd, dtype=torch.bfloat16, device=q2.device)
    if splits <= 0:
        splits = int(lib.dptb_attn_decode_splits_hd(B, Sq, Hkv, Sk, hd))
    need = int(lib.dptb_attn_decode_ws_floats(B, Sq, Hq, hd, splits))
    if need and (workspace is None or workspace.numel() < need):
        workspace = torch.empty(need, dtype=torch.float32, device=q2.device)
    a = DecodeArgs()
    a.q, a.k, a.v, a.o = q2.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr()
    a.ws, a.ws_floats = (workspace.data_ptr(), workspace.numel()) if need else (None, 0)
    a.ldq, a.ldkv, a.ldo, a.kv_batch_stride = q2.stride(0), k_cache.stride(1), out.stride(0), k_cache.stride(0)
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.head_dim = B, Sq, Sk, Hq, Hkv, hd
    a.splits, a.q_offset = splits, q_offset
    a.pos_ptr, a.cap = (pos.data_ptr() if pos is not None else None), k_cache.shape[1]
    a.scale = 1.0 / math.sqrt(hd) if scale is None else scale
    N.check(lib.dptb_attn_decode(ctypes.byref(a), N.stream_ptr()), "attn_decode")
    return out


def decode_workspace_floats(B: int, Sq: int, Hq: int, Hkv: int, hd: int, max_sk: int) -> int:
    """Workspace size that covers every context length up to ``max_sk`` (for preallocation before graph capture)."""
    lib = _lib()
    splits = int(lib.dptb_attn_decode_splits_hd(B, Sq, Hkv, max_sk, hd))
    return int(lib.dptb_attn_decode_ws_floats(B, Sq, Hq, hd, max(splits, 1)))


def rope_kv_append_reference(qkv, k_cache, v_cache, B, S, Hq, Hkv, hd, pos0, rotary_dim, base):
    dq, dkv = Hq * hd, Hkv * hd
    x = qkv.float().reshape(B, S, -1)
    pos = torch.arange(pos0, pos0 + S, device=qkv.device, dtype=torch.float32)
    half = rotary_dim // 2
    inv = base ** (-2.0 * torch.arange(half, device=qkv.device, dtype=torch.float32) / rotary_dim)
    ang = pos.view(S, 1) * inv.view(1, half)
    cs, sn = torch.cos(ang).view(1, S, 1, half), torch.sin(ang).view(1, S, 1, half)

    def rot(t, heads):
        t = t.reshape(B, S, heads, hd).clone()
        a, b = t[..., :half].clone(), t[..., half:rotary_dim].clone()
        t[..., :half] = a * cs - b * sn
        t[..., half:rotary_dim] = b * cs + a * sn
        return t.reshape(B, S, heads * hd)
    q = rot(x[..., :dq], Hq)
    k = rot(x[..., dq:dq + dkv], Hkv)
    v = x[..., dq + dkv:dq + 2 * dkv]
    qkv.reshape(B, S, -1)[..., :dq] = q.to(qkv.dtype)
    k_cache[:B, pos0:pos0 + S, :dkv] = k.to(k_cache.dtype)
    v_cache[:B, pos0:pos0 + S, :dkv] = v.to(v_cache.dtype)


def rope_kv_append(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, B: int, S: int, Hq: int, Hkv: int,
                   hd: int, pos0: int, rotary_dim: Optional[int] = None, base: float = 10000.0,
                   pos: Optional[torch.Tensor] = None) -> None:
    """In place: rotate the Q heads of ``qkv [B*S, (Hq + 2 Hkv) hd]``; rotate K and write K / V rows into the caches
    ``[B, cap, Hkv*hd]`` at positions ``pos0 .. pos0 + S``."""
    rotary_dim = hd if rotary_dim is None else rotary_dim
    if pos0 + S > k_cache.shape[1]:
        raise ValueError(f"rope_kv_append: positions up to {pos0 + S} exceed the cache capacity {k_cache.shape[1]}")
    if not qkv.is_cuda:
        return rope_kv_append_reference(qkv, k_cache, v_cache, B, S, Hq, Hkv, hd, pos0, rotary_dim, base)
    lib = _lib()
    if qkv.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16:
        raise TypeError("rope_kv_append: tensors must be bfloat16")
    if k_cache.stride() != v_cache.stride() or k_cache.stride(-1) != 1 or qkv.stride(-1) != 1:
        raise ValueError("rope_kv_append: unsupported layout")
    N.check(lib.dptb_rope_kv_append(qkv.data_ptr(), qkv.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
                                    k_cache.stride(1), k_cache.stride(0), B, S, Hq, Hkv, hd, pos0, rotary_dim,
                                    float(base), k_cache.shape[1], pos.data_ptr() if pos is not None else None,
                                    N.stream_ptr()), "rope_kv_append")
