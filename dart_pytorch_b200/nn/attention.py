"""Multi-head attention (GQA, RoPE, KV cache), cross-attention, rotary cache and the KV-cache containers.

The reference keeps one small ``Linear`` per head and loops over heads and batch elements in the host language
(lib/core/nn/attention/multi_head_attention.dart:27-253).  Here the projections are stored as ONE fused
``[(H + 2 Hkv) hd, D]`` weight, the whole layer is projection GEMM -> (RoPE) -> flash attention -> output GEMM, and the
per-head tensors of the reference exist only as views for checkpoints (``reference_parameters``).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import ops as F
from .layers import Dropout, Linear
from .module import Module, make_param, uniform_, normal_


class RopeCache:
    """Rotary position configuration.  Angles are computed from ``(position, i)`` inside the kernel, so nothing is
    precomputed; the class keeps the reference's constructor and ``apply`` contract
    (reference: lib/core/nn/rotary.dart:28-202)."""

    def __init__(self, max_ctx: int, head_dim: int, rotary_dim: Optional[int] = None, base: float = 10000.0,
                 device=None):
        rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if rotary_dim % 2 or rotary_dim > head_dim or rotary_dim <= 0:
            raise ValueError("RopeCache: rotaryDim must be even and in (0, headDim]")
        self.max_ctx, self.head_dim, self.rotary_dim, self.base = max_ctx, head_dim, rotary_dim, float(base)

    def check_window(self, start_pos: int, n: int) -> None:
        if start_pos < 0 or start_pos + n > self.max_ctx:
            raise ValueError(f"RopeCache: window [{start_pos}, {start_pos + n}) exceeds maxCtx {self.max_ctx}")

    def apply(self, x, start_pos: int = 0, heads: int = 1):
        """Rotate ``x [..., N, heads*headDim]`` at positions ``start_pos .. start_pos+N-1``."""
        self.check_window(start_pos, x.shape[-2])
        return F.rope(x, start_pos, self.base, self.rotary_dim, heads=heads)


class MHACache:
    """Device KV cache of one attention layer: ``k`` / ``v`` buffers ``[B, capacity, Hkv*hd]`` written in place.
    ``seq_len`` tokens are valid.  (The reference grows per-head tensors by concatenation through the host:
    lib/core/nn/kv_cache.dart:22-63.)"""

    def __init__(self, num_kv_heads: int, max_len: int = 0):
        self.num_kv_heads = num_kv_heads
        self.max_len = max_len
        self.k_buf: Optional[torch.Tensor] = None
        self.v_buf: Optional[torch.Tensor] = None
        self.seq_len = 0

    @property
    def seqLen(self) -> int:
        return self.seq_len

    def _ensure(self, batch: int, need: int, width: int, like: torch.Tensor) -> None:
        cap = 0 if self.k_buf is None else self.k_buf.shape[1]
        if self.k_buf is not None and (self.k_buf.shape[0] != batch or self.k_buf.shape[2] != width):
            raise ValueError("MHACache: batch size or width changed between calls")
        if need <= cap:
            return
        new_cap = max(need, self.max_len, 2 * cap, 16)
        new_cap = (new_cap + 127) // 128 * 128
        k = torch.zeros(batch, new_cap, width, dtype=like.dtype, device=like.device)
        v = torch.zeros_like(k)
        if self.k_buf is not None and self.seq_len:
            k[:, :self.seq_len] = self.k_buf[:, :self.seq_len]
            v[:, :self.seq_len] = self.v_buf[:, :self.seq_len]
        self.k_buf, self.v_buf = k, v

    def append(self, k_new: torch.Tensor, v_new: torch.Tensor):
        """Append ``[B, S, Hkv*hd]`` keys / values; returns views of the full valid history."""
        b, s, w = k_new.shape
        self._ensure(b, self.seq_len + s, w, k_new)
        self.k_buf[:, self.seq_len:self.seq_len + s] = k_new
        self.v_buf[:, self.seq_len:self.seq_len + s] = v_new
        self.seq_len += s
        self.__dict__.pop("_fills", None)
        return self.k_buf[:, :self.seq_len], self.v_buf[:, :self.seq_len]

    # Per-head accessors with the reference's shapes (``[T_seen, hd]``, batch 1).
    def _head(self, buf, h):
        hd = buf.shape[2] // self.num_kv_heads
        return buf[0, :self.seq_len, h * hd:(h + 1) * hd]

    @property
    def k(self) -> List[Optional[torch.Tensor]]:
        return [None if self.k_buf is None else self._head(self.k_buf, h) for h in range(self.num_kv_heads)]

    @property
    def v(self) -> List[Optional[torch.Tensor]]:
        return [None if self.v_buf is None else self._head(self.v_buf, h) for h in range(self.num_kv_heads)]

    # Per-head appends with the reference's signature (``[N_new, hd]`` for one KV head; returns that head's full
    # history).  They write into the same buffers; the cache length follows the furthest head.
    def _append_head(self, which: str, kv_head: int, new: torch.Tensor) -> torch.Tensor:
        if not (0 <= kv_head < self.num_kv_heads):
            raise IndexError(f"MHACache: kv head {kv_head} out of range [0, {self.num_kv_heads})")
        n, hd = new.shape
        fills = self.__dict__.setdefault("_fills", {"base": self.seq_len})    # rows valid before per-head appends began
        fill = fills.setdefault(which, [fills["base"]] * self.num_kv_heads)
        start = fill[kv_head]
        self._ensure(1, start + n, self.num_kv_heads * hd, new)
        buf = self.k_buf if which == "k" else self.v_buf
        buf[0, start:start + n, kv_head * hd:(kv_head + 1) * hd] = new.detach()
        fill[kv_head] = start + n
        self.seq_len = max(self.seq_len, start + n)
        return buf[0, :start + n, kv_head * hd:(kv_head + 1) * hd]

    def append_k(self, kv_head: int, new_k: torch.Tensor) -> torch.Tensor:
        return self._append_head("k", kv_head, new_k)

    def append_v(self, kv_head: int, new_v: torch.Tensor) -> torch.Tensor:
        return self._append_head("v", kv_head, new_v)

    appendK, appendV = append_k, append_v

    def reset(self) -> None:
        self.seq_len = 0
        self.__dict__.pop("_fills", None)


class EncoderCache:
    """One ``MHACache`` per layer (reference: lib/core/nn/kv_cache.dart:66-84)."""

    def __init__(self, layers: List[MHACache]):
        self.layers = layers

    @staticmethod
    def empty(num_layers: int, num_kv_heads: int, max_len: int = 0) -> "EncoderCache":
        return EncoderCache([MHACache(num_kv_heads, max_len) for _ in range(num_layers)])

    @property
    def seq_len(self) -> int:
        return self.layers[0].seq_len if self.layers else 0

    seqLen = seq_len

    def reset(self) -> None:
        for c in self.layers:
            c.reset()


class MultiHeadAttention(Module):
    """Self-attention with grouped-query sharing, optional RoPE and KV cache
    (reference: lib/core/nn/attention/multi_head_attention.dart:27-253).

    Parameters (storage): ``w_qkv [(H + 2 Hkv) hd, D]`` (+ ``b_qkv``), ``wo`` (+ bias).  Checkpoint order: every
    ``wq[h]`` ``[hd, D]`` (+ ``[1, hd]`` bias), every ``wk[h]``, every ``wv[h]``, then ``wo``.
    """

    def __init__(self, embed_dim: int, num_heads: int, num_kv_heads: Optional[int] = None, bias: bool = False,
                 dropout_p: float = 0.0, device=None, seed: int = 0, rope: Optional[RopeCache] = None,
                 dtype=torch.float32, init_std: Optional[float] = None, head_dim: Optional[int] = None):
        super().__init__()
        num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        if head_dim is None and embed_dim % num_heads:
            raise ValueError("MultiHeadAttention: embedDim must be divisible by numHeads")
        if num_kv_heads <= 0 or num_heads % num_kv_heads:
            raise ValueError("MultiHeadAttention: numHeads must be a multiple of numKvHeads")
        self.embed_dim, self.num_heads, self.num_kv_heads = embed_dim, num_heads, num_kv_heads
        self.head_dim = head_dim or embed_dim // num_heads
        self.num_head_groups = num_heads // num_kv_heads
        self.rope = rope
        hd, D = self.head_dim, embed_dim
        bound = 1.0 / math.sqrt(D)
        rows, brows = [], []
        # Per-head seeds follow the reference: wq seed+h, wk seed+1000+h, wv seed+2000+h, wo seed+3000.
        for base, count in ((0, num_heads), (1000, num_kv_heads), (2000, num_kv_heads)):
            for h in range(count):
                if init_std is None:
                    rows.append(uniform_((hd, D), bound, seed + base + h, device, dtype))
                    brows.append(uniform_((hd,), bound, seed + base + h + 1, device, dtype))
                else:
                    rows.append(normal_((hd, D), init_std, seed + base + h, device, dtype))
                    brows.append(torch.zeros(hd, device=device, dtype=dtype))
        self.w_qkv = make_param(torch.cat(rows, 0))
        self.b_qkv = make_param(torch.cat(brows, 0)) if bias else None
        self.wo = Linear(num_heads * hd, D, bias=bias, device=device, seed=seed + 3000, dtype=dtype, init_std=init_std)
        self.attn_dropout = Dropout(dropout_p) if dropout_p > 0 else None

    # ---- parameters ------------------------------------------------------------------------------
    def own_parameters(self):
        return [self.w_qkv] + ([self.b_qkv] if self.b_qkv is not None else [])

    def own_reference_parameters(self):
        hd = self.head_dim
        out = []
        total = self.num_heads + 2 * self.num_kv_heads
        for h in range(total):
            out.append(self.w_qkv.data[h * hd:(h + 1) * hd])
            if self.b_qkv is not None:
                out.append(self.b_qkv.data[h * hd:(h + 1) * hd].view(1, hd))
        return out

    def submodules(self):
        return [self.wo] + ([self.attn_dropout] if self.attn_dropout is not None else [])

    # Views with the reference's names, for loaders and tests.
    def wq_weight(self, h):
        return self.w_qkv.data[h * self.head_dim:(h + 1) * self.head_dim]

    def wk_weight(self, h):
        o = self.num_heads + h
        return self.w_qkv.data[o * self.head_dim:(o + 1) * self.head_dim]

    def wv_weight(self, h):
        o = self.num_heads + self.num_kv_heads + h
        return self.w_qkv.data[o * self.head_dim:(o + 1) * self.head_dim]

    # ---- forward ---------------------------------------------------------------------------------
    def forward(self, x, mask=None, cache: Optional[MHACache] = None, start_pos: int = 0, causal: bool = False,
                residual=None):
        """``x``: ``[N, D]`` or ``[B, N, D]``.  ``causal=True`` is the kernel-side equivalent of passing
        ``causalMask(N)``; an explicit additive ``mask`` selects the composed (score-matrix) path."""
        if x.dim() not in (2, 3):
            raise ValueError("MultiHeadAttention: input must be [N, D] or [B, N, D]")
        if x.shape[-1] != self.embed_dim:
            raise ValueError(f"MultiHeadAttention: expected last dim {self.embed_dim}, got {x.shape[-1]}")
        if cache is not None and mask is not None and cache.seq_len > 0:
            raise ValueError("MultiHeadAttention: cannot pass mask when appending to a non-empty cache")
        batched = x.dim() == 3
        B = x.shape[0] if batched else 1
        S = x.shape[-2]
        H, Hkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        dq, dkv = H * hd, Hkv * hd
        x2 = x.reshape(B * S, self.embed_dim)
        qkv = F.linear(x2, self.w_qkv, self.b_qkv)  # [B*S, dq + 2 dkv]
        if self.rope is not None:
            self.rope.check_window(start_pos, S)
            qkv = self._rope_qk(qkv, S, start_pos)
        if cache is None and mask is None:
            o = F.attention_packed(qkv, B, S, H, Hkv, hd, causal=causal)
        else:
            q = qkv[:, :dq]
            k_new = qkv[:, dq:dq + dkv].reshape(B, S, dkv)
            v_new = qkv[:, dq + dkv:].reshape(B, S, dkv)
            if cache is not None:
                past = cache.seq_len
                k_all, v_all = cache.append(k_new.detach(), v_new.detach())
                o = self._attend_tokens(q, k_all, v_all, B, S, past + S, causal, past, mask)
            else:
                o = self._attend_tokens(q, k_new, v_new, B, S, S, causal, 0, mask)
        out = self.wo(o, residual=None if residual is None else residual.reshape(B * S, -1))
        if self.attn_dropout is not None:
            out = self.attn_dropout(out)
        return out.reshape(*x.shape[:-1], self.embed_dim)

    def _rope_qk(self, qkv, S, start_pos):
        """Rotate the Q and K column blocks of the fused projection output."""
        H, Hkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        n_rot = (H + Hkv) * hd
        if qkv.is_cuda:
            from ..ops.cuda import RopeColsFn
            return RopeColsFn.apply(qkv, H + Hkv, hd, self.rope.rotary_dim, S, start_pos, self.rope.base)
        rot = F.rope(qkv[:, :n_rot].reshape(-1, S, n_rot), start_pos, self.rope.base, self.rope.rotary_dim, heads=H + Hkv)
        return torch.cat([rot.reshape(-1, n_rot), qkv[:, n_rot:]], dim=1)

    def _attend_tokens(self, q2, k3, v3, B, Sq, Sk, causal, q_offset, mask):
        H, Hkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        if q2.is_cuda and mask is None and q2.dtype == torch.bfloat16 and not q2.requires_grad:
            from ..ops import flash
            if flash.kernel_head_dim(hd) == hd:
                k2 = k3.reshape(-1, k3.shape[-1]) if k3.is_contiguous() else None
                if k2 is not None:
                    o, _ = flash.attn_fwd(q2, k2, v3.reshape(-1, v3.shape[-1]), B, Sq, Sk, H, Hkv, hd, causal,
                                          q_offset=q_offset, need_lse=False)
                    return o
                # cache views: rows of batch b start at b * capacity
                cap = k3.stride(0) // k3.stride(1)
                kf = k3.as_strided((B * cap, k3.shape[-1]), (k3.stride(1), 1))
                vf = v3.as_strided((B * cap, v3.shape[-1]), (v3.stride(1), 1))
                o, _ = flash.attn_fwd(q2, kf, vf, B, Sq, Sk, H, Hkv, hd, causal, q_offset=q_offset, need_lse=False,
                                      kv_batch_rows=cap)
                return o
        if q2.is_cuda and mask is None and q2.dtype == torch.bfloat16:
            from ..ops import flash
            return flash.attention_tokens(q2, k3.reshape(B * Sk, Hkv * hd), v3.reshape(B * Sk, Hkv * hd), B, Sq, Sk, H,
                                          Hkv, hd, causal, q_offset)
        q = q2.reshape(B, Sq, H, hd).transpose(1, 2)
        k = k3.reshape(B, Sk, Hkv, hd).transpose(1, 2)
        v = v3.reshape(B, Sk, Hkv, hd).transpose(1, 2)
        o = F.attention(q, k, v, causal=causal, mask=mask, q_offset=q_offset)
        return o.transpose(1, 2).reshape(B * Sq, H * hd)


class MultiHeadCrossAttention(Module):
    """Queries from ``xq [.., Nq, D]``, keys / values from ``xkv [.., Nk, kvDim]``; no mask, no cache
    (reference: lib/core/nn/attention/multi_head_cross_attention.dart:27-193)."""

    def __init__(self, embed_dim: int, kv_dim: int, num_heads: int, bias: bool = False, device=None, seed: int = 0,
                 dtype=torch.float32, init_std: Optional[float] = None):
        super().__init__()
        if embed_dim % num_heads:
            raise ValueError("MultiHeadCrossAttention: embedDim must be divisible by numHeads")
        self.embed_dim, self.kv_dim, self.num_heads = embed_dim, kv_dim, num_heads
        self.head_dim = embed_dim // num_heads
        hd = self.head_dim

        def rows(in_dim, base):
            bound = 1.0 / math.sqrt(in_dim)
            ws, bs = [], []
            for h in range(num_heads):
                if init_std is None:
                    ws.append(uniform_((hd, in_dim), bound, seed + base + h, device, dtype))
                    bs.append(uniform_((hd,), bound, seed + base + h + 1, device, dtype))
                else:
                    ws.append(normal_((hd, in_dim), init_std, seed + base + h, device, dtype))
                    bs.append(torch.zeros(hd, device=device, dtype=dtype))
            return torch.cat(ws, 0), torch.cat(bs, 0)

        wq, bq = rows(embed_dim, 0)
        wk, bk = rows(kv_dim, 1000)
        wv, bv = rows(kv_dim, 2000)
        self.w_q = make_param(wq)
        self.w_kv = make_param(torch.cat([wk, wv], 0))
        self.b_q = make_param(bq) if bias else None
        self.b_kv = make_param(torch.cat([bk, bv], 0)) if bias else None
        self.wo = Linear(embed_dim, embed_dim, bias=bias, device=device, seed=seed + 3000, dtype=dtype,
                         init_std=init_std)

    def own_parameters(self):
        ps = [self.w_q, self.w_kv]
        if self.b_q is not None:
            ps += [self.b_q, self.b_kv]
        return ps

    def own_reference_parameters(self):
        hd, H = self.head_dim, self.num_heads
        out = []
        for h in range(H):
            out.append(self.w_q.data[h * hd:(h + 1) * hd])
            if self.b_q is not None:
                out.append(self.b_q.data[h * hd:(h + 1) * hd].view(1, hd))
        for h in range(2 * H):
            out.append(self.w_kv.data[h * hd:(h + 1) * hd])
            if self.b_kv is not None:
                out.append(self.b_kv.data[h * hd:(h + 1) * hd].view(1, hd))
        return out

    def submodules(self):
        return [self.wo]

    def forward(self, xq, xkv, residual=None):
        if xq.dim() != xkv.dim() or xq.dim() not in (2, 3):
            raise ValueError("MultiHeadCrossAttention: xq and xkv must both be 2-D or both 3-D")
        if xq.shape[-1] != self.embed_dim or xkv.shape[-1] != self.kv_dim:
            raise ValueError(f"MultiHeadCrossAttention: expected last dims {self.embed_dim} / {self.kv_dim}, got "
                             f"{xq.shape[-1]} / {xkv.shape[-1]}")
        if xq.dim() == 3 and xq.shape[0] != xkv.shape[0]:
            raise ValueError(f"MultiHeadCrossAttention: batch sizes differ ({xq.shape[0]} vs {xkv.shape[0]})")
        batched = xq.dim() == 3
        B = xq.shape[0] if batched else 1
        Sq, Sk = xq.shape[-2], xkv.shape[-2]
        H, hd = self.num_heads, self.head_dim
        q2 = F.linear(xq.reshape(B * Sq, -1), self.w_q, self.b_q)
        kv2 = F.linear(xkv.reshape(B * Sk, -1), self.w_kv, self.b_kv)
        D = H * hd
        if q2.is_cuda and q2.dtype == torch.bfloat16:
            from ..ops import flash
            o = flash.attention_tokens(q2, kv2[:, :D], kv2[:, D:], B, Sq, Sk, H, H, hd, causal=False)
        else:
            q = q2.reshape(B, Sq, H, hd).transpose(1, 2)
            k = kv2[:, :D].reshape(B, Sk, H, hd).transpose(1, 2)
            v = kv2[:, D:].reshape(B, Sk, H, hd).transpose(1, 2)
            o = F.attention(q, k, v, causal=False).transpose(1, 2).reshape(B * Sq, D)
        out = self.wo(o, residual=None if residual is None else residual.reshape(B * Sq, -1))
        return out.reshape(*xq.shape[:-1], self.embed_dim)
