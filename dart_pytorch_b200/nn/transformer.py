"""Pre-LN transformer blocks, encoder and decoder stacks.

(reference: lib/core/nn/transformer.dart:32-122, transformer_encoder.dart:15-76, transformer_decoder_block.dart:26-115,
transformer_decoder.dart:19-74).  A block forward on the device is seven kernels: LN, QKV GEMM, attention, output
GEMM (+bias +residual), LN, FFN GEMM (+bias +activation), FFN GEMM (+bias +residual).
"""
from __future__ import annotations

from enum import Enum
from typing import List, Optional

import torch

from .. import ops as F
from .attention import EncoderCache, MHACache, MultiHeadAttention, MultiHeadCrossAttention, RopeCache
from .layers import Dropout, LayerNorm, Linear, activation_name
from .module import Module


class Activation(str, Enum):
    relu = "relu"
    geluTanh = "geluTanh"
    quickGelu = "quickGelu"


class TransformerBlock(Module):
    """``h = x + drop(mha(ln1(x)))``, ``y = h + drop(ffn2(act(ffn1(ln2(h)))))``; parameter order ln1, ln2, mha, ffn1, ffn2."""

    def __init__(self, embed_dim: int, num_heads: int, ffn_dim: Optional[int] = None, dropout_p: float = 0.0,
                 attn_bias: bool = False, activation=Activation.relu, device=None, seed: int = 0,
                 num_kv_heads: Optional[int] = None, rope: Optional[RopeCache] = None, dtype=torch.float32,
                 init_std: Optional[float] = None):
        super().__init__()
        self.embed_dim, self.num_heads = embed_dim, num_heads
        self.ffn_dim = ffn_dim or embed_dim * 4
        self.activation = activation
        self.ln1 = LayerNorm(embed_dim, device=device, dtype=dtype)
        self.ln2 = LayerNorm(embed_dim, device=device, dtype=dtype)
        self.mha = MultiHeadAttention(embed_dim, num_heads, num_kv_heads=num_kv_heads, bias=attn_bias,
                                      dropout_p=dropout_p, device=device, seed=seed, rope=rope, dtype=dtype,
                                      init_std=init_std)
        self.ffn1 = Linear(embed_dim, self.ffn_dim, device=device, seed=seed + 4000, dtype=dtype, init_std=init_std)
        self.ffn2 = Linear(self.ffn_dim, embed_dim, device=device, seed=seed + 5000, dtype=dtype, init_std=init_std)
        self.dropout = Dropout(dropout_p)

    def submodules(self):
        return [self.ln1, self.ln2, self.mha, self.ffn1, self.ffn2, self.dropout]

    def forward(self, x, mask=None, cache: Optional[MHACache] = None, causal: bool = False, start_pos: int = 0):
        act = activation_name(self.activation)
        fuse = not (self.training and self.dropout.p > 0)
        if fuse:
            # Residual adds ride in the GEMM epilogues; residual gradients are added inside the norm backward.
            xr, y = self.ln1.with_residual(x)
            h = self.mha(y, mask=mask, cache=cache, causal=causal, start_pos=start_pos, residual=xr)
            hr, y2 = self.ln2.with_residual(h)
            return F.mlp(y2, self.ffn1.weight, self.ffn1.bias, self.ffn2.weight, self.ffn2.bias, act, residual=hr)
        h = F.add(x, self.dropout(self.mha(self.ln1(x), mask=mask, cache=cache, causal=causal, start_pos=start_pos)))
        ff = self.ffn2(self.ffn1(self.ln2(h), activation=act))
        return F.add(h, self.dropout(ff))


class TransformerEncoder(Module):
    """Stack of blocks (block ``i`` seeded ``seed + i*10000``) with an optional final LayerNorm."""

    def __init__(self, num_layers: int, embed_dim: int, num_heads: int, ffn_dim: Optional[int] = None,
                 dropout_p: float = 0.0, attn_bias: bool = False, activation=Activation.relu, final_norm: bool = True,
                 device=None, seed: int = 0, num_kv_heads: Optional[int] = None, rope: Optional[RopeCache] = None,
                 dtype=torch.float32, init_std: Optional[float] = None):
        super().__init__()
        self.blocks: List[TransformerBlock] = [
            TransformerBlock(embed_dim, num_heads, ffn_dim=ffn_dim, dropout_p=dropout_p, attn_bias=attn_bias,
                             activation=activation, device=device, seed=seed + i * 10000, num_kv_heads=num_kv_heads,
                             rope=rope, dtype=dtype, init_std=init_std)
            for i in range(num_layers)]
        self.final_norm = LayerNorm(embed_dim, device=device, dtype=dtype) if final_norm else None

    def submodules(self):
        return list(self.blocks) + ([self.final_norm] if self.final_norm is not None else [])

    def forward(self, x, mask=None, cache: Optional[EncoderCache] = None, causal: bool = False, start_pos: int = 0):
        if cache is not None and len(cache.layers) != len(self.blocks):
            raise ValueError("TransformerEncoder: cache has a different number of layers")
        for i, blk in enumerate(self.blocks):
            x = blk(x, mask=mask, cache=None if cache is None else cache.layers[i], causal=causal, start_pos=start_pos)
        return self.final_norm(x) if self.final_norm is not None else x


class TransformerDecoderBlock(Module):
    """Causal self-attention, cross-attention over the encoder memory, ReLU FFN; three pre-LNs."""

    def __init__(self, embed_dim: int, num_heads: int, ffn_dim: Optional[int] = None, dropout_p: float = 0.0,
                 memory_dim: Optional[int] = None, device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.ffn_dim = ffn_dim or embed_dim * 4
        self.ln1 = LayerNorm(embed_dim, device=device, dtype=dtype)
        self.ln2 = LayerNorm(embed_dim, device=device, dtype=dtype)
        self.ln3 = LayerNorm(embed_dim, device=device, dtype=dtype)
        self.self_attn = MultiHeadAttention(embed_dim, num_heads, dropout_p=dropout_p, device=device, seed=seed,
                                            dtype=dtype)
        self.cross_attn = MultiHeadCrossAttention(embed_dim, memory_dim or embed_dim, num_heads, device=device,
                                                  seed=seed + 6000, dtype=dtype)
        self.ffn1 = Linear(embed_dim, self.ffn_dim, device=device, seed=seed + 4000, dtype=dtype)
        self.ffn2 = Linear(self.ffn_dim, embed_dim, device=device, seed=seed + 5000, dtype=dtype)
        self.dropout = Dropout(dropout_p)

    def submodules(self):
        return [self.ln1, self.ln2, self.ln3, self.self_attn, self.cross_attn, self.ffn1, self.ffn2, self.dropout]

    def forward(self, x, memory, mask=None, causal: bool = True):
        h = F.add(x, self.dropout(self.self_attn(self.ln1(x), mask=mask, causal=causal and mask is None)))
        h = F.add(h, self.dropout(self.cross_attn(self.ln2(h), memory)))
        ff = self.ffn2(self.ffn1(self.ln3(h), activation="relu"))
        return F.add(h, self.dropout(ff))


class TransformerDecoder(Module):
    def __init__(self, num_layers: int, embed_dim: int, num_heads: int, ffn_dim: Optional[int] = None,
                 dropout_p: float = 0.0, memory_dim: Optional[int] = None, final_norm: bool = True, device=None,
                 seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.blocks = [TransformerDecoderBlock(embed_dim, num_heads, ffn_dim=ffn_dim, dropout_p=dropout_p,
                                               memory_dim=memory_dim, device=device, seed=seed + i * 10000, dtype=dtype)
                       for i in range(num_layers)]
        self.final_norm = LayerNorm(embed_dim, device=device, dtype=dtype) if final_norm else None

    def submodules(self):
        return list(self.blocks) + ([self.final_norm] if self.final_norm is not None else [])

    def forward(self, x, memory, mask=None, causal: bool = True):
        for blk in self.blocks:
            x = blk(x, memory, mask=mask, causal=causal)
        return self.final_norm(x) if self.final_norm is not None else x
