"""BERT encoder (post-LN) used as a sentence-embedding backbone (reference: lib/core/nn/bert.dart:21-247).

Token-type embeddings are folded into one learned ``[1, D]`` bias (type id 0 only), positions are a learned table,
attention and feed-forward Linears all carry biases, the activation is tanh-GELU and every sub-layer is followed by a
LayerNorm of ``x + sublayer(x)``.  Takes ``[N]`` (reference contract) or ``[B, N]`` token ids.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops as F
from ..nn.attention import MultiHeadAttention
from ..nn.layers import Embedding, LayerNorm, Linear
from ..nn.module import Module, make_param
from .gpt import _as_token_tensor


@dataclass
class BertConfig:
    vocab_size: int
    max_position_embeddings: int
    embed_dim: int
    num_layers: int
    num_heads: int
    intermediate_size: int
    layer_norm_eps: float = 1e-12
    type_vocab_size: int = 2
    device: object = None
    seed: int = 0
    dtype: torch.dtype = torch.float32


class BertEmbeddings(Module):
    """``LayerNorm(word[tokens] + position[0..N) + token_type_bias)``; parameter order word, position, type bias, LN."""

    def __init__(self, vocab_size: int, max_position_embeddings: int, embed_dim: int, layer_norm_eps: float = 1e-12,
                 device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.embed_dim, self.max_len = embed_dim, max_position_embeddings
        self.word_embeddings = Embedding(vocab_size, embed_dim, device=device, seed=seed + 1, dtype=dtype)
        self.position_embeddings = Embedding(max_position_embeddings, embed_dim, device=device, seed=seed + 2,
                                             dtype=dtype)
        self.token_type_bias = make_param(torch.zeros(1, embed_dim, device=device, dtype=dtype))
        self.layer_norm = LayerNorm(embed_dim, eps=layer_norm_eps, device=device, dtype=dtype)

    def _walk_params(self, reference: bool):
        yield from self.word_embeddings._walk_params(reference)
        yield from self.position_embeddings._walk_params(reference)
        yield self.token_type_bias.data if reference else self.token_type_bias
        yield from self.layer_norm._walk_params(reference)

    def submodules(self):
        return [self.word_embeddings, self.position_embeddings, self.layer_norm]

    def forward(self, tokens):
        if tokens.dim() not in (1, 2):
            raise ValueError(f"BertEmbeddings: expected [seqLen] or [B, seqLen]; got {list(tokens.shape)}")
        s = tokens.shape[-1]
        if s == 0:
            raise ValueError("BertEmbeddings: empty sequence")
        if s > self.max_len:
            raise ValueError(f"BertEmbeddings: seqLen {s} exceeds maxPositionEmbeddings {self.max_len}")
        h = F.embedding(self.word_embeddings.weight, tokens, pos_table=self.position_embeddings.weight, pos_start=0)
        h = F.add(h, self.token_type_bias.reshape(-1))
        return self.layer_norm(h)


class BertLayer(Module):
    def __init__(self, embed_dim: int, num_heads: int, intermediate_size: int, layer_norm_eps: float = 1e-12,
                 device=None, seed: int = 0, dtype=torch.float32):
        super().__init__()
        self.attention = MultiHeadAttention(embed_dim, num_heads, bias=True, device=device, seed=seed, dtype=dtype)
        self.attention_output_ln = LayerNorm(embed_dim, eps=layer_norm_eps, device=device, dtype=dtype)
        self.intermediate = Linear(embed_dim, intermediate_size, device=device, seed=seed + 4000, dtype=dtype)
        self.output = Linear(intermediate_size, embed_dim, device=device, seed=seed + 5000, dtype=dtype)
        self.output_ln = LayerNorm(embed_dim, eps=layer_norm_eps, device=device, dtype=dtype)

    def submodules(self):
        return [self.attention, self.attention_output_ln, self.intermediate, self.output, self.output_ln]

    def forward(self, x):
        h = self.attention_output_ln(self.attention(x, residual=x))       # LN(x + attn(x)); add fused in wo's epilogue
        ff = F.mlp(h, self.intermediate.weight, self.intermediate.bias, self.output.weight, self.output.bias,
                   "gelu_tanh", residual=h)
        return self.output_ln(ff)


class BertModel(Module):
    """Token features ``[N, D]`` / ``[B, N, D]``; satisfies the ``TokenEncoder`` protocol (``embed_dim`` + call)."""

    def __init__(self, config: BertConfig):
        super().__init__()
        c = config
        self.config = c
        self.embeddings = BertEmbeddings(c.vocab_size, c.max_position_embeddings, c.embed_dim, c.layer_norm_eps,
                                         device=c.device, seed=c.seed, dtype=c.dtype)
        self.layers = [BertLayer(c.embed_dim, c.num_heads, c.intermediate_size, c.layer_norm_eps, device=c.device,
                                 seed=c.seed + 100 + i * 10000, dtype=c.dtype) for i in range(c.num_layers)]

    @property
    def embed_dim(self) -> int:
        return self.config.embed_dim

    embedDim = embed_dim

    def submodules(self):
        return [self.embeddings] + list(self.layers)

    def forward(self, tokens):
        h = self.embeddings(_as_token_tensor(tokens, self.device))
        for layer in self.layers:
            h = layer(h)
        return h
