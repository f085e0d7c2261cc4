"""Mixture-of-experts causal language model (reference: lib/core/nn/moe_transformer.dart:27-221).

Reference defaults are kept: LayerNorm, sinusoidal positions, multi-head attention, an ``MoEFeedForward`` in every
block, a biased untied head, 4 routed + 1 shared expert with top-2 routing.  Options cover the expert-parallel
benchmark configuration: ``norm="rms"``, ``rope_base`` (rotary positions instead of sinusoidal), bias-free SwiGLU
experts, ``capacity_factor`` and a load-balance auxiliary loss that ``loss()`` adds to the cross-entropy.
Tokens may be ``[N]`` (the reference contract) or ``[B, N]``.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops as F
from ..nn.attention import MultiHeadAttention, RopeCache
from ..nn.layers import Dropout, Embedding, LayerNorm, Linear, RMSNorm, SinusoidalPositionalEncoding
from ..nn.module import Module
from ..nn.moe import (BiasUpdateRule, ExpertActivation, ExpertVariant, GateFunction, MoEFeedForward)
from .gpt import _as_token_tensor


class MoEBlock(Module):
    """``h = x + drop(attn(norm1(x)))``; ``y = h + drop(moe(norm2(h)))``; parameter order norm1, norm2, attn, moe."""

    def __init__(self, embed_dim: int, num_heads: int, num_routed_experts: int, num_shared_experts: int, top_k: int,
                 expert_hidden_dim: int, dropout_p: float = 0.0, device=None, seed: int = 0, norm: str = "layer",
                 rope: Optional[RopeCache] = None, dtype=torch.float32, init_std: Optional[float] = None,
                 ep_group=None, **moe_kw):
        super().__init__()
        mk_norm = (lambda: RMSNorm(embed_dim, device=device, dtype=dtype)) if norm == "rms" else \
            (lambda: LayerNorm(embed_dim, device=device, dtype=dtype))
        self.ln1, self.ln2 = mk_norm(), mk_norm()
        self.attn = MultiHeadAttention(embed_dim, num_heads, dropout_p=dropout_p, device=device, seed=seed, rope=rope,
                                       dtype=dtype, init_std=init_std)
        if ep_group is not None:
            # experts sharded over the ranks of `ep_group`: SwiGLU experts, softmax top-k, per-source capacity quota
            from ..parallel.ep import ExpertParallelMoE
            self.moe = ExpertParallelMoE(embed_dim, expert_hidden_dim, num_routed_experts, top_k=top_k,
                                         capacity_factor=moe_kw.get("capacity_factor") or 1.25,
                                         aux_loss_coef=moe_kw.get("aux_loss_coef", 0.0), group=ep_group,
                                         renormalize_top_k=bool(moe_kw.get("renormalize_top_k")),
                                         route_scale=moe_kw.get("route_scale", 1.0), device=device, seed=seed + 4000,
                                         dtype=dtype, init_std=init_std)
        else:
            self.moe = MoEFeedForward(embed_dim, num_routed_experts, num_shared_experts, top_k, expert_hidden_dim,
                                      device=device, seed=seed + 4000, dtype=dtype, init_std=init_std, **moe_kw)
        self.dropout = Dropout(dropout_p)

    def submodules(self):
        return [self.ln1, self.ln2, self.attn, self.moe, self.dropout]

    def forward(self, x, mask=None, causal: bool = False):
        h = F.add(x, self.dropout(self.attn(self.ln1(x), mask=mask, causal=causal)))
        y = self.ln2(h)
        flat = y.reshape(-1, y.shape[-1])
        return F.add(h, self.dropout(self.moe(flat).reshape(y.shape)))


class MoELanguageModel(Module):
    def __init__(self, vocab_size: int, embed_dim: int, num_layers: int, num_heads: int, max_len: int,
                 num_routed_experts: int = 4, num_shared_experts: int = 1, top_k: int = 2,
                 expert_hidden_dim: Optional[int] = None, bias_update_rate: float = 0.001, dropout_p: float = 0.0,
                 device=None, seed: int = 0, activation=ExpertActivation.relu, expert_variant=ExpertVariant.mlp,
                 gate_function=GateFunction.softmax, bias_update_rule=BiasUpdateRule.sign, num_expert_groups: int = 1,
                 top_k_groups: Optional[int] = None, route_scale: float = 1.0, sparse_execution: bool = False,
                 renormalize_top_k: Optional[bool] = None, norm: str = "layer", rope_base: Optional[float] = None,
                 capacity_factor: Optional[float] = None, aux_loss_coef: float = 0.0, expert_bias: bool = True,
                 head_bias: bool = True, dtype=torch.float32, init_std: Optional[float] = None, ep_group=None):
        super().__init__()
        self.ep_group = ep_group
        self.vocab_size, self.embed_dim, self.num_layers, self.num_heads = vocab_size, embed_dim, num_layers, num_heads
        self.max_len = max_len
        self.token_emb = Embedding(vocab_size, embed_dim, device=device, seed=seed, dtype=dtype, init_std=init_std)
        self.rope = RopeCache(max_len, embed_dim // num_heads, base=rope_base) if rope_base else None
        self.pos_enc = None if self.rope is not None else SinusoidalPositionalEncoding(embed_dim)
        hidden = expert_hidden_dim or embed_dim * 4
        self.blocks: List[MoEBlock] = [
            MoEBlock(embed_dim, num_heads, num_routed_experts, num_shared_experts, top_k, hidden, dropout_p=dropout_p,
                     device=device, seed=seed + 100000 + i * 10000, norm=norm, rope=self.rope, dtype=dtype,
                     init_std=init_std, bias_update_rate=bias_update_rate, activation=activation,
                     expert_variant=expert_variant, gate_function=gate_function, bias_update_rule=bias_update_rule,
                     num_expert_groups=num_expert_groups, top_k_groups=top_k_groups, route_scale=route_scale,
                     sparse_execution=sparse_execution, renormalize_top_k=renormalize_top_k,
                     capacity_factor=capacity_factor, aux_loss_coef=aux_loss_coef, expert_bias=expert_bias,
                     ep_group=ep_group)
            for i in range(num_layers)]
        self.final_ln = RMSNorm(embed_dim, device=device, dtype=dtype) if norm == "rms" else \
            LayerNorm(embed_dim, device=device, dtype=dtype)
        self.head = Linear(embed_dim, vocab_size, bias=head_bias, device=device, seed=seed + 900000, dtype=dtype,
                           init_std=init_std)

    def submodules(self):
        return [self.token_emb] + list(self.blocks) + [self.final_ln, self.head]

    def hidden(self, tokens):
        if tokens.dim() not in (1, 2):
            raise ValueError(f"MoELanguageModel: tokens must be 1D [seqLen] or [B, seqLen]; got {list(tokens.shape)}")
        n = tokens.shape[-1]
        if n > self.max_len:
            raise ValueError(f"MoELanguageModel: seqLen {n} exceeds maxLen {self.max_len}")
        x = F.embedding(self.token_emb.weight, tokens)
        if self.pos_enc is not None:
            x = self.pos_enc(x)
        for b in self.blocks:
            x = b(x, causal=n > 1)
        return self.final_ln(x)

    def forward(self, tokens):
        return self.head(self.hidden(_as_token_tensor(tokens, self.device)))

    def aux_loss(self):
        """Sum of the blocks' load-balance terms of the last forward (None when the option is off)."""
        terms = [b.moe.last_aux_loss for b in self.blocks if b.moe.last_aux_loss is not None]
        if not terms:
            return None
        total = terms[0]
        for t in terms[1:]:
            total = total + t
        return total

    def loss(self, tokens, targets):
        tokens = _as_token_tensor(tokens, self.device)
        targets = _as_token_tensor(targets, self.device)
        logits = self.head(self.hidden(tokens))
        ce = F.mean(F.cross_entropy(logits.reshape(-1, self.vocab_size), targets.reshape(-1))).reshape(())
        aux = self.aux_loss()
        return ce if aux is None else ce + aux.to(ce.dtype)

    def expert_parameters(self):
        """Parameters that live on one rank only (expert-parallel shards); data-parallel reduction must skip them."""
        out = []
        for b in self.blocks:
            if hasattr(b.moe, "expert_parameters"):
                out.extend(b.moe.expert_parameters())
        return out

    def update_routing_bias(self) -> None:
        for b in self.blocks:
            b.moe.update_routing_bias()

    updateRoutingBias = update_routing_bias
