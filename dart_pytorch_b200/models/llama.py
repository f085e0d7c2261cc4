"""Llama-family decoder: RMSNorm, rotary positions, grouped-query attention, SwiGLU feed-forward, no biases
(reference: lib/core/nn/llama.dart:37-424).

The reference model takes one 1-D token sequence; this one also takes ``[B, N]`` batches (prefill and decode of many
prompts at once).  Checkpoint order is the reference's: ``embedIn`` · per block {attnNorm, ffnNorm, wq[0..H), wk[0..Hkv),
wv[0..Hkv), wo, gate, up, down} · finalNorm · (untied head).
"""
from __future__ import annotations

import random as _random
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import ops as F
from ..nn.attention import EncoderCache, MHACache, MultiHeadAttention, RopeCache
from ..nn.layers import Embedding, Linear, RMSNorm, SwiGluFfn
from ..nn.module import Module
from .gpt import _as_token_tensor


@dataclass
class LlamaConfig:
    vocab_size: int
    max_ctx: int
    embed_dim: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    ffn_dim: int
    rope_base: float = 500000.0
    rms_norm_eps: float = 1e-5
    tie_weights: bool = True
    device: object = None
    seed: int = 0
    dtype: torch.dtype = torch.float32
    init_std: Optional[float] = None

    def __post_init__(self):
        if self.embed_dim % self.num_heads:
            raise ValueError("LlamaConfig: embedDim must be divisible by numHeads")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("LlamaConfig: numHeads must be a multiple of numKvHeads")
        if (self.embed_dim // self.num_heads) % 2:
            raise ValueError("LlamaConfig: head dimension must be even for rotary embeddings")

    @property
    def head_dim(self) -> int:
        return self.embed_dim // self.num_heads


class LlamaBlock(Module):
    """``h = x + attn(rms(x))``; ``y = h + swiglu(rms(h))`` (reference: lib/core/nn/llama.dart:80-122)."""

    def __init__(self, c: LlamaConfig, rope: RopeCache, seed: int):
        super().__init__()
        self.attn_norm = RMSNorm(c.embed_dim, eps=c.rms_norm_eps, device=c.device, dtype=c.dtype)
        self.ffn_norm = RMSNorm(c.embed_dim, eps=c.rms_norm_eps, device=c.device, dtype=c.dtype)
        self.attn = MultiHeadAttention(c.embed_dim, c.num_heads, num_kv_heads=c.num_kv_heads, bias=False,
                                       device=c.device, seed=seed, rope=rope, dtype=c.dtype, init_std=c.init_std)
        self.ffn = SwiGluFfn(c.embed_dim, c.ffn_dim, device=c.device, seed=seed + 4000, dtype=c.dtype,
                             init_std=c.init_std)

    def submodules(self):
        return [self.attn_norm, self.ffn_norm, self.attn, self.ffn]

    def forward(self, x, cache: Optional[MHACache] = None, start_pos: int = 0, causal: bool = True):
        xr, y = self.attn_norm.with_residual(x)
        h = self.attn(y, cache=cache, start_pos=start_pos, causal=causal, residual=xr)
        hr, y2 = self.ffn_norm.with_residual(h)
        return self.ffn(y2, residual=hr)


class Llama(Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        c = config
        self.config = c
        self.embed_in = Embedding(c.vocab_size, c.embed_dim, device=c.device, seed=c.seed, dtype=c.dtype,
                                  init_std=c.init_std)
        self.rope = RopeCache(c.max_ctx, c.head_dim, base=c.rope_base)
        self.blocks = [LlamaBlock(c, self.rope, c.seed + 100000 + i * 10000) for i in range(c.num_layers)]
        self.final_norm = RMSNorm(c.embed_dim, eps=c.rms_norm_eps, device=c.device, dtype=c.dtype)
        self.untied_head = None
        if not c.tie_weights:
            self.untied_head = Linear(c.embed_dim, c.vocab_size, bias=False, device=c.device, seed=c.seed + 900000,
                                      dtype=c.dtype, init_std=c.init_std)

    def submodules(self):
        mods = [self.embed_in] + list(self.blocks) + [self.final_norm]
        if self.untied_head is not None:
            mods.append(self.untied_head)
        return mods

    @property
    def head_weight(self):
        return self.embed_in.weight if self.untied_head is None else self.untied_head.weight

    def hidden_from_embeddings(self, h, start_pos: int = 0, cache: Optional[EncoderCache] = None):
        """Run the decoder stack on precomputed input embeddings ``[N, D]`` / ``[B, N, D]``; returns the final-norm
        hidden states."""
        n = h.shape[-2]
        if start_pos + n > self.config.max_ctx:
            raise ValueError(f"Llama: sequence of {start_pos + n} tokens exceeds maxCtx {self.config.max_ctx}")
        if cache is not None and len(cache.layers) != len(self.blocks):
            raise ValueError("Llama: cache has a different number of layers")
        for i, blk in enumerate(self.blocks):
            h = blk(h, cache=None if cache is None else cache.layers[i], start_pos=start_pos, causal=n > 1)
        return self.final_norm(h)

    def forward_from_embeddings(self, h, start_pos: int = 0, cache: Optional[EncoderCache] = None):
        """Logits for precomputed input embeddings (multimodal prefixes mixed with text embeddings): block stack,
        final norm and output head, skipping the token embedding (reference: lib/core/nn/llama.dart:217-236)."""
        if h.dim() not in (2, 3) or h.shape[-1] != self.config.embed_dim:
            raise ValueError(f"Llama.forwardFromEmbeddings: expected [N, {self.config.embed_dim}]; got {list(h.shape)}")
        return F.linear(self.hidden_from_embeddings(h, start_pos, cache), self.head_weight)

    forwardFromEmbeddings = forward_from_embeddings

    def hidden(self, tokens, start_pos: int = 0, cache: Optional[EncoderCache] = None):
        if tokens.dim() not in (1, 2):
            raise ValueError("Llama: tokens must be [N] or [B, N]")
        return self.hidden_from_embeddings(F.embedding(self.embed_in.weight, tokens), start_pos, cache)

    def forward(self, tokens, start_pos: int = 0, cache: Optional[EncoderCache] = None):
        tokens = _as_token_tensor(tokens, self.device)
        return F.linear(self.hidden(tokens, start_pos, cache), self.head_weight)

    def loss(self, tokens, targets):
        tokens = _as_token_tensor(tokens, self.device)
        targets = _as_token_tensor(targets, self.device)
        h = self.hidden(tokens)
        return F.lm_head_loss(h.reshape(-1, h.shape[-1]), self.head_weight, targets.reshape(-1))

    # ---- generation (same sampler and loop as GPT; reference: lib/core/nn/llama.dart:259-408) ----------------
    def new_cache(self, max_len: Optional[int] = None) -> EncoderCache:
        return EncoderCache.empty(self.config.num_layers, self.config.num_kv_heads,
                                  max_len=max_len or self.config.max_ctx)

    def generate(self, prompt: Sequence[float], max_new_tokens: int, temperature: float = 1.0,
                 top_k: Optional[int] = None, rng=None, use_cache: bool = True) -> List[float]:
        from .gpt import GPT
        prompt = list(prompt)
        if not prompt:
            raise ValueError("Llama.generate: prompt must be non-empty")
        if use_cache and len(prompt) > self.config.max_ctx:
            raise ValueError(f"Llama.generate(useCache: true): prompt length {len(prompt)} exceeds maxCtx "
                             f"{self.config.max_ctx}. Pass useCache: false to enable sliding-window truncation.")
        rng = rng or _random.Random()
        was_training = self.training
        self.eval()
        try:
            with torch.no_grad():
                out = [float(t) for t in prompt]
                sample = lambda row: GPT._sample(self, row, temperature, top_k, rng)  # noqa: E731
                if use_cache:
                    cache = self.new_cache()
                    h = self.hidden(_as_token_tensor(prompt, self.device), 0, cache)
                    nxt = sample(F.linear(h[-1:], self.head_weight)[0])
                    out.append(float(nxt))
                    for _ in range(1, max_new_tokens):
                        if cache.seq_len >= self.config.max_ctx:
                            break
                        tok = torch.tensor([nxt], dtype=torch.long, device=self.device)
                        h = self.hidden(tok, cache.seq_len, cache)
                        nxt = sample(F.linear(h, self.head_weight)[0])
                        out.append(float(nxt))
                else:
                    for _ in range(max_new_tokens):
                        ctx = out[-self.config.max_ctx:]
                        h = self.hidden(_as_token_tensor(ctx, self.device))
                        out.append(float(sample(F.linear(h[-1:], self.head_weight)[0])))
                return out
        finally:
            if was_training:
                self.train()

    def generate_batch(self, prompts: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        """Greedy decoding of a ``[B, N]`` batch of equal-length prompts with the device KV cache and device argmax;
        returns ``[B, N + new]`` token ids.  Nothing but the final ids leaves the device."""
        from ..ops import kernels as K
        c = self.config
        was_training = self.training
        self.eval()
        try:
            with torch.no_grad():
                toks = _as_token_tensor(prompts, self.device)
                B, n = toks.shape
                cache = self.new_cache(max_len=min(c.max_ctx, n + max_new_tokens))
                h = self.hidden(toks, 0, cache)
                outs = [toks]
                last = h[:, -1, :]
                for step in range(max_new_tokens):
                    logits = F.linear(last, self.head_weight)
                    if logits.is_cuda:
                        nxt = K.argmax_rows(logits.reshape(B, -1), n_cols=c.vocab_size)
                    else:
                        nxt = logits.argmax(-1)
                    outs.append(nxt.reshape(B, 1))
                    if step + 1 == max_new_tokens or cache.seq_len >= c.max_ctx:
                        break
                    last = self.hidden(nxt.reshape(B, 1), cache.seq_len, cache)[:, -1, :]
                return torch.cat(outs, dim=1)
        finally:
            if was_training:
                self.train()
