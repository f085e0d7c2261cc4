"""GPT: weight-tied causal language model with learned positions and KV-cache generation
(reference: lib/core/nn/gpt.dart:39-360).

Differences in kind from the reference, not in behaviour: token + position lookup is one kernel, the causal mask is a
flag of the attention kernel (no ``[N, N]`` tensor), the tied head never transposes the table (the GEMM reads it K-major
as stored), ``loss()`` fuses head GEMM + cross-entropy + both gradient GEMMs around one padded logits buffer, and
``generate()`` samples on the device from a cache that is appended in place.
"""
from __future__ import annotations

import random as _random
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import ops as F
from ..nn.attention import EncoderCache
from ..nn.layers import Dropout, Embedding, LearnedPositionalEmbedding, Linear
from ..nn.module import Module
from ..nn.transformer import Activation, TransformerEncoder


@dataclass
class GPTConfig:
    vocab_size: int
    max_ctx: int
    embed_dim: int
    num_layers: int
    num_heads: int
    ffn_dim: Optional[int] = None
    dropout_p: float = 0.0
    tie_weights: bool = True
    attn_bias: bool = False
    activation: object = Activation.relu
    device: object = None
    seed: int = 0
    dtype: torch.dtype = torch.float32
    init_std: Optional[float] = None   # None: the reference's U(+-1/sqrt(in)) / N(0, 1/D) initialisers

    def __post_init__(self):
        if self.vocab_size <= 0 or self.max_ctx <= 0 or self.embed_dim <= 0 or self.num_layers <= 0:
            raise ValueError("GPTConfig: sizes must be positive")
        if self.embed_dim % self.num_heads:
            raise ValueError("GPTConfig: embedDim must be divisible by numHeads")

    # camelCase aliases of the reference's field names
    @property
    def vocabSize(self):
        return self.vocab_size

    @property
    def maxCtx(self):
        return self.max_ctx

    @property
    def embedDim(self):
        return self.embed_dim

    @property
    def numLayers(self):
        return self.num_layers

    @property
    def numHeads(self):
        return self.num_heads


def _as_token_tensor(tokens, device) -> torch.Tensor:
    if isinstance(tokens, torch.Tensor):
        t = tokens
        if t.is_floating_point():
            t = torch.floor(t + 0.5).to(torch.long)
        return t.to(device=device, dtype=torch.long)
    return torch.tensor([int(round(float(v))) for v in tokens], dtype=torch.long, device=device)


class GPT(Module):
    def __init__(self, config: GPTConfig):
        super().__init__()
        c = config
        self.config = c
        # Seeds: tokenEmb seed, posEmb +50000, encoder +100000, head +900000 (reference: gpt.dart:94-121).
        self.token_emb = Embedding(c.vocab_size, c.embed_dim, device=c.device, seed=c.seed, dtype=c.dtype,
                                   init_std=c.init_std)
        self.pos_emb = LearnedPositionalEmbedding(c.max_ctx, c.embed_dim, device=c.device, seed=c.seed + 50000,
                                                  dtype=c.dtype, init_std=c.init_std)
        self.embed_drop = Dropout(c.dropout_p)
        self.encoder = TransformerEncoder(c.num_layers, c.embed_dim, c.num_heads, ffn_dim=c.ffn_dim,
                                          dropout_p=c.dropout_p, attn_bias=c.attn_bias, activation=c.activation,
                                          final_norm=True, device=c.device, seed=c.seed + 100000, dtype=c.dtype,
                                          init_std=c.init_std)
        self.untied_head = None
        if not c.tie_weights:
            self.untied_head = Linear(c.embed_dim, c.vocab_size, bias=False, device=c.device, seed=c.seed + 900000,
                                      dtype=c.dtype, init_std=c.init_std)

    def submodules(self):
        mods = [self.token_emb, self.pos_emb, self.embed_drop, self.encoder]
        if self.untied_head is not None:
            mods.append(self.untied_head)
        return mods

    @property
    def head_weight(self) -> torch.Tensor:
        return self.token_emb.weight if self.untied_head is None else self.untied_head.weight

    # ---- forward ---------------------------------------------------------------------------------
    def hidden(self, tokens: torch.Tensor, start_pos: int = 0, cache: Optional[EncoderCache] = None):
        """Final hidden states ``[N, D]`` / ``[B, N, D]`` for token ids ``[N]`` / ``[B, N]``."""
        if tokens.dim() not in (1, 2):
            raise ValueError("GPT: tokens must be [N] or [B, N]")
        n = tokens.shape[-1]
        if start_pos + n > self.config.max_ctx:
            raise ValueError(f"GPT: sequence of {start_pos + n} tokens exceeds maxCtx {self.config.max_ctx}")
        h = F.embedding(self.token_emb.weight, tokens, pos_table=self.pos_emb.table.weight, pos_start=start_pos)
        h = self.embed_drop(h)
        return self.encoder(h, cache=cache, causal=n > 1, start_pos=start_pos)

    def forward(self, tokens, start_pos: int = 0, cache: Optional[EncoderCache] = None):
        """Logits ``[N, V]`` / ``[B, N, V]``."""
        tokens = _as_token_tensor(tokens, self.device)
        h = self.hidden(tokens, start_pos, cache)
        return F.linear(h, self.head_weight)

    def loss(self, tokens, targets):
        """Mean next-token cross-entropy; equals ``self(tokens).crossEntropy(targets).mean()`` of the reference recipe
        (bin/gpt_train.dart:111-131) without a logits tensor surviving to the backward."""
        tokens = _as_token_tensor(tokens, self.device)
        targets = _as_token_tensor(targets, self.device)
        h = self.hidden(tokens)
        return F.lm_head_loss(h.reshape(-1, h.shape[-1]), self.head_weight, targets.reshape(-1))

    # ---- generation ------------------------------------------------------------------------------
    def generate(self, prompt: Sequence[float], max_new_tokens: int, temperature: float = 1.0,
                 top_k: Optional[int] = None, rng=None, use_cache: bool = True) -> List[float]:
        """Autoregressive sampling; returns prompt + new tokens as floats (the reference's convention).

        Greedy when ``temperature <= 0`` or ``top_k <= 1``; otherwise temperature -> top-k filter -> softmax -> CDF draw
        with one uniform per token from ``rng.random()`` (reference: lib/core/nn/gpt.dart:185-342)."""
        prompt = list(prompt)
        if not prompt:
            raise ValueError("GPT.generate: prompt must be non-empty")
        if use_cache and len(prompt) > self.config.max_ctx:
            raise ValueError(f"GPT.generate(useCache: true): prompt length {len(prompt)} exceeds maxCtx "
                             f"{self.config.max_ctx}. Pass useCache: false to enable sliding-window truncation.")
        rng = rng or _random.Random()
        was_training = self.training
        self.eval()
        try:
            with torch.no_grad():
                if use_cache:
                    return self._generate_cached(prompt, max_new_tokens, temperature, top_k, rng)
                return self._generate_no_cache(prompt, max_new_tokens, temperature, top_k, rng)
        finally:
            if was_training:
                self.train()

    def _sample(self, logits_row: torch.Tensor, temperature, top_k, rng) -> int:
        v = self.config.vocab_size
        greedy = temperature <= 0.0 or (top_k is not None and top_k <= 1)
        if logits_row.is_cuda:
            from ..ops import kernels as K
            row = logits_row.reshape(1, -1)
            if greedy:
                return int(K.argmax_rows(row, n_cols=v).item())
            if top_k is not None and top_k <= 64:
                u = torch.tensor([rng.random()], dtype=torch.float32, device=row.device)
                return int(K.topk_sample(row, u, min(top_k, v), temperature, n_cols=v).item())
        return F.sample_from_logits(logits_row.float().reshape(-1)[:v].cpu(), temperature, top_k, rng)

    def _generate_cached(self, prompt, max_new, temperature, top_k, rng):
        c = self.config
        cache = EncoderCache.empty(c.num_layers, c.num_heads, max_len=c.max_ctx)
        out = [float(t) for t in prompt]
        toks = _as_token_tensor(prompt, self.device)
        h = self.hidden(toks, 0, cache)
        logits = F.linear(h[-1:], self.head_weight)
        nxt = self._sample(logits[0], temperature, top_k, rng)
        out.append(float(nxt))
        for _ in range(1, max_new):
            if cache.seq_len >= c.max_ctx:
                break
            tok = torch.tensor([nxt], dtype=torch.long, device=self.device)
            h = self.hidden(tok, cache.seq_len, cache)
            logits = F.linear(h, self.head_weight)
            nxt = self._sample(logits[0], temperature, top_k, rng)
            out.append(float(nxt))
        return out

    def _generate_no_cache(self, prompt, max_new, temperature, top_k, rng):
        c = self.config
        out = [float(t) for t in prompt]
        for _ in range(max_new):
            ctx = out[-c.max_ctx:]
            h = self.hidden(_as_token_tensor(ctx, self.device))
            logits = F.linear(h[-1:], self.head_weight)
            out.append(float(self._sample(logits[0], temperature, top_k, rng)))
        return out
