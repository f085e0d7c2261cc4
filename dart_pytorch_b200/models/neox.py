"""GPT-J and Pythia (GPT-NeoX) decoders: parallel-residual blocks with partial rotary embeddings
(reference: lib/core/nn/gptj.dart:53-478, lib/core/nn/pythia.dart:38-385).

* GPT-J block: one LayerNorm feeds both branches, ``y = x + attn(ln(x)) + mlp(ln(x))``; attention has no biases, the MLP
  and the ``lm_head`` have; rotary on the first ``rotaryDim`` dims of every head (half-split form: loaders permute
  GPT-J's interleaved rows when they read a checkpoint).
* Pythia block: two LayerNorms, ``y = x + attn(ln1(x)) + mlp(ln2(x))``; every Linear has a bias except the untied
  output embedding; ``rotaryDim = even(floor(headDim * rotaryPct))`` clamped to ``[2, headDim]``.

Both take ``[N]`` or ``[B, N]`` token ids.  GPT-J keeps the reference's per-layer placement API (``layer_devices``,
``embedding_device``, ``lm_head_device``): activations hop between devices at block boundaries.
"""
from __future__ import annotations

import math
import random as _random
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .. import ops as F
from ..nn.attention import EncoderCache, MHACache, MultiHeadAttention, RopeCache
from ..nn.layers import Embedding, LayerNorm, Linear
from ..nn.module import Module
from .gpt import GPT, _as_token_tensor


class CausalLMMixin:
    """Sampling loop shared by the decoder-only families: needs ``self.config.{max_ctx, vocab_size}``,
    ``self.logits(tokens, start_pos, cache)`` and ``self.new_cache()`` (reference: lib/core/nn/gpt.dart:185-342 —
    the other families repeat that loop verbatim)."""

    _name = "Model"

    def generate(self, prompt: Sequence[float], max_new_tokens: int, temperature: float = 1.0,
                 top_k: Optional[int] = None, rng=None, use_cache: bool = True,
                 stop_id: Optional[int] = None) -> List[float]:
        prompt = list(prompt)
        c = self.config
        if not prompt:
            raise ValueError(f"{self._name}.generate: prompt must be non-empty")
        if use_cache and len(prompt) > c.max_ctx:
            raise ValueError(f"{self._name}.generate(useCache: true): prompt length {len(prompt)} exceeds maxCtx "
                             f"{c.max_ctx}. Pass useCache: false to enable sliding-window truncation.")
        rng = rng or _random.Random()
        was_training = self.training
        self.eval()
        try:
            with torch.no_grad():
                out = [float(t) for t in prompt]
                sample = lambda row: GPT._sample(self, row, temperature, top_k, rng)  # noqa: E731
                if use_cache:
                    cache = self.new_cache()
                    logits = self.logits(_as_token_tensor(prompt, self.input_device), 0, cache)
                    nxt = sample(logits[-1])
                    out.append(float(nxt))
                    for _ in range(1, max_new_tokens):
                        if cache.seq_len >= c.max_ctx or (stop_id is not None and nxt == stop_id):
                            break
                        tok = torch.tensor([nxt], dtype=torch.long, device=self.input_device)
                        nxt = sample(self.logits(tok, cache.seq_len, cache)[-1])
                        out.append(float(nxt))
                else:
                    for _ in range(max_new_tokens):
                        ctx = out[-c.max_ctx:]
                        nxt = sample(self.logits(_as_token_tensor(ctx, self.input_device), 0, None)[-1])
                        out.append(float(nxt))
                        if stop_id is not None and nxt == stop_id:
                            break
                return out
        finally:
            if was_training:
                self.train()

    @property
    def input_device(self):
        return self.device


def compute_rotary_dim(head_dim: int, pct: float) -> int:
    """``rotary_pct`` -> even rotary width in ``[2, head_dim]`` (reference: lib/core/nn/pythia.dart:130-142)."""
    if pct <= 0.0:
        raise ValueError(f"rotaryPct ({pct}) must be > 0")
    if pct >= 1.0:
        return head_dim
    r = int(math.floor(head_dim * pct))
    if r % 2:
        r -= 1
    return max(r, 2)


# ---------------------------------------------------------------------------------------------------------
@dataclass
class GPTJConfig:
    vocab_size: int
    max_ctx: int
    embed_dim: int
    num_layers: int
    num_heads: int
    ffn_dim: Optional[int] = None
    rotary_dim: int = 64
    rope_base: float = 10000.0
    device: object = None
    layer_devices: Optional[List[object]] = None
    embedding_device: object = None
    lm_head_device: object = None
    seed: int = 0
    dtype: torch.dtype = torch.float32
    init_std: Optional[float] = None

    def __post_init__(self):
        if self.ffn_dim is None:
            self.ffn_dim = 4 * self.embed_dim
        if self.embed_dim % self.num_heads:
            raise ValueError("GPTJConfig: embedDim must be divisible by numHeads")
        hd = self.embed_dim // self.num_heads
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= hd):
            raise ValueError(f"GPTJConfig: rotaryDim ({self.rotary_dim}) must be even and in (0, headDim={hd}]")
        if self.layer_devices is not None and len(self.layer_devices) != self.num_layers:
            raise ValueError("GPTJConfig: layerDevices length must equal numLayers")

    def device_for_layer(self, i: int):
        return self.layer_devices[i] if self.layer_devices is not None else self.device

    @property
    def embed_device(self):
        return self.embedding_device if self.embedding_device is not None else self.device

    @property
    def lm_device(self):
        return self.lm_head_device if self.lm_head_device is not None else self.device

    @property
    def has_mixed_placement(self) -> bool:
        devs = {str(torch.device(d or "cpu")) for d in
                [self.embed_device, self.lm_device] + [self.device_for_layer(i) for i in range(self.num_layers)]}
        return len(devs) > 1

    deviceForLayer, embedDevice, lmDevice, hasMixedPlacement = (device_for_layer, embed_device, lm_device,
                                                                 has_mixed_placement)


class GPTJBlock(Module):
    """``x + attn(ln(x)) + fc_out(gelu_tanh(fc_in(ln(x))))`` (reference: lib/core/nn/gptj.dart:141-203)."""

    def __init__(self, embed_dim: int, num_heads: int, ffn_dim: Optional[int] = None, rope: Optional[RopeCache] = None,
                 device=None, seed: int = 0, dtype=torch.float32, init_std: Optional[float] = None):
        super().__init__()
        ffn_dim = ffn_dim or 4 * embed_dim
        self.ln = LayerNorm(embed_dim, device=device, dtype=dtype)
        self.attn = MultiHeadAttention(embed_dim, num_heads, bias=False, device=device, seed=seed, rope=rope,
                                       dtype=dtype, init_std=init_std)
        self.ffn1 = Linear(embed_dim, ffn_dim, bias=True, device=device, seed=seed + 10000, dtype=dtype,
                           init_std=init_std)
        self.ffn2 = Linear(ffn_dim, embed_dim, bias=True, device=device, seed=seed + 20000, dtype=dtype,
                           init_std=init_std)

    def submodules(self):
        return [self.ln, self.attn, self.ffn1, self.ffn2]

    def forward(self, x, mask=None, cache: Optional[MHACache] = None, start_pos: int = 0, causal: bool = True):
        h = self.ln(x)
        # both residual adds ride in GEMM epilogues: attn-out adds x, the MLP's second GEMM adds that sum
        a = self.attn(h, mask=mask, cache=cache, start_pos=start_pos, causal=causal and mask is None, residual=x)
        return F.mlp(h, self.ffn1.weight, self.ffn1.bias, self.ffn2.weight, self.ffn2.bias, "gelu_tanh", residual=a)


class GPTJModel(CausalLMMixin, Module):
    _name = "GPTJModel"

    def __init__(self, config: GPTJConfig):
        super().__init__()
        c = config
        self.config = c
        hd = c.embed_dim // c.num_heads
        self.wte = Embedding(c.vocab_size, c.embed_dim, device=c.embed_device, seed=c.seed, dtype=c.dtype,
                             init_std=c.init_std)
        self.rope = RopeCache(c.max_ctx, hd, rotary_dim=c.rotary_dim, base=c.rope_base)
        self.blocks = [GPTJBlock(c.embed_dim, c.num_heads, c.ffn_dim, rope=self.rope, device=c.device_for_layer(i),
                                 seed=c.seed + 100000 + i * 1000, dtype=c.dtype, init_std=c.init_std)
                       for i in range(c.num_layers)]
        self.final_ln = LayerNorm(c.embed_dim, device=c.lm_device, dtype=c.dtype)
        self.lm_head = Linear(c.embed_dim, c.vocab_size, bias=True, device=c.lm_device, seed=c.seed + 900000,
                              dtype=c.dtype, init_std=c.init_std)

    def submodules(self):
        return [self.wte] + list(self.blocks) + [self.final_ln, self.lm_head]

    @property
    def input_device(self):
        return self.wte.weight.device

    def new_cache(self) -> EncoderCache:
        return EncoderCache.empty(self.config.num_layers, self.config.num_heads, max_len=self.config.max_ctx)

    def hidden(self, tokens, start_pos: int = 0, cache: Optional[EncoderCache] = None):
        c = self.config
        if tokens.dim() not in (1, 2):
            raise ValueError(f"GPTJModel: tokens must be [N] or [B, N]; got {list(tokens.shape)}")
        n = tokens.shape[-1]
        if start_pos + n > c.max_ctx:
            raise ValueError(f"GPTJModel: window [{start_pos}, {start_pos + n}) exceeds maxCtx={c.max_ctx}")
        h = F.embedding(self.wte.weight, tokens.to(self.wte.weight.device))
        for i, blk in enumerate(self.blocks):
            dev = blk.ln.gamma.device
            if h.device != dev:
                h = h.to(dev)      # layer-placement hop (reference: lib/core/nn/gptj.dart:294-313)
            h = blk(h, cache=None if cache is None else cache.layers[i], start_pos=start_pos, causal=n > 1)
        if h.device != self.final_ln.gamma.device:
            h = h.to(self.final_ln.gamma.device)
        return self.final_ln(h)

    def logits(self, tokens, start_pos: int = 0, cache: Optional[EncoderCache] = None):
        return self.lm_head(self.hidden(tokens, start_pos, cache))

    def forward(self, tokens):
        return self.logits(_as_token_tensor(tokens, self.input_device))

    def loss(self, tokens, targets):
        logits = self.forward(tokens)
        tgt = _as_token_tensor(targets, logits.device).reshape(-1)
        return F.mean(F.cross_entropy(logits.reshape(-1, logits.shape[-1]), tgt))


# ---------------------------------------------------------------------------------------------------------
@dataclass
class PythiaConfig:
    vocab_size: int
    max_ctx: int
    embed_dim: int
    num_layers: int
    num_heads: int
    ffn_dim: Optional[int] = None
    rope_base: float = 10000.0
    rotary_pct: float = 0.25
    device: object = None
    seed: int = 0
    dtype: torch.dtype = torch.float32
    init_std: Optional[float] = None

    def __post_init__(self):
        if self.ffn_dim is None:
            self.ffn_dim = 4 * self.embed_dim
        if self.embed_dim % self.num_heads:
            raise ValueError("PythiaConfig: embedDim must be divisible by numHeads")


class PythiaBlock(Module):
    """``x + attn(input_ln(x)) + mlp(post_attn_ln(x))`` — both norms read the block input
    (reference: lib/core/nn/pythia.dart:64-128)."""

    def __init__(self, embed_dim: int, num_heads: int, ffn_dim: Optional[int] = None, rope: Optional[RopeCache] = None,
                 device=None, seed: int = 0, dtype=torch.float32, init_std: Optional[float] = None):
        super().__init__()
        ffn_dim = ffn_dim or 4 * embed_dim
        self.input_ln = LayerNorm(embed_dim, device=device, dtype=dtype)
        self.post_attn_ln = LayerNorm(embed_dim, device=device, dtype=dtype)
        self.attn = MultiHeadAttention(embed_dim, num_heads, bias=True, device=device, seed=seed, rope=rope,
                                       dtype=dtype, init_std=init_std)
        self.ffn1 = Linear(embed_dim, ffn_dim, bias=True, device=device, seed=seed + 10000, dtype=dtype,
                           init_std=init_std)
        self.ffn2 = Linear(ffn_dim, embed_dim, bias=True, device=device, seed=seed + 20000, dtype=dtype,
                           init_std=init_std)

    def submodules(self):
        return [self.input_ln, self.post_attn_ln, self.attn, self.ffn1, self.ffn2]

    def forward(self, x, mask=None, cache: Optional[MHACache] = None, start_pos: int = 0, causal: bool = True):
        a = self.attn(self.input_ln(x), mask=mask, cache=cache, start_pos=start_pos,
                      causal=causal and mask is None, residual=x)
        return F.mlp(self.post_attn_ln(x), self.ffn1.weight, self.ffn1.bias, self.ffn2.weight, self.ffn2.bias,
                     "gelu_tanh", residual=a)


class PythiaModel(CausalLMMixin, Module):
    _name = "PythiaModel"

    def __init__(self, config: PythiaConfig):
        super().__init__()
        c = config
        self.config = c
        hd = c.embed_dim // c.num_heads
        self.embed_in = Embedding(c.vocab_size, c.embed_dim, device=c.device, seed=c.seed, dtype=c.dtype,
                                  init_std=c.init_std)
        self.embed_out = Linear(c.embed_dim, c.vocab_size, bias=False, device=c.device, seed=c.seed + 900000,
                                dtype=c.dtype, init_std=c.init_std)
        self.rope = RopeCache(c.max_ctx, hd, rotary_dim=compute_rotary_dim(hd, c.rotary_pct), base=c.rope_base)
        self.blocks = [PythiaBlock(c.embed_dim, c.num_heads, c.ffn_dim, rope=self.rope, device=c.device,
                                   seed=c.seed + 100000 + i * 1000, dtype=c.dtype, init_std=c.init_std)
                       for i in range(c.num_layers)]
        self.final_ln = LayerNorm(c.embed_dim, device=c.device, dtype=c.dtype)

    def submodules(self):
        # checkpoint order: embed_in, blocks, final_ln, embed_out (reference: lib/core/nn/pythia.dart:372-384)
        return [self.embed_in] + list(self.blocks) + [self.final_ln, self.embed_out]

    def new_cache(self) -> EncoderCache:
        return EncoderCache.empty(self.config.num_layers, self.config.num_heads, max_len=self.config.max_ctx)

    def hidden(self, tokens, start_pos: int = 0, cache: Optional[EncoderCache] = None):
        c = self.config
        if tokens.dim() not in (1, 2):
            raise ValueError(f"PythiaModel: tokens must be [N] or [B, N]; got {list(tokens.shape)}")
        n = tokens.shape[-1]
        if start_pos + n > c.max_ctx:
            raise ValueError(f"PythiaModel: window [{start_pos}, {start_pos + n}) exceeds maxCtx={c.max_ctx}")
        h = F.embedding(self.embed_in.weight, tokens)
        for i, blk in enumerate(self.blocks):
            h = blk(h, cache=None if cache is None else cache.layers[i], start_pos=start_pos, causal=n > 1)
        return self.final_ln(h)

    def logits(self, tokens, start_pos: int = 0, cache: Optional[EncoderCache] = None):
        return self.embed_out(self.hidden(tokens, start_pos, cache))

    def forward(self, tokens):
        return self.logits(_as_token_tensor(tokens, self.device))

    def loss(self, tokens, targets):
        tokens = _as_token_tensor(tokens, self.device)
        h = self.hidden(tokens)
        tgt = _as_token_tensor(targets, self.device).reshape(-1)
        return F.lm_head_loss(h.reshape(-1, h.shape[-1]), self.embed_out.weight, tgt)
