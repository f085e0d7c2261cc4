"""CLIP vision tower and the LLaVA-style ``LlamaVision`` wrapper
(reference: lib/core/nn/vision/clip_vision_model.dart:61-190, lib/core/nn/llama_vision.dart:37-248).

``CLIPVisionModel``: bias-free patch projection (the HF conv weight permuted to ``(o, dy, dx, c)`` acts as a Linear),
CLS token, learned positions, a pre-LayerNorm, then a pre-LN encoder with attention biases and QuickGELU whose final
LayerNorm is CLIP's ``post_layernorm``.  Input: one pre-patchified image ``[numPatches, P*P*C]``, a batch of those, or
raw ``[B, C, H, W]`` images (patch gather kernel + the same GEMM).

``LlamaVision``: image tokens ``projector(vit(image))`` are prepended to the text embeddings and the packed sequence
runs through ``llama.forward_from_embeddings``; generation is cache-less with a sliding text window and a stop id.
"""
from __future__ import annotations

import random as _random
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import ops as F
from ..nn.layers import LayerNorm, Linear, VisionProjector
from ..nn.module import Module, make_param, normal_
from ..nn.transformer import Activation, TransformerEncoder
from .gpt import GPT, _as_token_tensor
from .llama import Llama
from .vit import VisionEncoder, patchify


@dataclass
class CLIPVisionConfig:
    image_size: int = 224
    patch_size: int = 32
    num_channels: int = 3
    embed_dim: int = 768
    num_layers: int = 12
    num_heads: int = 12
    ffn_dim: int = 3072
    layer_norm_eps: float = 1e-5
    device: object = None
    seed: int = 0
    dtype: torch.dtype = torch.float32

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2

    @property
    def patch_pixels(self) -> int:
        return self.patch_size * self.patch_size * self.num_channels

    numPatches, patchPixels = num_patches, patch_pixels


class CLIPVisionModel(Module, VisionEncoder):
    def __init__(self, config: Optional[CLIPVisionConfig] = None):
        super().__init__()
        c = config or CLIPVisionConfig()
        self.config = c
        self.embed_dim, self.num_patches = c.embed_dim, c.num_patches
        self.patch_projection = Linear(c.patch_pixels, c.embed_dim, bias=False, device=c.device, seed=c.seed + 1,
                                       dtype=c.dtype)
        self.cls_token = make_param(normal_((1, c.embed_dim), 0.02, c.seed + 2, c.device, c.dtype))
        self.pos_embeddings = make_param(normal_((c.num_patches + 1, c.embed_dim), 0.02, c.seed + 3, c.device, c.dtype))
        self.pre_layer_norm = LayerNorm(c.embed_dim, eps=c.layer_norm_eps, device=c.device, dtype=c.dtype)
        self.encoder = TransformerEncoder(c.num_layers, c.embed_dim, c.num_heads, ffn_dim=c.ffn_dim, final_norm=True,
                                          attn_bias=True, activation=Activation.quickGelu, device=c.device,
                                          seed=c.seed + 100, dtype=c.dtype)

    def submodules(self):
        return [self.patch_projection, self.pre_layer_norm, self.encoder]

    def _walk_params(self, reference: bool):
        # order: patch projection, cls, positions, pre-LN, encoder
        yield from self.patch_projection._walk_params(reference)
        yield self.cls_token.data if reference else self.cls_token
        yield self.pos_embeddings.data if reference else self.pos_embeddings
        yield from self.pre_layer_norm._walk_params(reference)
        yield from self.encoder._walk_params(reference)

    def forward(self, x):
        c = self.config
        single = x.dim() == 2
        if x.dim() == 4:
            x = patchify(x, c.patch_size, out_dtype=self.patch_projection.weight.dtype)
        if single:
            x = x.unsqueeze(0)
        if x.dim() != 3 or x.shape[1] != c.num_patches or x.shape[2] != c.patch_pixels:
            raise ValueError(f"CLIPVisionModel: expected input [{c.num_patches}, {c.patch_pixels}]; "
                             f"got {list(x.shape[1:] if single else x.shape)}")
        B = x.shape[0]
        tok = self.patch_projection(x)
        h = torch.cat([self.cls_token.to(tok.dtype).expand(B, 1, c.embed_dim), tok], dim=1)
        h = F.add(h, self.pos_embeddings.to(h.dtype).expand(B, -1, -1).contiguous())
        h = self.encoder(self.pre_layer_norm(h))
        return h[0] if single else h


class LlamaVision(Module):
    def __init__(self, vit, projector: VisionProjector, llama: Llama):
        super().__init__()
        if projector.out_dim != llama.config.embed_dim:
            raise ValueError(f"projector.outDim ({projector.out_dim}) must equal llama.config.embedDim "
                             f"({llama.config.embed_dim})")
        if projector.in_dim != vit.embed_dim:
            raise ValueError(f"projector.inDim ({projector.in_dim}) must equal vit.embedDim ({vit.embed_dim})")
        self.vit, self.projector, self.llama = vit, projector, llama

    @classmethod
    def build(cls, vit, llama: Llama, projector_hidden_dim: Optional[int] = None, seed: int = 0) -> "LlamaVision":
        proj = VisionProjector(vit.embed_dim, llama.config.embed_dim, hidden=projector_hidden_dim,
                               device=llama.device, seed=seed, dtype=llama.dtype)
        return cls(vit, proj, llama)

    @property
    def num_image_tokens(self) -> int:
        return self.vit.num_patches + 1

    numImageTokens = num_image_tokens

    def submodules(self):
        return [self.vit, self.projector, self.llama]

    def encode_image(self, patchified_image):
        return self.projector(self.vit(patchified_image))

    encodeImage = encode_image

    def _packed(self, image_tokens, text_tokens):
        text_emb = self.llama.embed_in(text_tokens)
        full = F.concat([image_tokens.to(text_emb.dtype), text_emb], axis=0)
        if full.shape[0] > self.llama.config.max_ctx:
            raise ValueError(f"LlamaVision: total sequence length {full.shape[0]} exceeds "
                             f"llama.maxCtx={self.llama.config.max_ctx}")
        return full

    def forward(self, patchified_image, text_tokens):
        text_tokens = _as_token_tensor(text_tokens, self.llama.device)
        if text_tokens.dim() != 1:
            raise ValueError(f"LlamaVision: textTokens must be 1D [T]; got {list(text_tokens.shape)}")
        return self.llama.forward_from_embeddings(self._packed(self.encode_image(patchified_image), text_tokens))

    def loss(self, patchified_image, text_tokens, targets):
        """Mean next-token loss over the text positions only (image positions carry no target)."""
        logits = self.forward(patchified_image, text_tokens)
        t = _as_token_tensor(targets, logits.device).reshape(-1)
        text_logits = logits[self.num_image_tokens:]
        return F.mean(F.cross_entropy(text_logits, t))

    def generate(self, patchified_image, text_prompt: Sequence[float], max_new_tokens: int, temperature: float = 1.0,
                 top_k: Optional[int] = None, rng=None, stop_id: Optional[int] = None) -> List[float]:
        prompt = list(text_prompt)
        if not prompt:
            raise ValueError("LlamaVision.generate: prompt must be non-empty")
        rng = rng or _random.Random()
        was_training = self.training
        self.eval()
        try:
            with torch.no_grad():
                image_tokens = self.encode_image(patchified_image)
                num_img = image_tokens.shape[0]
                out = [float(t) for t in prompt]
                for _ in range(max_new_tokens):
                    max_text = self.llama.config.max_ctx - num_img
                    if max_text <= 0:
                        break
                    ctx = _as_token_tensor(out[-max_text:], self.llama.device)
                    logits = self.llama.forward_from_embeddings(self._packed(image_tokens, ctx))
                    nxt = GPT._sample(self.llama, logits[-1], temperature, top_k, rng)
                    out.append(float(nxt))
                    if stop_id is not None and nxt == stop_id:
                        break
                return out
        finally:
            if was_training:
                self.train()
