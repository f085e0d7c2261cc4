"""Vision transformers: backbone, classifier, face-embedding head, DETR-style detector, CLS feature helper
(reference: lib/core/nn/vision/vit_backbone.dart:21-166, vit_classifier.dart:19-67, vit_face_embedding.dart,
vit_object_detector.dart, vision_encoder.dart).

The reference takes ONE pre-patchified image ``[numPatches, P*P*C]`` and projects patches with a ``Linear``.  That
contract is kept (2-D input), and two inputs are added: a batch of pre-patchified images ``[B, numPatches, P*P*C]`` and
raw images ``[B, C, H, W]``, for which the 16x16 stride-16 patch convolution runs as patch gather (one kernel, ``(dy, dx,
c)`` order) + the tensor-core GEMM against the very same ``[D, P*P*C]`` weight, so checkpoints are interchangeable.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops as F
from ..nn.layers import LayerNorm, Linear
from ..nn.module import Module, make_param, normal_
from ..nn.transformer import Activation, TransformerEncoder


def patchify(images: torch.Tensor, patch: int, out_dtype=None) -> torch.Tensor:
    """``[B, C, H, W]`` -> ``[B, (H/P)*(W/P), P*P*C]`` with per-patch order ``(dy, dx, c)`` and row-major patch order
    (reference order: lib/core/data/image_folder_dataset.dart:180-205)."""
    B, C, H, W = images.shape
    if H % patch or W % patch:
        raise ValueError("patchify: image size must be a multiple of the patch size")
    gh, gw = H // patch, W // patch
    if images.is_cuda:
        from ..ops import kernels as K
        rows = K.patchify(images, patch, out_dtype=out_dtype or images.dtype)
        return rows.view(B, gh * gw, patch * patch * C)
    x = images.reshape(B, C, gh, patch, gw, patch).permute(0, 2, 4, 3, 5, 1)  # B, gy, gx, dy, dx, c
    out = x.reshape(B, gh * gw, patch * patch * C)
    return out.to(out_dtype) if out_dtype is not None else out


class VisionEncoder:
    """Interface of image encoders: ``embed_dim``, ``num_patches`` and a call returning ``[numPatches + 1, D]`` token
    features (reference: lib/core/nn/vision/vision_encoder.dart)."""
    embed_dim: int
    num_patches: int


class ViTBackbone(Module, VisionEncoder):
    def __init__(self, image_size: int = 32, patch_size: int = 8, channels: int = 3, embed_dim: int = 64,
                 num_layers: int = 4, num_heads: int = 4, ffn_dim: Optional[int] = None, dropout_p: float = 0.0,
                 activation=Activation.relu, attn_bias: bool = False, device=None, seed: int = 0,
                 dtype=torch.float32, init_std: Optional[float] = None):
        super().__init__()
        if image_size % patch_size:
            raise ValueError("ViTBackbone: imageSize must be a multiple of patchSize")
        self.image_size, self.patch_size, self.channels = image_size, patch_size, channels
        self.embed_dim = embed_dim
        self.num_patches = (image_size // patch_size) ** 2
        self.patch_dim = patch_size * patch_size * channels
        self.patch_proj = Linear(self.patch_dim, embed_dim, bias=True, device=device, seed=seed, dtype=dtype,
                                 init_std=init_std)
        self.cls_token = make_param(normal_((1, embed_dim), 0.02, seed + 1, device, dtype))
        self.pos_emb = make_param(normal_((self.num_patches + 1, embed_dim), 0.02, seed + 2, device, dtype))
        self.encoder = TransformerEncoder(num_layers, embed_dim, num_heads, ffn_dim=ffn_dim, dropout_p=dropout_p,
                                          attn_bias=attn_bias, activation=activation, final_norm=True, device=device,
                                          seed=seed + 100, dtype=dtype, init_std=init_std)

    def own_parameters(self):
        return [self.cls_token, self.pos_emb]

    def submodules(self):
        return [self.patch_proj, self.encoder]

    def _walk_params(self, reference: bool):
        # reference order: patchProj, cls, pos, encoder
        yield from self.patch_proj._walk_params(reference)
        yield from (self.own_reference_parameters() if reference else self.own_parameters())
        yield from self.encoder._walk_params(reference)

    def forward(self, x):
        """``[numPatches, patchDim]`` (one image), ``[B, numPatches, patchDim]`` or raw ``[B, C, H, W]`` images.
        Returns token features ``[(B,) numPatches + 1, D]`` with the CLS token first."""
        single = x.dim() == 2
        if x.dim() == 4:
            x = patchify(x, self.patch_size, out_dtype=self.patch_proj.weight.dtype)
        if single:
            x = x.unsqueeze(0)
        if x.dim() != 3 or x.shape[1] != self.num_patches or x.shape[2] != self.patch_dim:
            raise ValueError(f"ViTBackbone: expected [{self.num_patches}, {self.patch_dim}] patches, got {tuple(x.shape)}")
        B = x.shape[0]
        tok = self.patch_proj(x)                                   # [B, P, D]
        cls = self.cls_token.to(tok.dtype).expand(B, 1, self.embed_dim)
        h = torch.cat([cls, tok], dim=1)
        h = F.add(h, self.pos_emb.to(h.dtype).expand(B, -1, -1).contiguous())
        h = self.encoder(h)
        return h[0] if single else h


def vit_cls_feature(features: torch.Tensor) -> torch.Tensor:
    """CLS row(s) of backbone features: ``[1, D]`` for one image, ``[B, D]`` for a batch
    (reference: lib/core/nn/vision/vit_backbone.dart ``vitClsFeature``)."""
    return features[:1] if features.dim() == 2 else features[:, 0, :]


vitClsFeature = vit_cls_feature


class ViTClassifier(Module):
    """Backbone + linear head on the CLS token (reference: lib/core/nn/vision/vit_classifier.dart:19-67)."""

    def __init__(self, image_size: int = 32, patch_size: int = 8, channels: int = 3, embed_dim: int = 64,
                 num_layers: int = 4, num_heads: int = 4, num_classes: int = 10, ffn_dim: Optional[int] = None,
                 dropout_p: float = 0.0, activation=Activation.relu, attn_bias: bool = False, device=None, seed: int = 0,
                 dtype=torch.float32, init_std: Optional[float] = None):
        super().__init__()
        self.backbone = ViTBackbone(image_size, patch_size, channels, embed_dim, num_layers, num_heads, ffn_dim,
                                    dropout_p, activation, attn_bias, device, seed, dtype, init_std)
        self.head = Linear(embed_dim, num_classes, device=device, seed=seed + 7000, dtype=dtype, init_std=init_std)
        self.num_classes = num_classes

    def submodules(self):
        return [self.backbone, self.head]

    def forward(self, x):
        return self.head(vit_cls_feature(self.backbone(x)))

    def loss(self, images, labels):
        """Mean cross-entropy of the class logits."""
        logits = self.forward(images)
        return F.mean(F.cross_entropy(logits.reshape(-1, self.num_classes), labels.reshape(-1))).reshape(())


class ViTFaceEmbedding(Module):
    """Backbone + projection + L2 normalisation; ``cosine_similarity`` compares two embeddings
    (reference: lib/core/nn/vision/vit_face_embedding.dart)."""

    def __init__(self, image_size: int = 32, patch_size: int = 8, channels: int = 3, embed_dim: int = 64,
                 num_layers: int = 4, num_heads: int = 4, face_dim: int = 32, device=None, seed: int = 0,
                 dtype=torch.float32):
        super().__init__()
        self.backbone = ViTBackbone(image_size, patch_size, channels, embed_dim, num_layers, num_heads, device=device,
                                    seed=seed, dtype=dtype)
        self.proj = Linear(embed_dim, face_dim, device=device, seed=seed + 7000, dtype=dtype)

    def submodules(self):
        return [self.backbone, self.proj]

    def forward(self, x):
        e = self.proj(vit_cls_feature(self.backbone(x)))
        norm = F.sqrt(F.add(F.sum(F.mul(e, e)), 1e-12)) if e.shape[0] == 1 else None
        if norm is not None:
            return F.div(e, norm.reshape(1))
        n = torch.sqrt((e.float() * e.float()).sum(-1, keepdim=True) + 1e-12).to(e.dtype)
        return e / n

    @staticmethod
    def cosine_similarity(a: torch.Tensor, b: torch.Tensor) -> float:
        a, b = a.reshape(-1).float(), b.reshape(-1).float()
        return float((a * b).sum() / (a.norm() * b.norm() + 1e-12))

    cosineSimilarity = cosine_similarity


class ViTObjectDetector(Module):
    """DETR-style head: ``numQueries`` learned queries read the patch features through one cross-attention step and
    emit class logits (``numClasses + 1`` with a no-object class) and normalised boxes ``(cx, cy, w, h)`` in (0, 1)
    (reference: lib/core/nn/vision/vit_object_detector.dart)."""

    def __init__(self, image_size: int = 32, patch_size: int = 8, channels: int = 3, embed_dim: int = 64,
                 num_layers: int = 4, num_heads: int = 4, num_queries: int = 8, num_classes: int = 4, device=None,
                 seed: int = 0, dtype=torch.float32):
        super().__init__()
        from ..nn.attention import MultiHeadCrossAttention
        self.backbone = ViTBackbone(image_size, patch_size, channels, embed_dim, num_layers, num_heads, device=device,
                                    seed=seed, dtype=dtype)
        self.queries = make_param(normal_((num_queries, embed_dim), 0.02, seed + 8000, device, dtype))
        self.cross = MultiHeadCrossAttention(embed_dim, embed_dim, num_heads, device=device, seed=seed + 8100,
                                             dtype=dtype)
        self.norm = LayerNorm(embed_dim, device=device, dtype=dtype)
        self.class_head = Linear(embed_dim, num_classes + 1, device=device, seed=seed + 8200, dtype=dtype)
        self.box_head = Linear(embed_dim, 4, device=device, seed=seed + 8300, dtype=dtype)
        self.num_queries, self.num_classes = num_queries, num_classes

    def own_parameters(self):
        return [self.queries]

    def submodules(self):
        return [self.backbone, self.cross, self.norm, self.class_head, self.box_head]

    def forward(self, x):
        feats = self.backbone(x)
        if feats.dim() == 2:
            q = self.norm(F.add(self.queries, self.cross(self.queries, feats)))
        else:
            qb = self.queries.unsqueeze(0).expand(feats.shape[0], -1, -1).contiguous()
            q = self.norm(F.add(qb, self.cross(qb, feats)))
        return self.class_head(q), F.sigmoid(self.box_head(q))
