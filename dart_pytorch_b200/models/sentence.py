"""Sentence embeddings: bi-encoder, cross-encoder, similarity search and contrastive losses
(reference: lib/core/nn/sentence/sentence_encoder.dart, cross_encoder.dart, similarity.dart, losses.dart).

A *token encoder* is any module with ``embed_dim`` whose call maps ``[N]`` token ids to ``[N, D]`` features
(``TextTransformer``, ``BertModel``).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import List, Optional, Sequence

import torch

from .. import ops as F
from ..nn.layers import Linear
from ..nn.module import Module
from .modalities import TextTransformer, mean_rows


class PoolingMode(str, Enum):
    mean = "mean"
    cls = "cls"


class TokenEncoder:
    """Protocol marker: ``embed_dim`` attribute and ``__call__(tokens [N]) -> [N, D]``."""


def pool_tokens(token_features, mode: PoolingMode = PoolingMode.mean):
    if token_features.dim() != 2:
        raise ValueError(f"poolTokens: expected [seqLen, D]; got {list(token_features.shape)}")
    if token_features.shape[0] == 0:
        raise ValueError("poolTokens: cannot pool empty sequence")
    if PoolingMode(mode) == PoolingMode.mean:
        return mean_rows(token_features)
    return token_features[0:1]


def l2_normalize_row(x, eps: float = 1e-12):
    """``x / sqrt(sum(x^2) + eps)`` for one ``[1, D]`` row."""
    if x.dim() != 2 or x.shape[0] != 1:
        raise ValueError(f"l2NormalizeRow: expected [1, D]; got {list(x.shape)}")
    norm = F.pow(F.add(F.sum(F.mul(x, x)), eps), 0.5)
    return F.div(x, norm.reshape(1))


poolTokens, l2NormalizeRow = pool_tokens, l2_normalize_row


class SentenceEncoder(Module):
    """Token encoder -> pooling -> optional L2 normalisation; one ``[1, D]`` embedding per sequence."""

    def __init__(self, vocab_size: Optional[int] = None, max_seq_len: Optional[int] = None,
                 embed_dim: Optional[int] = None, num_layers: int = 4, num_heads: int = 4, dropout_p: float = 0.0,
                 pooling: PoolingMode = PoolingMode.mean, normalize: bool = True, eps: float = 1e-12, device=None,
                 seed: int = 0, backbone=None):
        super().__init__()
        self.backbone = backbone if backbone is not None else TextTransformer(
            vocab_size, max_seq_len, embed_dim, num_layers=num_layers, num_heads=num_heads, dropout_p=dropout_p,
            device=device, seed=seed)
        self.pooling, self.normalize, self.eps = PoolingMode(pooling), normalize, eps

    @classmethod
    def wrap(cls, backbone, pooling: PoolingMode = PoolingMode.mean, normalize: bool = True, eps: float = 1e-12):
        return cls(backbone=backbone, pooling=pooling, normalize=normalize, eps=eps)

    @property
    def embed_dim(self) -> int:
        return self.backbone.embed_dim

    embedDim = embed_dim

    def submodules(self):
        return [self.backbone]

    def forward(self, tokens):
        pooled = pool_tokens(self.backbone(tokens), self.pooling)
        return l2_normalize_row(pooled, self.eps) if self.normalize else pooled

    def encode_batch(self, token_sequences: Sequence):
        if len(token_sequences) == 0:
            raise ValueError("encodeBatch: input list is empty")
        return F.concat([self.forward(t) for t in token_sequences], axis=0)

    encodeBatch = encode_batch


class CrossEncoder(Module):
    """Scores a packed ``[CLS] a [SEP] b [SEP]`` pair: backbone -> pooled row -> ``Linear(D, numLabels)``."""

    def __init__(self, vocab_size: Optional[int] = None, max_seq_len: Optional[int] = None,
                 embed_dim: Optional[int] = None, num_layers: int = 4, num_heads: int = 4, dropout_p: float = 0.0,
                 pooling: PoolingMode = PoolingMode.cls, num_labels: int = 1, device=None, seed: int = 0,
                 backbone=None, head_seed: Optional[int] = None):
        super().__init__()
        if backbone is None:
            backbone = TextTransformer(vocab_size, max_seq_len, embed_dim, num_layers=num_layers, num_heads=num_heads,
                                       dropout_p=dropout_p, device=device, seed=seed)
            head_seed = seed + 424242 if head_seed is None else head_seed
        self.backbone = backbone
        self.pooling, self.num_labels = PoolingMode(pooling), num_labels
        self.head = Linear(backbone.embed_dim, num_labels, device=device,
                           seed=424242 if head_seed is None else head_seed, dtype=backbone.dtype)

    @classmethod
    def wrap(cls, backbone, pooling: PoolingMode = PoolingMode.cls, num_labels: int = 1, device=None,
             seed: int = 424242):
        return cls(backbone=backbone, pooling=pooling, num_labels=num_labels, device=device, head_seed=seed)

    @property
    def embed_dim(self) -> int:
        return self.backbone.embed_dim

    def submodules(self):
        return [self.backbone, self.head]

    def forward(self, pair_tokens):
        return self.head(pool_tokens(self.backbone(pair_tokens), self.pooling))

    def score(self, pair_tokens) -> float:
        with torch.no_grad():
            return float(torch.sigmoid(self.forward(pair_tokens).float()).reshape(-1)[0])


@dataclass
class SemanticSearchHit:
    corpus_index: int
    score: float

    @property
    def corpusIndex(self):
        return self.corpus_index

    def __str__(self):
        return f"SemanticSearchHit(idx={self.corpus_index}, score={self.score:.4f})"


class Similarity:
    """Dot-product scores over L2-normalised rows (so cosine = dot)."""

    @staticmethod
    def _require_row(t, name):
        if t.dim() != 2 or t.shape[0] != 1:
            raise ValueError(f"{name}: expected [1, D]; got {list(t.shape)}")

    @staticmethod
    def cos_sim(a, b) -> float:
        Similarity._require_row(a, "cosSim.a")
        Similarity._require_row(b, "cosSim.b")
        if a.shape[1] != b.shape[1]:
            raise ValueError(f"cosSim: dim mismatch {a.shape[1]} vs {b.shape[1]}")
        with torch.no_grad():
            return float((a.float() * b.float()).sum())

    dot_score = cos_sim

    @staticmethod
    def pairwise(a, b):
        if a.dim() != 2 or b.dim() != 2:
            raise ValueError(f"pairwise: expected 2D [N, D]; got {list(a.shape)} and {list(b.shape)}")
        if a.shape[1] != b.shape[1]:
            raise ValueError(f"pairwise: dim mismatch {a.shape[1]} vs {b.shape[1]}")
        with torch.no_grad():
            return F.matmul(a, F.transpose(b))

    @staticmethod
    def semantic_search(queries, corpus, top_k: int = 10) -> List[List[SemanticSearchHit]]:
        if queries.dim() != 2 or corpus.dim() != 2:
            raise ValueError(f"semanticSearch: expected 2D [Q, D] and [N, D]; got {list(queries.shape)} and "
                             f"{list(corpus.shape)}")
        if queries.shape[1] != corpus.shape[1]:
            raise ValueError(f"semanticSearch: dim mismatch {queries.shape[1]} vs {corpus.shape[1]}")
        k = min(top_k, corpus.shape[0])
        scores = Similarity.pairwise(queries, corpus).float()
        vals, idx = torch.sort(scores, dim=1, descending=True, stable=True)
        vals, idx = vals[:, :k].cpu(), idx[:, :k].cpu()
        return [[SemanticSearchHit(int(idx[i, j]), float(vals[i, j])) for j in range(k)]
                for i in range(queries.shape[0])]

    cosSim, dotScore, semanticSearch = cos_sim, dot_score, semantic_search


class SentenceLosses:
    @staticmethod
    def _require_matrix(t, name):
        if t.dim() != 2:
            raise ValueError(f"{name}: expected 2D [N, D]; got {list(t.shape)}")

    @staticmethod
    def multiple_negatives_ranking_loss(anchors, positives, scale: float = 20.0):
        """In-batch softmax: row ``i`` of ``scale * A P^T`` should pick column ``i``; returns the ``[N]`` losses."""
        SentenceLosses._require_matrix(anchors, "multipleNegativesRankingLoss.anchors")
        SentenceLosses._require_matrix(positives, "multipleNegativesRankingLoss.positives")
        if anchors.shape != positives.shape:
            raise ValueError(f"multipleNegativesRankingLoss: shape mismatch {list(anchors.shape)} vs "
                             f"{list(positives.shape)}")
        scores = F.mul(F.matmul(anchors, F.transpose(positives)), scale)
        targets = torch.arange(anchors.shape[0], device=anchors.device)
        return F.cross_entropy(scores, targets)

    @staticmethod
    def _row_dots(a, b):
        ones = torch.ones(a.shape[1], 1, device=a.device, dtype=a.dtype)
        return F.matmul(F.mul(a, b), ones)            # [N, 1]

    @staticmethod
    def cosine_similarity_loss(a, b, targets):
        SentenceLosses._require_matrix(a, "cosineSimilarityLoss.a")
        SentenceLosses._require_matrix(b, "cosineSimilarityLoss.b")
        if a.shape != b.shape:
            raise ValueError(f"cosineSimilarityLoss: shape mismatch {list(a.shape)} vs {list(b.shape)}")
        n = a.shape[0]
        if targets.dim() != 1 or targets.shape[0] != n:
            raise ValueError(f"cosineSimilarityLoss: targets must be [{n}]; got {list(targets.shape)}")
        diff = F.sub(SentenceLosses._row_dots(a, b), targets.reshape(n, 1).to(a.dtype))
        return F.mean(F.mul(diff, diff))

    @staticmethod
    def triplet_loss(anchors, positives, negatives, margin: float = 0.5):
        for t, nm in ((anchors, "anchors"), (positives, "positives"), (negatives, "negatives")):
            SentenceLosses._require_matrix(t, f"tripletLoss.{nm}")
        if not (anchors.shape == positives.shape == negatives.shape):
            raise ValueError(f"tripletLoss: shape mismatch a={list(anchors.shape)} p={list(positives.shape)} "
                             f"n={list(negatives.shape)}")
        gap = F.add(F.sub(SentenceLosses._row_dots(anchors, negatives), SentenceLosses._row_dots(anchors, positives)),
                    margin)
        return F.mean(F.relu(gap))

    multipleNegativesRankingLoss = multiple_negatives_ranking_loss
    cosineSimilarityLoss, tripletLoss = cosine_similarity_loss, triplet_loss
