"""Vector-store core types (reference: lib/core/vector_store/index.dart:1-331).

Vectors are rows of a C-contiguous ``float32`` NumPy array ``[n, d]`` (lists of rows and torch tensors are accepted and
converted).  A search returns ``SearchResult(distances [nq, k], ids [nq, k])`` with unfilled slots ``(+inf | -inf, -1)``;
L2 results are squared distances in ascending order, inner-product results are similarities in descending order.
"""
from __future__ import annotations

from enum import Enum
from typing import Iterable, List, Sequence, Set

import numpy as np


class Metric(Enum):
    l2 = 0
    inner_product = 1
    innerProduct = 1


def as_rows(xs, d: int) -> np.ndarray:
    """Anything row-like -> contiguous float32 ``[n, d]``; raises on a width mismatch."""
    if hasattr(xs, "detach"):
        xs = xs.detach().float().cpu().numpy()
    a = np.asarray(xs, dtype=np.float32)
    if a.ndim == 1:
        a = a.reshape(1, -1) if a.size else a.reshape(0, d)
    if a.ndim != 2 or a.shape[1] != d:
        raise ValueError(f"expected rows of length {d}, got array of shape {tuple(a.shape)}")
    return np.ascontiguousarray(a)


to_float32_rows = as_rows


class SearchResult:
    def __init__(self, distances: np.ndarray, ids: np.ndarray):
        self.distances = np.asarray(distances, dtype=np.float32)
        self.ids = np.asarray(ids, dtype=np.int64)

    @property
    def nq(self) -> int:
        return self.distances.shape[0]

    @property
    def k(self) -> int:
        return 0 if self.nq == 0 else self.distances.shape[1]


class RangeSearchResult:
    """CSR layout: matches of query ``q`` are ``[limits[q], limits[q+1])`` of ``distances`` / ``ids``."""

    def __init__(self, limits, distances, ids):
        self.limits = np.asarray(limits, dtype=np.int64)
        self.distances = np.asarray(distances, dtype=np.float32)
        self.ids = np.asarray(ids, dtype=np.int64)

    @property
    def nq(self) -> int:
        return len(self.limits) - 1

    @property
    def total_matches(self) -> int:
        return int(self.limits[-1]) if len(self.limits) else 0

    totalMatches = total_matches

    def length_for(self, qi: int) -> int:
        return int(self.limits[qi + 1] - self.limits[qi])

    lengthFor = length_for

    @classmethod
    def from_per_query(cls, per_query_dist: Sequence[Sequence[float]], per_query_ids: Sequence[Sequence[int]]):
        limits = np.zeros(len(per_query_dist) + 1, dtype=np.int64)
        for i, row in enumerate(per_query_dist):
            limits[i + 1] = limits[i] + len(row)
        dist = np.concatenate([np.asarray(r, dtype=np.float32) for r in per_query_dist]) if len(per_query_dist) \
            else np.zeros(0, np.float32)
        ids = np.concatenate([np.asarray(r, dtype=np.int64) for r in per_query_ids]) if len(per_query_ids) \
            else np.zeros(0, np.int64)
        return cls(limits, dist, ids)

    fromPerQuery = from_per_query

    def to_rows(self):
        ds = [self.distances[self.limits[q]:self.limits[q + 1]] for q in range(self.nq)]
        is_ = [self.ids[self.limits[q]:self.limits[q + 1]] for q in range(self.nq)]
        return ds, is_

    toRows = to_rows


def l2sq(a, b) -> float:
    diff = np.asarray(a, dtype=np.float32) - np.asarray(b, dtype=np.float32)
    return float(np.dot(diff, diff))


def dot(a, b) -> float:
    return float(np.dot(np.asarray(a, dtype=np.float32), np.asarray(b, dtype=np.float32)))


def pairwise_scores(q: np.ndarray, x: np.ndarray, metric: Metric) -> np.ndarray:
    """``[nq, n]`` squared L2 distances (clamped at 0) or inner products."""
    if metric == Metric.l2:
        qq = np.einsum("ij,ij->i", q, q)[:, None]
        xx = np.einsum("ij,ij->i", x, x)[None, :]
        return np.maximum(qq + xx - 2.0 * (q @ x.T), 0.0).astype(np.float32)
    return (q @ x.T).astype(np.float32)


def select_topk(scores: np.ndarray, k: int, metric: Metric, ids: np.ndarray = None):
    """Best ``k`` per row of ``scores [nq, n]`` -> padded ``(distances [nq, k], ids [nq, k])``; ties by lower index."""
    nq, n = scores.shape
    largest = metric != Metric.l2
    pad = -np.inf if largest else np.inf
    out_d = np.full((nq, k), pad, dtype=np.float32)
    out_i = np.full((nq, k), -1, dtype=np.int64)
    kk = min(k, n)
    if kk == 0:
        return out_d, out_i
    key = -scores if largest else scores
    if ids is None:
        order = np.argsort(key, axis=1, kind="stable")[:, :kk]
        out_i[:, :kk] = order
    else:
        ids = np.asarray(ids, dtype=np.int64)
        by_id = np.argsort(ids, kind="stable")               # equal scores resolve to the lower id
        order = by_id[np.argsort(key[:, by_id], axis=1, kind="stable")[:, :kk]]
        out_i[:, :kk] = ids[order]
    out_d[:, :kk] = np.take_along_axis(scores, order, axis=1)
    return out_d, out_i


class TopK:
    """Bounded best-``k`` collector (a binary heap with the worst kept element at the root)."""

    def __init__(self, k: int, max_is_worst: bool):
        self.k, self.max_is_worst = k, max_is_worst
        self._score: List[float] = []
        self._id: List[int] = []

    @property
    def size(self) -> int:
        return len(self._score)

    @property
    def worst(self) -> float:
        if self.size < self.k:
            return float("inf") if self.max_is_worst else float("-inf")
        return self._score[0]

    def worse_than_worst(self, s: float) -> bool:
        if self.size < self.k:
            return False
        return s >= self._score[0] if self.max_is_worst else s <= self._score[0]

    worseThanWorst = worse_than_worst

    def _worse(self, i: int, j: int) -> bool:
        return self._score[i] > self._score[j] if self.max_is_worst else self._score[i] < self._score[j]

    def _swap(self, i, j):
        self._score[i], self._score[j] = self._score[j], self._score[i]
        self._id[i], self._id[j] = self._id[j], self._id[i]

    def push(self, score: float, idx: int) -> None:
        if self.k <= 0:
            return
        if self.size < self.k:
            self._score.append(float(score))
            self._id.append(int(idx))
            i = self.size - 1
            while i > 0:
                p = (i - 1) >> 1
                if not self._worse(i, p):
                    break
                self._swap(i, p)
                i = p
        elif (self.max_is_worst and score < self._score[0]) or (not self.max_is_worst and score > self._score[0]):
            self._score[0], self._id[0] = float(score), int(idx)
            i, n = 0, self.size
            while True:
                l, r, w = 2 * i + 1, 2 * i + 2, i
                if l < n and self._worse(l, w):
                    w = l
                if r < n and self._worse(r, w):
                    w = r
                if w == i:
                    break
                self._swap(i, w)
                i = w

    def sorted(self):
        """``(scores [k], ids [k])`` best first, padded with ``(+-inf, -1)``."""
        pad = float("inf") if self.max_is_worst else float("-inf")
        scores = np.full(self.k, pad, dtype=np.float32)
        ids = np.full(self.k, -1, dtype=np.int64)
        order = sorted(range(self.size), key=(lambda i: self._score[i]) if self.max_is_worst
                       else (lambda i: -self._score[i]))
        for j, i in enumerate(order):
            scores[j], ids[j] = self._score[i], self._id[i]
        return scores, ids


class Index:
    """Base of every float index: ``d``, ``metric``, ``ntotal``, ``is_trained``; ``train / add / search`` and the optional
    ``range_search`` / ``remove_ids``."""

    def __init__(self, d: int, metric: Metric = Metric.l2):
        if d <= 0:
            raise ValueError("Index: d must be positive")
        self.d, self.metric = int(d), metric
        self.ntotal = 0
        self.is_trained = True

    # camelCase aliases of the reference API
    @property
    def isTrained(self):
        return self.is_trained

    def train(self, xs) -> None:
        self.is_trained = True

    def add(self, xs) -> None:
        raise NotImplementedError

    def search(self, queries, k: int) -> SearchResult:
        raise NotImplementedError

    def range_search(self, queries, radius: float) -> RangeSearchResult:
        raise NotImplementedError(f"{type(self).__name__} does not support rangeSearch")

    def remove_ids(self, ids: Set[int]) -> int:
        raise NotImplementedError(f"{type(self).__name__} does not support removeIds")

    def add_rows(self, xs) -> None:
        self.add(as_rows(xs, self.d))

    def search_rows(self, queries, k: int) -> SearchResult:
        return self.search(as_rows(queries, self.d), k)

    def reconstruct(self, i: int) -> np.ndarray:
        raise NotImplementedError(f"{type(self).__name__} does not support reconstruct")

    rangeSearch, removeIds, addRows, searchRows = range_search, remove_ids, add_rows, search_rows

    def _check_k(self, k: int):
        if k <= 0:
            raise ValueError("search: k must be positive")

    def _range_from_scores(self, scores: np.ndarray, radius: float, ids: np.ndarray = None) -> RangeSearchResult:
        """Matches are ``dist < radius`` for L2 and ``sim > radius`` for inner product, ordered best first."""
        dist_rows, id_rows = [], []
        for row in scores:
            hit = np.nonzero(row < radius if self.metric == Metric.l2 else row > radius)[0]
            order = np.argsort(row[hit] if self.metric == Metric.l2 else -row[hit], kind="stable")
            hit = hit[order]
            dist_rows.append(row[hit])
            id_rows.append(hit if ids is None else np.asarray(ids)[hit])
        return RangeSearchResult.from_per_query(dist_rows, id_rows)
