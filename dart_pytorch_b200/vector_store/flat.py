"""Exact indexes and k-means (reference: lib/core/vector_store/index_flat.dart:1-196, kmeans.dart:1-163,
gpu_index_flat.dart:40-194).

``IndexFlat`` keeps raw rows and scans them; ``remove_ids`` compacts and renumbers.  ``GpuIndexFlat`` keeps a bf16 / fp32
copy of the database on the GPU, scores ``Q D^T`` with the framework's tensor-core GEMM, forms L2 as
``|q|^2 + |d|^2 - 2 q.d`` and selects the top-k on the device; below ``2^18`` multiply-adds it falls back to the CPU scan,
as the reference does.
"""
from __future__ import annotations

from typing import Optional, Set

import numpy as np

from .base import Index, Metric, RangeSearchResult, SearchResult, as_rows, pairwise_scores, select_topk


class _RowStore:
    """Growable ``[n, d]`` float32 array."""

    def __init__(self, d: int, dtype=np.float32):
        self._buf = np.zeros((0, d), dtype=dtype)
        self.n = 0

    def append(self, rows: np.ndarray) -> None:
        need = self.n + len(rows)
        if need > len(self._buf):
            cap = max(need, 2 * len(self._buf), 16)
            nb = np.zeros((cap, self._buf.shape[1]), dtype=self._buf.dtype)
            nb[:self.n] = self._buf[:self.n]
            self._buf = nb
        self._buf[self.n:need] = rows
        self.n = need

    @property
    def view(self) -> np.ndarray:
        return self._buf[:self.n]

    def keep(self, mask: np.ndarray) -> None:
        kept = self._buf[:self.n][mask]
        self._buf[:len(kept)] = kept
        self.n = len(kept)


class IndexFlat(Index):
    def __init__(self, d: int, metric: Metric = Metric.l2):
        super().__init__(d, metric)
        self._store = _RowStore(d)

    @property
    def storage(self) -> np.ndarray:
        return self._store.view

    def add(self, xs) -> None:
        self._store.append(as_rows(xs, self.d))
        self.ntotal = self._store.n

    def reconstruct(self, i: int) -> np.ndarray:
        if not (0 <= i < self.ntotal):
            raise IndexError(f"reconstruct: id {i} out of range [0, {self.ntotal})")
        return self._store.view[i]

    def search(self, queries, k: int) -> SearchResult:
        self._check_k(k)
        q = as_rows(queries, self.d)
        return SearchResult(*select_topk(pairwise_scores(q, self.storage, self.metric), k, self.metric))

    def range_search(self, queries, radius: float) -> RangeSearchResult:
        q = as_rows(queries, self.d)
        return self._range_from_scores(pairwise_scores(q, self.storage, self.metric), radius)

    def remove_ids(self, ids: Set[int]) -> int:
        if not ids:
            return 0
        mask = np.ones(self.ntotal, dtype=bool)
        hit = [i for i in ids if 0 <= i < self.ntotal]
        mask[hit] = False
        self._store.keep(mask)
        self.ntotal = self._store.n
        return len(hit)

    rangeSearch, removeIds = range_search, remove_ids


class IndexFlatIP(IndexFlat):
    def __init__(self, d: int):
        super().__init__(d, Metric.inner_product)


class IndexFlatL2(IndexFlat):
    def __init__(self, d: int):
        super().__init__(d, Metric.l2)


GPU_INDEX_FLAT_MIN_DOT = 1 << 18


class GpuIndexFlat(Index):
    def __init__(self, backing: IndexFlat, device: Optional[str] = None, dtype=None):
        super().__init__(backing.d, backing.metric)
        self._backing = backing
        self.ntotal, self.is_trained = backing.ntotal, backing.is_trained
        self._device, self._dtype = device, dtype
        self._db = None
        self._db_norms = None

    @classmethod
    def l2(cls, d: int, **kw):
        return cls(IndexFlat(d, Metric.l2), **kw)

    @classmethod
    def ip(cls, d: int, **kw):
        return cls(IndexFlat(d, Metric.inner_product), **kw)

    @classmethod
    def wrap(cls, src: IndexFlat, **kw):
        return cls(src, **kw)

    @property
    def backing(self) -> IndexFlat:
        return self._backing

    def train(self, xs) -> None:
        self._backing.train(xs)

    def add(self, xs) -> None:
        self._backing.add(xs)
        self._db = self._db_norms = None
        self.ntotal, self.is_trained = self._backing.ntotal, self._backing.is_trained

    def _resolve_device(self):
        import torch
        if self._device is not None:
            return torch.device(self._device)
        return torch.device("cuda" if torch.cuda.is_available() else "cpu")

    def warmup(self) -> None:
        import torch
        if self._db is not None or self._backing.ntotal == 0:
            return
        dev = self._resolve_device()
        dtype = self._dtype or (torch.bfloat16 if dev.type == "cuda" else torch.float32)
        host = torch.from_numpy(np.ascontiguousarray(self._backing.storage))
        self._db = host.to(device=dev, dtype=dtype)
        if self.metric == Metric.l2:
            self._db_norms = (self._db.float() ** 2).sum(1)

    def search(self, queries, k: int) -> SearchResult:
        import torch
        from .. import ops as F
        self._check_k(k)
        q = as_rows(queries, self.d)
        n = self._backing.ntotal
        if len(q) == 0:
            return SearchResult(np.zeros((0, k), np.float32), np.zeros((0, k), np.int64))
        if n == 0 or len(q) * n * self.d < GPU_INDEX_FLAT_MIN_DOT:
            return self._backing.search(q, k)
        self.warmup()
        qt = torch.from_numpy(q).to(device=self._db.device, dtype=self._db.dtype)
        with torch.no_grad():
            scores = F.linear(qt, self._db).float()                       # [nq, n] = Q D^T
            if self.metric == Metric.l2:
                scores = ((qt.float() ** 2).sum(1, keepdim=True) + self._db_norms[None, :] - 2.0 * scores).clamp_min_(0)
            kk = min(k, n)
            vals, idx = torch.topk(scores, kk, dim=1, largest=self.metric != Metric.l2, sorted=True)
        pad = np.inf if self.metric == Metric.l2 else -np.inf
        out_d = np.full((len(q), k), pad, dtype=np.float32)
        out_i = np.full((len(q), k), -1, dtype=np.int64)
        out_d[:, :kk], out_i[:, :kk] = vals.cpu().numpy(), idx.cpu().numpy()
        return SearchResult(out_d, out_i)


class KmeansResult:
    def __init__(self, centroids: np.ndarray, assignments: np.ndarray, objective: float):
        self.centroids, self.assignments, self.objective = centroids, assignments, objective


class Kmeans:
    """k-means++ seeding and Lloyd iterations; empty clusters are re-seeded from the point farthest from its centroid."""

    def __init__(self, d: int, k: int, niter: int = 20, seed: int = 1234, min_points_per_centroid: int = 1,
                 verbose: bool = False):
        self.d, self.k, self.niter, self.seed = d, k, niter, seed
        self.min_points_per_centroid, self.verbose = min_points_per_centroid, verbose

    def train(self, xs) -> KmeansResult:
        x = as_rows(xs, self.d)
        n = len(x)
        if n < self.k * self.min_points_per_centroid:
            raise ValueError(f"Kmeans: need at least {self.k * self.min_points_per_centroid} training points for "
                             f"k={self.k}, got {n}")
        rng = np.random.default_rng(self.seed)
        cent = np.empty((self.k, self.d), dtype=np.float32)
        cent[0] = x[rng.integers(n)]
        best = ((x - cent[0]) ** 2).sum(1)
        for c in range(1, self.k):
            total = float(best.sum())
            pick = rng.integers(n) if total <= 0 else int(np.searchsorted(np.cumsum(best), rng.random() * total))
            cent[c] = x[min(pick, n - 1)]
            best = np.minimum(best, ((x - cent[c]) ** 2).sum(1))
        assign = np.zeros(n, dtype=np.int64)
        obj = float("inf")
        for it in range(max(1, self.niter)):
            dist = pairwise_scores(x, cent, Metric.l2)
            assign = dist.argmin(1)
            mind = dist[np.arange(n), assign]
            obj = float(mind.sum())
            counts = np.bincount(assign, minlength=self.k)
            sums = np.zeros((self.k, self.d), dtype=np.float64)
            np.add.at(sums, assign, x)
            nonempty = counts > 0
            cent[nonempty] = (sums[nonempty] / counts[nonempty, None]).astype(np.float32)
            for c in np.nonzero(~nonempty)[0]:
                far = int(mind.argmax())
                cent[c] = x[far]
                mind[far] = 0.0
            if self.verbose:
                print(f"kmeans iter {it}: objective {obj:.4f}")
        return KmeansResult(cent, assign.astype(np.int32), obj)
