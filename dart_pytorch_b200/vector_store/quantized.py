"""Product quantisation, inverted files and 8-bit scalar quantisation
(reference: lib/core/vector_store/index_pq.dart:1-356, index_ivf_flat.dart:1-337, index_ivf_pq.dart:1-287,
index_scalar_quantizer.dart:1-263).

* ``ProductQuantizer``: ``m`` sub-spaces of ``d/m`` dims, ``2^nbits`` k-means centroids each (``nbits <= 8``: one byte per
  sub-code); asymmetric distance through per-query look-up tables.
* ``IndexPQ``: flat list of codes.  ``IndexIVFFlat``: coarse k-means cells with raw vectors; ``nprobe`` cells scanned per
  query; ``remove_ids`` renumbers like ``IndexFlat``.  ``IndexIVFPQ``: cells hold PQ codes of the residual to the cell
  centroid.  ``IndexScalarQuantizer``: per-dimension min/max trained 8-bit codes.
"""
from __future__ import annotations

from typing import List, Optional, Set

import numpy as np

from .base import Index, Metric, RangeSearchResult, SearchResult, as_rows, pairwise_scores, select_topk
from .flat import IndexFlat, Kmeans, _RowStore


class ProductQuantizer:
    def __init__(self, d: int, m: int, nbits: int = 8, kmeans_iters: int = 25, seed: int = 1234):
        if d % m:
            raise ValueError(f"ProductQuantizer: d={d} not divisible by m={m}")
        if not (1 <= nbits <= 8):
            raise ValueError("ProductQuantizer: nbits must be in [1, 8]")
        self.d, self.m, self.nbits = d, m, nbits
        self.ksub, self.dsub = 1 << nbits, d // m
        self.kmeans_iters, self.seed = kmeans_iters, seed
        self.is_trained = False
        self.codebooks = np.zeros((m, self.ksub, self.dsub), dtype=np.float32)

    def train(self, xs) -> None:
        x = as_rows(xs, self.d)
        if len(x) < self.ksub:
            raise ValueError(f"ProductQuantizer.train: need >= {self.ksub} vectors, got {len(x)}")
        for s in range(self.m):
            sub = np.ascontiguousarray(x[:, s * self.dsub:(s + 1) * self.dsub])
            self.codebooks[s] = Kmeans(self.dsub, self.ksub, niter=self.kmeans_iters, seed=self.seed + s).train(
                sub).centroids
        self.is_trained = True

    def encode(self, xs) -> np.ndarray:
        """``[n, m]`` uint8 codes."""
        x = as_rows(xs, self.d)
        codes = np.empty((len(x), self.m), dtype=np.uint8)
        for s in range(self.m):
            sub = np.ascontiguousarray(x[:, s * self.dsub:(s + 1) * self.dsub])
            codes[:, s] = pairwise_scores(sub, self.codebooks[s], Metric.l2).argmin(1)
        return codes

    def decode(self, codes: np.ndarray) -> np.ndarray:
        codes = np.asarray(codes, dtype=np.uint8).reshape(-1, self.m)
        return np.concatenate([self.codebooks[s][codes[:, s]] for s in range(self.m)], axis=1)

    def decode_one(self, codes: np.ndarray, i: int) -> np.ndarray:
        return self.decode(np.asarray(codes).reshape(-1, self.m)[i:i + 1])[0]

    def build_l2_lut(self, q) -> np.ndarray:
        """``[m, ksub]`` squared distances from each query sub-vector to each centroid."""
        qs = np.asarray(q, dtype=np.float32).reshape(self.m, 1, self.dsub)
        return ((self.codebooks - qs) ** 2).sum(-1)

    def build_ip_lut(self, q) -> np.ndarray:
        qs = np.asarray(q, dtype=np.float32).reshape(self.m, self.dsub, 1)
        return (self.codebooks @ qs)[..., 0]

    def lut(self, q, metric: Metric) -> np.ndarray:
        return self.build_l2_lut(q) if metric == Metric.l2 else self.build_ip_lut(q)

    def adc(self, lut: np.ndarray, codes: np.ndarray) -> np.ndarray:
        """Asymmetric scores of ``codes [n, m]`` under one query's table."""
        return lut[np.arange(self.m)[None, :], codes].sum(1).astype(np.float32)

    decodeOne, buildL2LUT, buildIPLUT = decode_one, build_l2_lut, build_ip_lut


class IndexPQ(Index):
    def __init__(self, d: int, m: int, nbits: int = 8, kmeans_iters: int = 25, seed: int = 1234,
                 metric: Metric = Metric.l2):
        super().__init__(d, metric)
        self.m = m
        self.pq = ProductQuantizer(d, m, nbits, kmeans_iters, seed)
        self.is_trained = False
        self._codes = _RowStore(m, dtype=np.uint8)

    @property
    def codes(self) -> np.ndarray:
        return self._codes.view

    def train(self, xs) -> None:
        self.pq.train(xs)
        self.is_trained = True

    def add(self, xs) -> None:
        if not self.is_trained:
            raise RuntimeError("IndexPQ.add before train()")
        self._codes.append(self.pq.encode(xs))
        self.ntotal = self._codes.n

    def reconstruct(self, i: int) -> np.ndarray:
        return self.pq.decode_one(self.codes, i)

    def search(self, queries, k: int) -> SearchResult:
        self._check_k(k)
        if not self.is_trained:
            raise RuntimeError("IndexPQ.search before train()")
        q = as_rows(queries, self.d)
        scores = np.stack([self.pq.adc(self.pq.lut(row, self.metric), self.codes) for row in q]) if len(q) else \
            np.zeros((0, self.ntotal), np.float32)
        return SearchResult(*select_topk(scores, k, self.metric))


class _IVFBase(Index):
    def __init__(self, d: int, nlist: int, nprobe: int, kmeans_iters: int, seed: int, metric: Metric):
        super().__init__(d, metric)
        if nlist <= 0:
            raise ValueError("nlist must be positive")
        self.nlist, self.nprobe, self.kmeans_iters, self.seed = nlist, nprobe, kmeans_iters, seed
        self.quantizer = IndexFlat(d, metric)
        self.is_trained = False

    def _train_coarse(self, x: np.ndarray, who: str):
        if len(x) < self.nlist:
            raise ValueError(f"{who}.train: need >= nlist={self.nlist} vectors, got {len(x)}")
        res = Kmeans(self.d, self.nlist, niter=self.kmeans_iters, seed=self.seed).train(x)
        self.quantizer.add(res.centroids)
        return res

    def _probe(self, q: np.ndarray) -> np.ndarray:
        return self.quantizer.search(q, max(1, min(self.nprobe, self.nlist))).ids


class IndexIVFFlat(_IVFBase):
    def __init__(self, d: int, nlist: int, nprobe: int = 1, kmeans_iters: int = 20, seed: int = 1234,
                 metric: Metric = Metric.l2):
        super().__init__(d, nlist, nprobe, kmeans_iters, seed, metric)
        self._store = _RowStore(d)
        self._inv_lists: List[List[int]] = [[] for _ in range(nlist)]

    @property
    def storage(self) -> np.ndarray:
        return self._store.view

    @property
    def inv_lists(self) -> List[List[int]]:
        return self._inv_lists

    invLists = inv_lists

    def list_sizes(self) -> List[int]:
        return [len(l) for l in self._inv_lists]

    listSizes = list_sizes

    def train(self, xs) -> None:
        self._train_coarse(as_rows(xs, self.d), "IndexIVFFlat")
        self.is_trained = True

    def add(self, xs) -> None:
        if not self.is_trained:
            raise RuntimeError("IndexIVFFlat.add before train()")
        x = as_rows(xs, self.d)
        if not len(x):
            return
        cells = self.quantizer.search(x, 1).ids[:, 0]
        for i, c in enumerate(cells):
            self._inv_lists[int(c)].append(self.ntotal + i)
        self._store.append(x)
        self.ntotal = self._store.n

    def reconstruct(self, i: int) -> np.ndarray:
        return self._store.view[i]

    def search(self, queries, k: int) -> SearchResult:
        self._check_k(k)
        if not self.is_trained:
            raise RuntimeError("IndexIVFFlat.search before train()")
        q = as_rows(queries, self.d)
        probes = self._probe(q)
        out_d, out_i = [], []
        for qi in range(len(q)):
            ids = np.fromiter((i for c in probes[qi] if c >= 0 for i in self._inv_lists[int(c)]), dtype=np.int64)
            scores = pairwise_scores(q[qi:qi + 1], self._store.view[ids], self.metric) if len(ids) else \
                np.zeros((1, 0), np.float32)
            dd, ii = select_topk(scores, k, self.metric, ids)
            out_d.append(dd[0])
            out_i.append(ii[0])
        return SearchResult(np.stack(out_d) if out_d else np.zeros((0, k), np.float32),
                            np.stack(out_i) if out_i else np.zeros((0, k), np.int64))

    def range_search(self, queries, radius: float) -> RangeSearchResult:
        """Every stored vector of the ``nprobe`` probed cells within ``radius`` (L2: distance below it, inner product:
        similarity above it), best first; equals the flat result when ``nprobe == nlist``
        (reference: lib/core/vector_store/index_ivf_flat.dart:173-215)."""
        if not self.is_trained:
            raise RuntimeError("IndexIVFFlat.rangeSearch before train()")
        q = as_rows(queries, self.d)
        probes = self._probe(q)
        dist_rows, id_rows = [], []
        for qi in range(len(q)):
            ids = np.fromiter((i for c in probes[qi] if c >= 0 for i in self._inv_lists[int(c)]), dtype=np.int64)
            scores = pairwise_scores(q[qi:qi + 1], self._store.view[ids], self.metric) if len(ids) else \
                np.zeros((1, 0), np.float32)
            one = self._range_from_scores(scores, radius, ids)
            dist_rows.append(one.distances)
            id_rows.append(one.ids)
        return RangeSearchResult.from_per_query(dist_rows, id_rows)

    rangeSearch = range_search

    def remove_ids(self, ids: Set[int]) -> int:
        hit = sorted(i for i in ids if 0 <= i < self.ntotal)
        if not hit:
            return 0
        mask = np.ones(self.ntotal, dtype=bool)
        mask[hit] = False
        remap = np.cumsum(mask) - 1
        self._store.keep(mask)
        self._inv_lists = [[int(remap[i]) for i in lst if mask[i]] for lst in self._inv_lists]
        self.ntotal = self._store.n
        return len(hit)

    removeIds = remove_ids

    def io_set(self, storage: np.ndarray, inv_lists: List[List[int]]) -> None:
        """Install decoded state (persistence / conversion helpers)."""
        self._store = _RowStore(self.d)
        self._store.append(as_rows(storage, self.d))
        self._inv_lists = [list(map(int, l)) for l in inv_lists]
        self.ntotal = self._store.n


class IndexIVFPQ(_IVFBase):
    def __init__(self, d: int, nlist: int, m: int, nbits: int = 8, nprobe: int = 1, kmeans_iters: int = 20,
                 pq_kmeans_iters: int = 25, seed: int = 1234, metric: Metric = Metric.l2):
        super().__init__(d, nlist, nprobe, kmeans_iters, seed, metric)
        self.m, self.pq_kmeans_iters = m, pq_kmeans_iters
        self.pq = ProductQuantizer(d, m, nbits, pq_kmeans_iters, seed)
        self._ids: List[List[int]] = [[] for _ in range(nlist)]
        self._codes: List[List[np.ndarray]] = [[] for _ in range(nlist)]

    @property
    def inv_lists_ids(self) -> List[List[int]]:
        return self._ids

    def cell_codes(self, c: int) -> np.ndarray:
        return np.concatenate(self._codes[c]).reshape(-1, self.m) if self._codes[c] else \
            np.zeros((0, self.m), np.uint8)

    def list_sizes(self) -> List[int]:
        return [len(l) for l in self._ids]

    invListsIds, listSizes = inv_lists_ids, list_sizes

    def train(self, xs) -> None:
        x = as_rows(xs, self.d)
        res = self._train_coarse(x, "IndexIVFPQ")
        self.pq.train(x - res.centroids[res.assignments])
        self.is_trained = True

    def add(self, xs) -> None:
        if not self.is_trained:
            raise RuntimeError("IndexIVFPQ.add before train()")
        x = as_rows(xs, self.d)
        if not len(x):
            return
        cells = self.quantizer.search(x, 1).ids[:, 0]
        codes = self.pq.encode(x - self.quantizer.storage[cells])
        for i, c in enumerate(cells):
            self._ids[int(c)].append(self.ntotal + i)
            self._codes[int(c)].append(codes[i:i + 1])
        self.ntotal += len(x)

    def search(self, queries, k: int) -> SearchResult:
        self._check_k(k)
        if not self.is_trained:
            raise RuntimeError("IndexIVFPQ.search before train()")
        q = as_rows(queries, self.d)
        probes = self._probe(q)
        out_d = np.full((len(q), k), np.inf if self.metric == Metric.l2 else -np.inf, dtype=np.float32)
        out_i = np.full((len(q), k), -1, dtype=np.int64)
        for qi in range(len(q)):
            all_s, all_i = [], []
            for c in probes[qi]:
                if c < 0 or not self._ids[int(c)]:
                    continue
                cen = self.quantizer.storage[int(c)]
                s = self.pq.adc(self.pq.lut(q[qi] - cen, self.metric), self.cell_codes(int(c)))
                if self.metric != Metric.l2:
                    s = s + float(np.dot(q[qi], cen))       # q.x = q.cen + q.(x - cen)
                all_s.append(s)
                all_i.append(np.asarray(self._ids[int(c)], dtype=np.int64))
            if all_s:
                dd, ii = select_topk(np.concatenate(all_s)[None, :], k, self.metric, np.concatenate(all_i))
                out_d[qi], out_i[qi] = dd[0], ii[0]
        return SearchResult(out_d, out_i)

    def io_set(self, ids: List[List[int]], codes: List[np.ndarray], ntotal: int) -> None:
        if len(ids) != self.nlist or len(codes) != self.nlist:
            raise ValueError(f"ioSetInvLists: got {len(ids)}/{len(codes)} lists, expected nlist={self.nlist}")
        for c in range(self.nlist):
            cc = np.asarray(codes[c], dtype=np.uint8).reshape(-1)
            if len(cc) != len(ids[c]) * self.m:
                raise ValueError(f"ioSetInvLists: cell {c} has {len(cc)} code bytes but {len(ids[c])} ids")
            self._ids[c] = [int(i) for i in ids[c]]
            self._codes[c] = [cc.reshape(-1, self.m)] if len(cc) else []
        self.ntotal = ntotal


class IndexScalarQuantizer(Index):
    """Per-dimension ``code = round((x - vmin) / scale * 255)`` with ``vmin`` / ``scale = vmax - vmin`` from training."""

    def __init__(self, d: int, metric: Metric = Metric.l2):
        super().__init__(d, metric)
        self.is_trained = False
        self.vmin = np.zeros(d, dtype=np.float32)
        self.scale = np.ones(d, dtype=np.float32)
        self._codes = _RowStore(d, dtype=np.uint8)

    @property
    def codes(self) -> np.ndarray:
        return self._codes.view

    def train(self, xs) -> None:
        x = as_rows(xs, self.d)
        if not len(x):
            raise ValueError("IndexScalarQuantizer.train: empty training set")
        self.vmin = x.min(0)
        span = x.max(0) - self.vmin
        self.scale = np.where(span > 0, span, 1.0).astype(np.float32)
        self.is_trained = True

    def _encode(self, x: np.ndarray) -> np.ndarray:
        t = np.clip((x - self.vmin) / self.scale, 0.0, 1.0)
        return np.floor(t * 255.0 + 0.5).astype(np.uint8)

    def _decode(self, codes: np.ndarray) -> np.ndarray:
        return (self.vmin + codes.astype(np.float32) / 255.0 * self.scale).astype(np.float32)

    def add(self, xs) -> None:
        if not self.is_trained:
            raise RuntimeError("IndexScalarQuantizer.add before train()")
        self._codes.append(self._encode(as_rows(xs, self.d)))
        self.ntotal = self._codes.n

    def reconstruct(self, i: int) -> np.ndarray:
        return self._decode(self.codes[i])

    def search(self, queries, k: int) -> SearchResult:
        self._check_k(k)
        q = as_rows(queries, self.d)
        return SearchResult(*select_topk(pairwise_scores(q, self._decode(self.codes), self.metric), k, self.metric))
