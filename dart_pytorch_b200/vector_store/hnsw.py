"""Hierarchical navigable small-world graph index (reference: lib/core/vector_store/index_hnsw.dart:1-627).

Levels are drawn as ``floor(-ln(u) / ln(M))``; insertion descends greedily through the upper layers, then runs a beam
search of width ``efConstruction`` per layer, links to at most ``M`` (``2M`` on layer 0) neighbours chosen by the
diversity heuristic (a candidate is kept only if it is closer to the new point than to every neighbour already kept),
and re-prunes neighbours whose lists overflow.  Queries descend greedily and beam-search layer 0 with
``max(efSearch, k)``.  Inner-product search orders by negated similarity internally.
"""
from __future__ import annotations

import heapq
import math
import random
from typing import List, Sequence

import numpy as np

from .base import Index, Metric, SearchResult, as_rows
from .flat import _RowStore


class IndexHNSW(Index):
    def __init__(self, d: int, M: int = 16, ef_construction: int = 100, ef_search: int = 32, seed: int = 1234,
                 metric: Metric = Metric.l2):
        super().__init__(d, metric)
        if M < 2:
            raise ValueError("IndexHNSW: M must be >= 2")
        self.M, self.Mmax, self.Mmax0 = M, M, 2 * M
        self.ef_construction, self.ef_search, self.seed = ef_construction, ef_search, seed
        self._ml = 1.0 / math.log(M)
        self._rng = random.Random(seed)
        self._store = _RowStore(d)
        self._levels: List[int] = []
        self._nbrs: List[List[List[int]]] = []       # node -> layer -> neighbour ids
        self._entry, self._top = -1, -1

    # ---- introspection (persistence, tests) --------------------------------------------------
    @property
    def storage(self) -> np.ndarray:
        return self._store.view

    @property
    def entry_point(self) -> int:
        return self._entry

    @property
    def top_level(self) -> int:
        return self._top

    def node_level(self, i: int) -> int:
        return self._levels[i]

    def node_neighbors(self, i: int, layer: int) -> List[int]:
        return self._nbrs[i][layer]

    entryPoint, topLevel, nodeLevel, nodeNeighbors = entry_point, top_level, node_level, node_neighbors

    @property
    def efSearch(self):
        return self.ef_search

    @efSearch.setter
    def efSearch(self, v):
        self.ef_search = v

    def io_set(self, storage: np.ndarray, levels: Sequence[int], nbrs: List[List[List[int]]], entry: int,
               top: int) -> None:
        self._store = _RowStore(self.d)
        self._store.append(as_rows(storage, self.d))
        self._levels = [int(l) for l in levels]
        self._nbrs = [[list(map(int, layer)) for layer in node] for node in nbrs]
        self._entry, self._top, self.ntotal = int(entry), int(top), self._store.n

    # ---- distances --------------------------------------------------------------------------
    def _dist_many(self, ids: Sequence[int], q: np.ndarray) -> np.ndarray:
        x = self._store.view[np.asarray(ids, dtype=np.int64)]
        if self.metric == Metric.l2:
            diff = x - q
            return np.einsum("ij,ij->i", diff, diff)
        return -(x @ q)

    def _dist(self, a: int, q: np.ndarray) -> float:
        return float(self._dist_many([a], q)[0])

    # ---- graph walks ------------------------------------------------------------------------
    def _greedy(self, q: np.ndarray, entry: int, layer: int) -> int:
        cur, cur_d = entry, self._dist(entry, q)
        improved = True
        while improved:
            improved = False
            nb = self._nbrs[cur][layer]
            if not nb:
                break
            ds = self._dist_many(nb, q)
            j = int(ds.argmin())
            if ds[j] < cur_d:
                cur, cur_d, improved = nb[j], float(ds[j]), True
        return cur

    def _search_layer(self, q: np.ndarray, entries: Sequence[int], ef: int, layer: int):
        visited = set()
        cand: list = []          # min-heap of (dist, id)
        res: list = []           # max-heap via (-dist, id)
        for e in entries:
            if e in visited:
                continue
            visited.add(e)
            de = self._dist(e, q)
            heapq.heappush(cand, (de, e))
            heapq.heappush(res, (-de, e))
        while cand:
            dc, c = cand[0]
            if len(res) >= ef and dc > -res[0][0]:
                break
            heapq.heappop(cand)
            fresh = [n for n in self._nbrs[c][layer] if n not in visited]
            if not fresh:
                continue
            visited.update(fresh)
            for n, dn in zip(fresh, self._dist_many(fresh, q)):
                dn = float(dn)
                if len(res) < ef or dn < -res[0][0]:
                    heapq.heappush(cand, (dn, n))
                    heapq.heappush(res, (-dn, n))
                    if len(res) > ef:
                        heapq.heappop(res)
        out = sorted((-nd, i) for nd, i in res)
        return [i for _, i in out], [dd for dd, _ in out]

    def _select(self, cand_ids: Sequence[int], cand_d: Sequence[float], m: int) -> List[int]:
        chosen: List[int] = []
        for j in np.argsort(np.asarray(cand_d), kind="stable"):
            if len(chosen) >= m:
                break
            e, ed = cand_ids[int(j)], cand_d[int(j)]
            if chosen and float(self._dist_many(chosen, self._store.view[e]).min()) < ed:
                continue
            chosen.append(e)
        return chosen

    # ---- index API --------------------------------------------------------------------------
    def _sample_level(self) -> int:
        u = self._rng.random()
        return int(math.floor(-math.log(u if u > 0 else 1e-12) * self._ml))

    def _add_one(self, x: np.ndarray) -> None:
        idx = self.ntotal
        self._store.append(x[None, :])
        level = self._sample_level()
        self._levels.append(level)
        self._nbrs.append([[] for _ in range(level + 1)])
        self.ntotal += 1
        if self._entry < 0:
            self._entry, self._top = idx, level
            return
        cur = self._entry
        for l in range(self._top, level, -1):
            cur = self._greedy(x, cur, l)
        entries = [cur]
        for l in range(min(self._top, level), -1, -1):
            ids, ds = self._search_layer(x, entries, self.ef_construction, l)
            budget = self.Mmax0 if l == 0 else self.Mmax
            chosen = self._select(ids, ds, budget)
            self._nbrs[idx][l].extend(chosen)
            for nb in chosen:
                lst = self._nbrs[nb][l]
                lst.append(idx)
                if len(lst) > budget:
                    dd = self._dist_many(lst, self._store.view[nb]).tolist()
                    self._nbrs[nb][l] = self._select(list(lst), dd, budget)
            entries = ids
        if level > self._top:
            self._top, self._entry = level, idx

    def add(self, xs) -> None:
        for row in as_rows(xs, self.d):
            self._add_one(row)

    def reconstruct(self, i: int) -> np.ndarray:
        return self._store.view[i]

    def search(self, queries, k: int) -> SearchResult:
        self._check_k(k)
        q = as_rows(queries, self.d)
        pad = np.inf if self.metric == Metric.l2 else -np.inf
        out_d = np.full((len(q), k), pad, dtype=np.float32)
        out_i = np.full((len(q), k), -1, dtype=np.int64)
        if self.ntotal == 0 or self._entry < 0:
            return SearchResult(out_d, out_i)
        for qi, row in enumerate(q):
            cur = self._entry
            for l in range(self._top, 0, -1):
                cur = self._greedy(row, cur, l)
            ids, ds = self._search_layer(row, [cur], max(self.ef_search, k), 0)
            n = min(k, len(ids))
            out_i[qi, :n] = ids[:n]
            out_d[qi, :n] = ds[:n] if self.metric == Metric.l2 else [-v for v in ds[:n]]
        return SearchResult(out_d, out_i)
