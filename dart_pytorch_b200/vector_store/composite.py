"""Wrapper and hashing indexes, binary (Hamming) indexes, vector transforms, shards / replicas
(reference: lib/core/vector_store/index_id_map.dart, index_refine_flat.dart, index_lsh.dart, index_binary*.dart,
vector_transform.dart, l2_norm_transform.dart, random_rotation_transform.dart, pca_transform.dart,
index_pre_transform.dart, index_shards.dart:1-144, index_replicas.dart:1-106).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Set

import numpy as np

from .base import Index, Metric, RangeSearchResult, SearchResult, TopK, as_rows, pairwise_scores, select_topk
from .flat import IndexFlat, _RowStore


# ------------------------------------------------------------------------------------------ id map / refine --
class IndexIDMap(Index):
    """Maps the inner index's sequential ids to caller-chosen ids (which must fit in int32)."""

    def __init__(self, inner: Index):
        super().__init__(inner.d, inner.metric)
        self.inner = inner
        self._ext: List[int] = []
        self._reverse: Optional[Dict[int, int]] = None
        self.is_trained, self.ntotal = inner.is_trained, 0

    @property
    def size(self) -> int:
        return len(self._ext)

    def train(self, xs) -> None:
        self.inner.train(xs)
        self.is_trained = self.inner.is_trained

    def add(self, xs) -> None:
        x = as_rows(xs, self.d)
        self.add_with_ids(x, list(range(len(self._ext), len(self._ext) + len(x))))

    def add_with_ids(self, xs, ids: Sequence[int]) -> None:
        x = as_rows(xs, self.d)
        if len(x) != len(ids):
            raise ValueError(f"addWithIds: xs ({len(x)}) and ids ({len(ids)}) length mismatch")
        for i, v in enumerate(ids):
            if not (-0x80000000 <= int(v) <= 0x7FFFFFFF):
                raise ValueError(f"addWithIds: id {v} at position {i} does not fit in int32")
        self.inner.add(x)
        self._ext.extend(int(v) for v in ids)
        self.ntotal, self._reverse = len(self._ext), None

    def id_of(self, i: int) -> int:
        return self._ext[i]

    def internal_of(self, ext: int) -> int:
        if self._reverse is None:
            self._reverse = {e: i for i, e in enumerate(self._ext)}
        return self._reverse.get(ext, -1)

    def _map(self, ids: np.ndarray) -> np.ndarray:
        table = np.asarray(self._ext, dtype=np.int64)
        ok = (ids >= 0) & (ids < len(table))
        out = ids.copy()
        out[ok] = table[ids[ok]]
        return out

    def search(self, queries, k: int) -> SearchResult:
        r = self.inner.search(queries, k)
        return SearchResult(r.distances, self._map(r.ids))

    def range_search(self, queries, radius: float) -> RangeSearchResult:
        r = self.inner.range_search(queries, radius)
        return RangeSearchResult(r.limits, r.distances, self._map(r.ids))

    def remove_ids(self, ids: Set[int]) -> int:
        internal = {self.internal_of(e) for e in ids} - {-1}
        if not internal:
            return 0
        removed = self.inner.remove_ids(internal)
        self._ext = [e for i, e in enumerate(self._ext) if i not in internal]
        self.ntotal, self._reverse = len(self._ext), None
        return removed

    addWithIds, idOf, internalOf, rangeSearch, removeIds = add_with_ids, id_of, internal_of, range_search, remove_ids


class IndexRefineFlat(Index):
    """Approximate ``base`` proposes ``k * k_factor`` candidates that are re-scored exactly against raw vectors."""

    def __init__(self, base: Index, k_factor: int = 4, refine: Optional[IndexFlat] = None):
        super().__init__(base.d, base.metric)
        self.base, self.k_factor = base, k_factor
        self.refine = refine if refine is not None else IndexFlat(base.d, base.metric)
        self.is_trained, self.ntotal = base.is_trained, self.refine.ntotal

    @property
    def kFactor(self):
        return self.k_factor

    def train(self, xs) -> None:
        self.base.train(xs)
        self.is_trained = self.base.is_trained

    def add(self, xs) -> None:
        if not self.is_trained:
            raise RuntimeError("IndexRefineFlat.add before train()")
        x = as_rows(xs, self.d)
        self.base.add(x)
        self.refine.add(x)
        self.ntotal = self.refine.ntotal

    def search(self, queries, k: int) -> SearchResult:
        self._check_k(k)
        if not self.is_trained:
            raise RuntimeError("IndexRefineFlat.search before train()")
        q = as_rows(queries, self.d)
        coarse = self.base.search(q, min(k * self.k_factor, max(self.ntotal, 1)))
        out_d = np.full((len(q), k), np.inf if self.metric == Metric.l2 else -np.inf, dtype=np.float32)
        out_i = np.full((len(q), k), -1, dtype=np.int64)
        for qi in range(len(q)):
            cand = coarse.ids[qi]
            cand = cand[cand >= 0]
            if len(cand):
                s = pairwise_scores(q[qi:qi + 1], self.refine.storage[cand], self.metric)
                dd, ii = select_topk(s, k, self.metric, cand)
                out_d[qi], out_i[qi] = dd[0], ii[0]
        return SearchResult(out_d, out_i)


# --------------------------------------------------------------------------------------------------- binary --
_POPCOUNT8 = np.array([bin(i).count("1") for i in range(256)], dtype=np.uint8)
popcount8_table = _POPCOUNT8


def as_codes(xs, code_size: int) -> np.ndarray:
    a = np.asarray(xs, dtype=np.uint8)
    if a.ndim == 1:
        a = a.reshape(1, -1) if a.size else a.reshape(0, code_size)
    if a.ndim != 2 or a.shape[1] != code_size:
        raise ValueError(f"expected codes of {code_size} bytes, got array of shape {tuple(a.shape)}")
    return np.ascontiguousarray(a)


def hamming_matrix(q: np.ndarray, x: np.ndarray) -> np.ndarray:
    """``[nq, n]`` Hamming distances between packed byte codes."""
    return _POPCOUNT8[q[:, None, :] ^ x[None, :, :]].sum(-1, dtype=np.int32)


def hamming_distance(a, b, b_start: int = 0, code_size: Optional[int] = None) -> int:
    a = np.asarray(a, dtype=np.uint8)
    code_size = len(a) if code_size is None else code_size
    b = np.asarray(b, dtype=np.uint8)[b_start:b_start + code_size]
    return int(_POPCOUNT8[a[:code_size] ^ b].sum())


hammingDistance = hamming_distance


class IndexBinary:
    def __init__(self, code_size: int):
        self.code_size = code_size
        self.ntotal, self.is_trained = 0, True

    @property
    def d(self) -> int:
        return self.code_size * 8

    codeSize = property(lambda self: self.code_size)

    def train(self, xs) -> None:
        self.is_trained = True

    def add(self, xs) -> None:
        raise NotImplementedError

    def search(self, queries, k: int) -> SearchResult:
        raise NotImplementedError


class IndexBinaryFlat(IndexBinary):
    def __init__(self, code_size: int):
        super().__init__(code_size)
        self._codes = _RowStore(code_size, dtype=np.uint8)

    @property
    def codes(self) -> np.ndarray:
        return self._codes.view

    def add(self, xs) -> None:
        self._codes.append(as_codes(xs, self.code_size))
        self.ntotal = self._codes.n

    def reconstruct(self, i: int) -> np.ndarray:
        return self._codes.view[i]

    def search(self, queries, k: int) -> SearchResult:
        q = as_codes(queries, self.code_size)
        return SearchResult(*select_topk(hamming_matrix(q, self.codes).astype(np.float32), k, Metric.l2))


class IndexBinaryIVF(IndexBinary):
    """Binary k-majority clustering (centroid bit = majority vote of its members) + per-cell packed codes."""

    def __init__(self, code_size: int, nlist: int, nprobe: int = 1, kmeans_iters: int = 20, seed: int = 1234):
        super().__init__(code_size)
        self.nlist, self.nprobe, self.kmeans_iters, self.seed = nlist, nprobe, kmeans_iters, seed
        self.quantizer = IndexBinaryFlat(code_size)
        self.is_trained = False
        self._ids: List[List[int]] = [[] for _ in range(nlist)]
        self._codes: List[List[np.ndarray]] = [[] for _ in range(nlist)]

    def list_size(self, c: int) -> int:
        return len(self._ids[c])

    def inv_list_ids(self, c: int) -> List[int]:
        return list(self._ids[c])

    def inv_list_codes(self, c: int) -> np.ndarray:
        return np.concatenate(self._codes[c]) if self._codes[c] else np.zeros((0, self.code_size), np.uint8)

    listSize, invListIds, invListCodes = list_size, inv_list_ids, inv_list_codes

    def io_set_inverted_lists(self, ids, codes, ntotal: int) -> None:
        if len(ids) != self.nlist or len(codes) != self.nlist:
            raise ValueError(f"ioSetInvertedLists: got {len(ids)}/{len(codes)} lists, expected nlist={self.nlist}")
        for c in range(self.nlist):
            cc = np.asarray(codes[c], dtype=np.uint8).reshape(-1)
            if len(cc) != len(ids[c]) * self.code_size:
                raise ValueError(f"ioSetInvertedLists: cell {c} has {len(cc)} code bytes but {len(ids[c])} ids")
            self._ids[c] = [int(i) for i in ids[c]]
            self._codes[c] = [cc.reshape(-1, self.code_size)] if len(cc) else []
        self.ntotal = ntotal

    ioSetInvertedLists = io_set_inverted_lists

    def train(self, xs) -> None:
        x = as_codes(xs, self.code_size)
        if len(x) < self.nlist:
            raise ValueError(f"IndexBinaryIVF.train: need >= nlist={self.nlist} vectors, got {len(x)}")
        rng = np.random.default_rng(self.seed)
        cent = x[rng.choice(len(x), self.nlist, replace=False)].copy()
        bits = np.unpackbits(x, axis=1, bitorder="little").astype(np.int32)
        for _ in range(self.kmeans_iters):
            assign = hamming_matrix(x, cent).argmin(1)
            for c in range(self.nlist):
                members = bits[assign == c]
                if len(members) == 0:
                    cent[c] = x[rng.integers(len(x))]
                else:
                    cent[c] = np.packbits((members.sum(0) * 2 > len(members)).astype(np.uint8), bitorder="little")
        self.quantizer = IndexBinaryFlat(self.code_size)
        self.quantizer.add(cent)
        self.is_trained = True

    def add(self, xs) -> None:
        if not self.is_trained:
            raise RuntimeError("IndexBinaryIVF.add before train()")
        x = as_codes(xs, self.code_size)
        if not len(x):
            return
        cells = hamming_matrix(x, self.quantizer.codes).argmin(1)
        for i, c in enumerate(cells):
            self._ids[int(c)].append(self.ntotal + i)
            self._codes[int(c)].append(x[i:i + 1])
        self.ntotal += len(x)

    def search(self, queries, k: int) -> SearchResult:
        if not self.is_trained:
            raise RuntimeError("IndexBinaryIVF.search before train()")
        q = as_codes(queries, self.code_size)
        probes = self.quantizer.search(q, max(1, min(self.nprobe, self.nlist))).ids
        out_d = np.full((len(q), k), np.inf, dtype=np.float32)
        out_i = np.full((len(q), k), -1, dtype=np.int64)
        for qi in range(len(q)):
            cells = [int(c) for c in probes[qi] if c >= 0 and self._ids[int(c)]]
            if not cells:
                continue
            codes = np.concatenate([self.inv_list_codes(c) for c in cells])
            ids = np.concatenate([np.asarray(self._ids[c], dtype=np.int64) for c in cells])
            dd, ii = select_topk(hamming_matrix(q[qi:qi + 1], codes).astype(np.float32), k, Metric.l2, ids)
            out_d[qi], out_i[qi] = dd[0], ii[0]
        return SearchResult(out_d, out_i)


class IndexLSH(Index):
    """Sign bits of ``nbits`` Gaussian random projections; search ranks by Hamming distance (reported as distance)."""

    def __init__(self, d: int, nbits: int, seed: int = 1234):
        super().__init__(d, Metric.l2)
        self.nbits, self.code_size, self.seed = nbits, (nbits + 7) // 8, seed
        self.projection = np.zeros((nbits, d), dtype=np.float32)
        self.is_trained = False
        self._codes = _RowStore(self.code_size, dtype=np.uint8)

    codeSize = property(lambda self: self.code_size)

    @property
    def codes(self) -> np.ndarray:
        return self._codes.view

    def train(self, xs=None) -> None:
        self.train_projection()

    def train_projection(self) -> None:
        self.projection = np.random.default_rng(self.seed).standard_normal((self.nbits, self.d)).astype(np.float32)
        self.is_trained = True

    trainProjection = train_projection

    def _encode(self, x: np.ndarray) -> np.ndarray:
        bits = (x @ self.projection.T > 0).astype(np.uint8)
        return np.packbits(bits, axis=1, bitorder="little")[:, :self.code_size]

    def add(self, xs) -> None:
        if not self.is_trained:
            self.train_projection()
        x = as_rows(xs, self.d)
        if len(x):
            self._codes.append(self._encode(x))
            self.ntotal = self._codes.n

    def search(self, queries, k: int) -> SearchResult:
        self._check_k(k)
        if not self.is_trained:
            raise RuntimeError("IndexLSH.search before add/train")
        q = self._encode(as_rows(queries, self.d))
        return SearchResult(*select_topk(hamming_matrix(q, self.codes).astype(np.float32), k, Metric.l2))


# ----------------------------------------------------------------------------------------------- transforms --
class VectorTransform:
    def __init__(self, d_in: int, d_out: int):
        self.d_in, self.d_out = d_in, d_out
        self.is_trained = True

    dIn = property(lambda self: self.d_in)
    dOut = property(lambda self: self.d_out)

    def train(self, xs) -> None:
        self.is_trained = True

    def apply(self, xs) -> np.ndarray:
        raise NotImplementedError


class L2NormTransform(VectorTransform):
    def __init__(self, d: int):
        super().__init__(d, d)

    def apply(self, xs) -> np.ndarray:
        x = as_rows(xs, self.d_in)
        n = np.sqrt((x * x).sum(1, keepdims=True))
        return (x / np.where(n > 0, n, 1.0)).astype(np.float32)


class RandomRotationTransform(VectorTransform):
    """Orthonormal ``d x d`` matrix from the QR factorisation of a seeded Gaussian matrix (signs fixed by R's diagonal)."""

    def __init__(self, d: int, seed: int = 1234, matrix: Optional[np.ndarray] = None):
        super().__init__(d, d)
        self.seed = seed
        if matrix is None:
            g = np.random.default_rng(seed).standard_normal((d, d))
            qm, r = np.linalg.qr(g)
            matrix = qm * np.sign(np.where(np.diag(r) == 0, 1.0, np.diag(r)))[None, :]
        self.matrix = np.asarray(matrix, dtype=np.float32).reshape(d, d)

    def apply(self, xs) -> np.ndarray:
        return (as_rows(xs, self.d_in) @ self.matrix.T).astype(np.float32)


def jacobi_eigh(a: np.ndarray, sweeps: int = 64, tol: float = 1e-12):
    """Symmetric eigendecomposition by cyclic Jacobi rotations; eigenvalues descending, eigenvectors as columns
    (the reference's PCA uses the same method)."""
    a = np.array(a, dtype=np.float64)
    n = a.shape[0]
    v = np.eye(n)
    for _ in range(sweeps):
        off = float(np.sqrt((a * a).sum() - (np.diag(a) ** 2).sum()))
        if off < tol:
            break
        for p in range(n - 1):
            for q in range(p + 1, n):
                if abs(a[p, q]) < 1e-300:
                    continue
                theta = (a[q, q] - a[p, p]) / (2.0 * a[p, q])
                if abs(theta) > 1e150:
                    t = 0.5 / theta
                else:
                    t = (1.0 if theta >= 0 else -1.0) / (abs(theta) + math.sqrt(theta * theta + 1.0))
                c = 1.0 / math.sqrt(t * t + 1.0)
                s = t * c
                ap, aq = a[:, p].copy(), a[:, q].copy()
                a[:, p], a[:, q] = c * ap - s * aq, s * ap + c * aq
                ap, aq = a[p, :].copy(), a[q, :].copy()
                a[p, :], a[q, :] = c * ap - s * aq, s * ap + c * aq
                vp, vq = v[:, p].copy(), v[:, q].copy()
                v[:, p], v[:, q] = c * vp - s * vq, s * vp + c * vq
    w = np.diag(a).copy()
    order = np.argsort(-w, kind="stable")
    return w[order], v[:, order]


class PCATransform(VectorTransform):
    """``y = A (x - mean)`` with the top ``d_out`` principal directions scaled by ``eigenvalue ** eigen_power``
    (``-0.5`` whitens)."""

    def __init__(self, d_in: int, d_out: int, eigen_power: float = 0.0):
        super().__init__(d_in, d_out)
        if d_out > d_in:
            raise ValueError("PCATransform: dOut must be <= dIn")
        self.eigen_power = eigen_power
        self.is_trained = False
        self.mean = np.zeros(d_in, dtype=np.float32)
        self.matrix = np.zeros((d_out, d_in), dtype=np.float32)
        self.eigenvalues = np.zeros(d_out, dtype=np.float32)

    def train(self, xs) -> None:
        x = as_rows(xs, self.d_in).astype(np.float64)
        if len(x) < 2:
            raise ValueError("PCATransform.train: need at least 2 vectors")
        self.mean = x.mean(0).astype(np.float32)
        xc = x - x.mean(0)
        w, v = jacobi_eigh(xc.T @ xc / (len(x) - 1))
        w, v = w[:self.d_out], v[:, :self.d_out]
        scale = np.power(np.maximum(w, 1e-12), self.eigen_power) if self.eigen_power != 0.0 else np.ones_like(w)
        self.matrix = (v * scale[None, :]).T.astype(np.float32)
        self.eigenvalues = w.astype(np.float32)
        self.is_trained = True

    @property
    def bias(self) -> np.ndarray:
        """``b`` of the affine form ``y = A x + b``."""
        return (-(self.matrix @ self.mean)).astype(np.float32)

    def apply(self, xs) -> np.ndarray:
        if not self.is_trained:
            raise RuntimeError("PCATransform.apply before train()")
        return ((as_rows(xs, self.d_in) - self.mean) @ self.matrix.T).astype(np.float32)


class IndexPreTransform(Index):
    """Applies a chain of transforms to everything that enters ``inner`` (train, add and query vectors)."""

    def __init__(self, chain: Sequence[VectorTransform], inner: Index):
        if not chain:
            raise ValueError("IndexPreTransform: empty chain")
        super().__init__(chain[0].d_in, inner.metric)
        for a, b in zip(chain, chain[1:]):
            if a.d_out != b.d_in:
                raise ValueError(f"IndexPreTransform: chain mismatch {a.d_out} -> {b.d_in}")
        if chain[-1].d_out != inner.d:
            raise ValueError(f"IndexPreTransform: chain output {chain[-1].d_out} != inner d {inner.d}")
        self.chain, self.inner = list(chain), inner
        self._sync()

    def _sync(self):
        self.is_trained = self.inner.is_trained and all(t.is_trained for t in self.chain)
        self.ntotal = self.inner.ntotal

    def transform(self, xs) -> np.ndarray:
        x = as_rows(xs, self.d)
        for t in self.chain:
            x = t.apply(x)
        return x

    def train(self, xs) -> None:
        x = as_rows(xs, self.d)
        for t in self.chain:
            if not t.is_trained:
                t.train(x)
            x = t.apply(x)
        if not self.inner.is_trained:
            self.inner.train(x)
        self._sync()

    def add(self, xs) -> None:
        self.inner.add(self.transform(xs))
        self._sync()

    def search(self, queries, k: int) -> SearchResult:
        return self.inner.search(self.transform(queries), k)

    def range_search(self, queries, radius: float) -> RangeSearchResult:
        return self.inner.range_search(self.transform(queries), radius)

    def remove_ids(self, ids: Set[int]) -> int:
        n = self.inner.remove_ids(ids)
        self._sync()
        return n

    rangeSearch, removeIds = range_search, remove_ids


# ---------------------------------------------------------------------------------------- shards / replicas --
def _check_family(members: Sequence[Index], who: str, noun: str):
    if not members:
        raise ValueError(f"{who}: need at least one {noun}")
    for i, m in enumerate(members[1:], 1):
        if m.d != members[0].d:
            raise ValueError(f"{who}: {noun} {i} has d={m.d}, expected {members[0].d}")
        if m.metric != members[0].metric:
            raise ValueError(f"{who}: {noun} {i} has metric {m.metric}, expected {members[0].metric}")


class IndexShards(Index):
    """Round-robin placement: external id ``e`` lives in shard ``e % n`` as local id ``e // n``; a query visits every
    shard in turn and merges the per-shard top-k."""

    def __init__(self, shards: Sequence[Index]):
        _check_family(shards, "IndexShards", "shard")
        super().__init__(shards[0].d, shards[0].metric)
        self.shards = tuple(shards)
        self.is_trained = all(s.is_trained for s in shards)
        self.ntotal = sum(s.ntotal for s in shards)

    @property
    def nshards(self) -> int:
        return len(self.shards)

    def train(self, xs) -> None:
        for s in self.shards:
            if not s.is_trained:
                s.train(xs)
        self.is_trained = all(s.is_trained for s in self.shards)

    def add(self, xs) -> None:
        x = as_rows(xs, self.d)
        if not len(x):
            return
        ext = np.arange(self.ntotal, self.ntotal + len(x))
        for s in range(self.nshards):
            part = x[ext % self.nshards == s]
            if len(part):
                self.shards[s].add(part)
        self.ntotal += len(x)

    def search(self, queries, k: int) -> SearchResult:
        self._check_k(k)
        q = as_rows(queries, self.d)
        parts_d, parts_i = [], []
        for s, shard in enumerate(self.shards):
            r = shard.search(q, k)
            parts_d.append(r.distances)
            parts_i.append(np.where(r.ids >= 0, r.ids * self.nshards + s, -1))
        dd, ii = np.concatenate(parts_d, 1), np.concatenate(parts_i, 1)
        pad = np.inf if self.metric == Metric.l2 else -np.inf
        dd = np.where(ii >= 0, dd, pad)
        order = np.argsort(dd if self.metric == Metric.l2 else -dd, axis=1, kind="stable")[:, :k]
        return SearchResult(np.take_along_axis(dd, order, 1), np.take_along_axis(ii, order, 1))


class IndexReplicas(Index):
    """Every replica holds all vectors; successive searches rotate through the replicas."""

    def __init__(self, replicas: Sequence[Index]):
        _check_family(replicas, "IndexReplicas", "replica")
        super().__init__(replicas[0].d, replicas[0].metric)
        self.replicas = tuple(replicas)
        self._next = 0
        self._sync()

    def _sync(self):
        self.ntotal = self.replicas[0].ntotal
        self.is_trained = all(r.is_trained for r in self.replicas)

    @property
    def nreplicas(self) -> int:
        return len(self.replicas)

    def train(self, xs) -> None:
        for r in self.replicas:
            if not r.is_trained:
                r.train(xs)
        self._sync()

    def add(self, xs) -> None:
        x = as_rows(xs, self.d)
        for r in self.replicas:
            r.add(x)
        self.ntotal = self.replicas[0].ntotal

    def search(self, queries, k: int) -> SearchResult:
        chosen = self.replicas[self._next]
        self._next = (self._next + 1) % len(self.replicas)
        return chosen.search(queries, k)
