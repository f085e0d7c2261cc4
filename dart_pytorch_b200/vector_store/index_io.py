"""``FAISDART`` persistence of every index type (reference wire format: lib/core/vector_store/index_io.dart:1-419 and
the ``writeTo`` / ``readFrom`` pair of each index class).

Little-endian.  File header ``'FAISDART' | u32 version=1 | u32 kind``; then the common index header
``u32 d | u32 metric (0 L2, 1 IP) | u32 ntotal | u8 is_trained`` and the type's payload.  Nested indexes are embedded
as complete blobs (magic + version + kind + payload).  Binary indexes use their own header
(``u32 code_size ...``) behind the same file header.
"""
from __future__ import annotations

import io
import os
import struct
from typing import BinaryIO, List, Union

import numpy as np

from .base import Index, Metric
from .composite import (IndexBinary, IndexBinaryFlat, IndexBinaryIVF, IndexIDMap, IndexLSH, IndexPreTransform,
                        IndexRefineFlat, IndexReplicas, IndexShards, L2NormTransform, PCATransform,
                        RandomRotationTransform, VectorTransform)
from .flat import IndexFlat
from .hnsw import IndexHNSW
from .quantized import IndexIVFFlat, IndexIVFPQ, IndexPQ, IndexScalarQuantizer, ProductQuantizer

MAGIC = b"FAISDART"
VERSION = 1


class IndexKind:
    flat, ivf_flat, pq, ivf_pq, hnsw, id_map, scalar_quantizer, refine_flat = 1, 2, 3, 4, 5, 6, 7, 8
    lsh, binary_flat, pre_transform, binary_ivf, shards, replicas = 9, 10, 11, 12, 13, 14


class TransformKind:
    l2_norm, random_rotation, pca = 1, 2, 3


class IoWriter:
    def __init__(self):
        self._b = io.BytesIO()

    def take_bytes(self) -> bytes:
        return self._b.getvalue()

    def u8(self, v): self._b.write(struct.pack("<B", v & 0xFF))
    def u32(self, v): self._b.write(struct.pack("<I", int(v) & 0xFFFFFFFF))
    def i32(self, v): self._b.write(struct.pack("<i", int(v)))
    def f32(self, v): self._b.write(struct.pack("<f", float(v)))
    def i64(self, v): self._b.write(struct.pack("<q", int(v)))
    def raw(self, b: bytes): self._b.write(b)
    def f32s(self, a): self._b.write(np.ascontiguousarray(a, dtype="<f4").tobytes())
    def i32s(self, a): self._b.write(np.ascontiguousarray(a, dtype="<i4").tobytes())
    def u8s(self, a): self._b.write(np.ascontiguousarray(a, dtype=np.uint8).tobytes())


class IoReader:
    def __init__(self, data: bytes):
        self._d = memoryview(data)
        self.pos = 0

    @property
    def remaining(self) -> int:
        return len(self._d) - self.pos

    def _take(self, n: int) -> memoryview:
        if self.pos + n > len(self._d):
            raise ValueError(f"FAISDART: truncated file (wanted {n} bytes at offset {self.pos}, have {self.remaining})")
        out = self._d[self.pos:self.pos + n]
        self.pos += n
        return out

    def u8(self): return struct.unpack("<B", self._take(1))[0]
    def u32(self): return struct.unpack("<I", self._take(4))[0]
    def i32(self): return struct.unpack("<i", self._take(4))[0]
    def f32(self): return struct.unpack("<f", self._take(4))[0]
    def i64(self): return struct.unpack("<q", self._take(8))[0]
    def raw(self, n): return bytes(self._take(n))
    def f32s(self, n): return np.frombuffer(self._take(4 * n), dtype="<f4").astype(np.float32)
    def i32s(self, n): return np.frombuffer(self._take(4 * n), dtype="<i4").astype(np.int64)
    def u8s(self, n): return np.frombuffer(self._take(n), dtype=np.uint8).copy()


def _metric_code(m: Metric) -> int:
    return 0 if m == Metric.l2 else 1


def _metric_from(v: int) -> Metric:
    if v == 0:
        return Metric.l2
    if v == 1:
        return Metric.inner_product
    raise ValueError(f"Unknown metric code {v}")


def _head(w: IoWriter, x: Index, ntotal=None):
    w.u32(x.d)
    w.u32(_metric_code(x.metric))
    w.u32(x.ntotal if ntotal is None else ntotal)
    w.u8(1 if x.is_trained else 0)


def _read_head(r: IoReader):
    return r.u32(), _metric_from(r.u32()), r.u32(), r.u8() != 0


# ---------------------------------------------------------------------------------------------- transforms ----
def _write_transform(w: IoWriter, t: VectorTransform):
    if isinstance(t, L2NormTransform):
        w.u32(TransformKind.l2_norm)
        w.u32(t.d_in)
    elif isinstance(t, RandomRotationTransform):
        w.u32(TransformKind.random_rotation)
        w.u32(t.d_in)
        w.u32(t.seed)
        w.f32s(t.matrix)
    elif isinstance(t, PCATransform):
        w.u32(TransformKind.pca)
        w.u32(t.d_in)
        w.u32(t.d_out)
        w.f32(t.eigen_power)
        w.u8(1 if t.is_trained else 0)
        w.f32s(t.mean)
        w.f32s(t.matrix)
        w.u32(len(t.eigenvalues))
        if len(t.eigenvalues):
            w.f32s(t.eigenvalues)
    else:
        raise TypeError(f"writeIndex: unsupported transform {type(t).__name__}")


def _read_transform(r: IoReader) -> VectorTransform:
    kind = r.u32()
    if kind == TransformKind.l2_norm:
        return L2NormTransform(r.u32())
    if kind == TransformKind.random_rotation:
        d, seed = r.u32(), r.u32()
        return RandomRotationTransform(d, seed=seed, matrix=r.f32s(d * d).reshape(d, d))
    if kind == TransformKind.pca:
        d_in, d_out, power, trained = r.u32(), r.u32(), r.f32(), r.u8() != 0
        t = PCATransform(d_in, d_out, eigen_power=power)
        t.mean = r.f32s(d_in)
        t.matrix = r.f32s(d_out * d_in).reshape(d_out, d_in)
        n = r.u32()
        t.eigenvalues = r.f32s(n) if n else np.zeros(0, np.float32)
        t.is_trained = trained
        return t
    raise ValueError(f"readIndex: unknown transform kind 0x{kind:x}")


# --------------------------------------------------------------------------------------------------- write ----
def _write_pq(w: IoWriter, pq: ProductQuantizer):
    w.u8(1 if pq.is_trained else 0)
    if pq.is_trained:
        w.f32s(pq.codebooks)


def _read_pq(r: IoReader, pq: ProductQuantizer):
    if r.u8() != 0:
        pq.codebooks = r.f32s(pq.m * pq.ksub * pq.dsub).reshape(pq.m, pq.ksub, pq.dsub)
        pq.is_trained = True


def _kind_of(x) -> int:
    table = ((IndexIVFFlat, IndexKind.ivf_flat), (IndexIVFPQ, IndexKind.ivf_pq), (IndexPQ, IndexKind.pq),
             (IndexHNSW, IndexKind.hnsw), (IndexIDMap, IndexKind.id_map),
             (IndexScalarQuantizer, IndexKind.scalar_quantizer), (IndexRefineFlat, IndexKind.refine_flat),
             (IndexLSH, IndexKind.lsh), (IndexPreTransform, IndexKind.pre_transform), (IndexShards, IndexKind.shards),
             (IndexReplicas, IndexKind.replicas), (IndexFlat, IndexKind.flat),
             (IndexBinaryIVF, IndexKind.binary_ivf), (IndexBinaryFlat, IndexKind.binary_flat))
    for cls, kind in table:
        if isinstance(x, cls):
            return kind
    raise TypeError(f"writeIndex: unsupported index type {type(x).__name__}")


def write_child(w: IoWriter, x) -> None:
    w.raw(MAGIC)
    w.u32(VERSION)
    kind = _kind_of(x)
    w.u32(kind)
    _WRITERS[kind](w, x)


def _w_flat(w, x: IndexFlat):
    _head(w, x)
    if x.ntotal:
        w.f32s(x.storage)


def _w_ivf_flat(w, x: IndexIVFFlat):
    _head(w, x)
    for v in (x.nlist, x.nprobe, x.kmeans_iters, x.seed):
        w.u32(v)
    write_child(w, x.quantizer)
    if x.ntotal:
        w.f32s(x.storage)
    for lst in x.inv_lists:
        w.u32(len(lst))
        w.i32s(lst)


def _w_pq(w, x: IndexPQ):
    _head(w, x)
    for v in (x.m, x.pq.nbits, x.pq.kmeans_iters, x.pq.seed):
        w.u32(v)
    _write_pq(w, x.pq)
    if x.ntotal:
        w.u8s(x.codes)


def _w_ivf_pq(w, x: IndexIVFPQ):
    _head(w, x)
    for v in (x.nlist, x.m, x.pq.nbits, x.nprobe, x.kmeans_iters, x.pq_kmeans_iters, x.seed):
        w.u32(v)
    write_child(w, x.quantizer)
    _write_pq(w, x.pq)
    for c in range(x.nlist):
        w.u32(len(x.inv_lists_ids[c]))
        w.i32s(x.inv_lists_ids[c])
        w.u8s(x.cell_codes(c))


def _w_hnsw(w, x: IndexHNSW):
    _head(w, x)
    for v in (x.M, x.ef_construction, x.ef_search, x.seed):
        w.u32(v)
    w.i32(x.entry_point)
    w.i32(x.top_level)
    if x.ntotal:
        w.f32s(x.storage)
    for i in range(x.ntotal):
        w.u32(x.node_level(i))
        for l in range(x.node_level(i) + 1):
            nb = x.node_neighbors(i, l)
            w.u32(len(nb))
            w.i32s(nb)


def _w_id_map(w, x: IndexIDMap):
    _head(w, x)
    write_child(w, x.inner)
    w.u32(x.size)
    w.i32s([x.id_of(i) for i in range(x.size)])


def _w_sq(w, x: IndexScalarQuantizer):
    _head(w, x)
    w.f32s(x.vmin)
    w.f32s(x.scale)
    if x.ntotal:
        w.u8s(x.codes)


def _w_refine(w, x: IndexRefineFlat):
    _head(w, x)
    w.u32(x.k_factor)
    write_child(w, x.base)
    write_child(w, x.refine)


def _w_lsh(w, x: IndexLSH):
    _head(w, x)
    w.u32(x.nbits)
    w.u32(x.seed)
    w.f32s(x.projection)
    if x.ntotal:
        w.u8s(x.codes)


def _w_pre(w, x: IndexPreTransform):
    _head(w, x, ntotal=x.inner.ntotal)
    w.u32(len(x.chain))
    for t in x.chain:
        _write_transform(w, t)
    write_child(w, x.inner)


def _w_family(members_attr):
    def run(w, x):
        _head(w, x)
        members = getattr(x, members_attr)
        w.u32(len(members))
        for m in members:
            write_child(w, m)
    return run


def _w_bin_flat(w, x: IndexBinaryFlat):
    w.u32(x.code_size)
    w.u32(x.ntotal)
    w.u8(1 if x.is_trained else 0)
    if x.ntotal:
        w.u8s(x.codes)


def _w_bin_ivf(w, x: IndexBinaryIVF):
    for v in (x.code_size, x.nlist, x.nprobe, x.ntotal):
        w.u32(v)
    w.u8(1 if x.is_trained else 0)
    for c in range(x.nlist):
        w.u8s(x.quantizer.reconstruct(c) if x.is_trained else np.zeros(x.code_size, np.uint8))
    for c in range(x.nlist):
        ids = x.inv_list_ids(c)
        w.u32(len(ids))
        for i in ids:
            w.u32(i)
        if ids:
            w.u8s(x.inv_list_codes(c))


_WRITERS = {IndexKind.flat: _w_flat, IndexKind.ivf_flat: _w_ivf_flat, IndexKind.pq: _w_pq, IndexKind.ivf_pq: _w_ivf_pq,
            IndexKind.hnsw: _w_hnsw, IndexKind.id_map: _w_id_map, IndexKind.scalar_quantizer: _w_sq,
            IndexKind.refine_flat: _w_refine, IndexKind.lsh: _w_lsh, IndexKind.pre_transform: _w_pre,
            IndexKind.shards: _w_family("shards"), IndexKind.replicas: _w_family("replicas"),
            IndexKind.binary_flat: _w_bin_flat, IndexKind.binary_ivf: _w_bin_ivf}


# ---------------------------------------------------------------------------------------------------- read ----
def _r_flat(r) -> IndexFlat:
    d, metric, ntotal, trained = _read_head(r)
    x = IndexFlat(d, metric)
    if ntotal:
        x.add(r.f32s(ntotal * d).reshape(ntotal, d))
    x.is_trained = trained
    return x


def _expect_flat(x, who: str) -> IndexFlat:
    if not isinstance(x, IndexFlat):
        raise ValueError(f"{who}: embedded quantizer is {type(x).__name__}, expected IndexFlat")
    return x


def _r_ivf_flat(r) -> IndexIVFFlat:
    d, metric, ntotal, trained = _read_head(r)
    nlist, nprobe, iters, seed = r.u32(), r.u32(), r.u32(), r.u32()
    x = IndexIVFFlat(d, nlist, nprobe=nprobe, kmeans_iters=iters, seed=seed, metric=metric)
    x.quantizer = _expect_flat(read_child(r), "IndexIVFFlat")
    storage = r.f32s(ntotal * d).reshape(ntotal, d) if ntotal else np.zeros((0, d), np.float32)
    lists = [r.i32s(r.u32()).tolist() for _ in range(nlist)]
    x.io_set(storage, lists)
    x.is_trained = trained
    return x


def _r_pq(r) -> IndexPQ:
    d, metric, ntotal, trained = _read_head(r)
    m, nbits, iters, seed = r.u32(), r.u32(), r.u32(), r.u32()
    x = IndexPQ(d, m, nbits=nbits, kmeans_iters=iters, seed=seed, metric=metric)
    _read_pq(r, x.pq)
    if ntotal:
        x._codes.append(r.u8s(ntotal * m).reshape(ntotal, m))
    x.ntotal, x.is_trained = ntotal, trained
    return x


def _r_ivf_pq(r) -> IndexIVFPQ:
    d, metric, ntotal, trained = _read_head(r)
    nlist, m, nbits, nprobe, iters, pq_iters, seed = (r.u32() for _ in range(7))
    x = IndexIVFPQ(d, nlist, m, nbits=nbits, nprobe=nprobe, kmeans_iters=iters, pq_kmeans_iters=pq_iters, seed=seed,
                   metric=metric)
    x.quantizer = _expect_flat(read_child(r), "IndexIVFPQ")
    _read_pq(r, x.pq)
    ids, codes = [], []
    for _ in range(nlist):
        n = r.u32()
        ids.append(r.i32s(n).tolist())
        codes.append(r.u8s(n * m))
    x.io_set(ids, codes, ntotal)
    x.is_trained = trained
    return x


def _r_hnsw(r) -> IndexHNSW:
    d, metric, ntotal, trained = _read_head(r)
    M, efc, efs, seed = r.u32(), r.u32(), r.u32(), r.u32()
    entry, top = r.i32(), r.i32()
    x = IndexHNSW(d, M=M, ef_construction=efc, ef_search=efs, seed=seed, metric=metric)
    storage = r.f32s(ntotal * d).reshape(ntotal, d) if ntotal else np.zeros((0, d), np.float32)
    levels, nbrs = [], []
    for _ in range(ntotal):
        level = r.u32()
        levels.append(level)
        nbrs.append([r.i32s(r.u32()).tolist() for _ in range(level + 1)])
    x.io_set(storage, levels, nbrs, entry, top)
    x.is_trained = trained
    return x


def _r_id_map(r) -> IndexIDMap:
    d, metric, ntotal, trained = _read_head(r)
    inner = read_child(r)
    if inner.d != d or inner.metric != metric:
        raise ValueError(f"IndexIDMap: header (d={d}, metric={metric}) disagrees with inner")
    x = IndexIDMap(inner)
    x._ext = r.i32s(r.u32()).tolist()
    x.ntotal, x.is_trained = ntotal, trained
    return x


def _r_sq(r) -> IndexScalarQuantizer:
    d, metric, ntotal, trained = _read_head(r)
    x = IndexScalarQuantizer(d, metric=metric)
    x.vmin, x.scale = r.f32s(d), r.f32s(d)
    if ntotal:
        x._codes.append(r.u8s(ntotal * d).reshape(ntotal, d))
    x.ntotal, x.is_trained = ntotal, trained
    return x


def _r_refine(r) -> IndexRefineFlat:
    d, metric, ntotal, trained = _read_head(r)
    k_factor = r.u32()
    base = read_child(r)
    refine = read_child(r)
    if not isinstance(refine, IndexFlat):
        raise ValueError(f"IndexRefineFlat: embedded refine is {type(refine).__name__}, expected IndexFlat")
    if base.d != d or base.metric != metric:
        raise ValueError(f"IndexRefineFlat: header (d={d}, metric={metric}) disagrees with base")
    x = IndexRefineFlat(base, k_factor=k_factor, refine=refine)
    x.ntotal, x.is_trained = ntotal, trained
    return x


def _r_lsh(r) -> IndexLSH:
    d, _metric, ntotal, trained = _read_head(r)
    nbits, seed = r.u32(), r.u32()
    x = IndexLSH(d, nbits, seed=seed)
    x.projection = r.f32s(nbits * d).reshape(nbits, d)
    if ntotal:
        x._codes.append(r.u8s(ntotal * x.code_size).reshape(ntotal, x.code_size))
    x.ntotal, x.is_trained = ntotal, trained
    return x


def _r_pre(r) -> IndexPreTransform:
    _d, _metric, _ntotal, trained = _read_head(r)
    chain = [_read_transform(r) for _ in range(r.u32())]
    x = IndexPreTransform(chain, read_child(r))
    x.is_trained = trained
    return x


def _r_family(cls):
    def run(r):
        _read_head_vals = _read_head(r)
        members = [read_child(r) for _ in range(r.u32())]
        x = cls(members)
        x.ntotal, x.is_trained = _read_head_vals[2], _read_head_vals[3]
        return x
    return run


def _r_bin_flat(r) -> IndexBinaryFlat:
    code_size, ntotal, trained = r.u32(), r.u32(), r.u8() != 0
    x = IndexBinaryFlat(code_size)
    if ntotal:
        x.add(r.u8s(ntotal * code_size).reshape(ntotal, code_size))
    x.is_trained = trained
    return x


def _r_bin_ivf(r) -> IndexBinaryIVF:
    code_size, nlist, nprobe, ntotal = r.u32(), r.u32(), r.u32(), r.u32()
    trained = r.u8() != 0
    x = IndexBinaryIVF(code_size, nlist, nprobe=nprobe)
    cent = r.u8s(nlist * code_size).reshape(nlist, code_size)
    if trained:
        x.quantizer.add(cent)
    ids, codes = [], []
    for _ in range(nlist):
        n = r.u32()
        ids.append([r.u32() for _ in range(n)])
        codes.append(r.u8s(n * code_size))
    x.io_set_inverted_lists(ids, codes, ntotal)
    x.is_trained = trained
    return x


_READERS = {IndexKind.flat: _r_flat, IndexKind.ivf_flat: _r_ivf_flat, IndexKind.pq: _r_pq, IndexKind.ivf_pq: _r_ivf_pq,
            IndexKind.hnsw: _r_hnsw, IndexKind.id_map: _r_id_map, IndexKind.scalar_quantizer: _r_sq,
            IndexKind.refine_flat: _r_refine, IndexKind.lsh: _r_lsh, IndexKind.pre_transform: _r_pre,
            IndexKind.shards: _r_family(IndexShards), IndexKind.replicas: _r_family(IndexReplicas)}
_BINARY_READERS = {IndexKind.binary_flat: _r_bin_flat, IndexKind.binary_ivf: _r_bin_ivf}


def _read_file_header(r: IoReader) -> int:
    if r.raw(8) != MAGIC:
        raise ValueError("readIndex: bad magic (not a FAISDART file)")
    version = r.u32()
    if version != VERSION:
        raise ValueError(f"readIndex: unsupported version {version}")
    return r.u32()


def read_child(r: IoReader) -> Index:
    kind = _read_file_header(r)
    if kind not in _READERS:
        raise ValueError(f"readIndex: unknown kind 0x{kind:x}")
    return _READERS[kind](r)


# ---- public entry points ------------------------------------------------------------------------------------
def write_index_bytes(x) -> bytes:
    w = IoWriter()
    write_child(w, x)
    return w.take_bytes()


def read_index_bytes(data: bytes) -> Index:
    return read_child(IoReader(data))


def read_binary_index_bytes(data: bytes) -> IndexBinary:
    r = IoReader(data)
    kind = _read_file_header(r)
    if kind not in _BINARY_READERS:
        raise ValueError(f"readBinaryIndex: kind 0x{kind:x} is not a binary index")
    return _BINARY_READERS[kind](r)


def write_index(x, path: str) -> None:
    parent = os.path.dirname(os.path.abspath(path))
    os.makedirs(parent, exist_ok=True)
    with open(path, "wb") as f:
        f.write(write_index_bytes(x))


def read_index(path: str) -> Index:
    with open(path, "rb") as f:
        return read_index_bytes(f.read())


def read_binary_index(path: str) -> IndexBinary:
    with open(path, "rb") as f:
        return read_binary_index_bytes(f.read())


write_binary_index, write_binary_index_bytes = write_index, write_index_bytes
writeIndex, readIndex, writeBinaryIndex, readBinaryIndex = write_index, read_index, write_binary_index, read_binary_index
