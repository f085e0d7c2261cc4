"""FAISS binary-format interop: read and write indexes in the on-disk layout of the C++ / Python FAISS library
(reference: lib/core/vector_store/faiss_io.dart:1-3188; upstream layout: faiss ``index_write`` / ``index_read``).

Little-endian, 64-bit ``size_t`` / ``idx_t``.  Every index starts with a 4-byte fourcc.  Supported: ``IxF2`` / ``IxFI``
(flat), ``IxMp`` / ``IxM2`` (id map), ``IxPT`` (pre-transform) with transforms ``VNrm``, ``rrot``, ``Pcam``; ``IxPq``,
``IxSQ`` (QT_8bit, RS_minmax), ``IxRF``, ``IwFl``, ``IwPQ``, ``IxHe`` (LSH with an inline rectangular ``rrot``),
``IHNf`` (HNSW over flat storage, CSR ``offsets`` / ``neighbors``), and the binary ``IBxF`` / ``IBwF``.  Inverted lists
use the ``ilar`` container in ``full`` or ``sprs`` size layout.  Anything else raises with the offending fourcc.

Common float header: ``i32 d | i64 ntotal | i64 1<<20 | i64 1<<20 | u8 is_trained | i32 metric (0 IP, 1 L2)``.
"""
from __future__ import annotations

import math
import struct
from typing import List, Tuple

import numpy as np

from .base import Index, Metric
from .composite import (IndexBinary, IndexBinaryFlat, IndexBinaryIVF, IndexIDMap, IndexLSH, IndexPreTransform,
                        IndexRefineFlat, L2NormTransform, PCATransform, RandomRotationTransform, VectorTransform)
from .flat import IndexFlat
from .hnsw import IndexHNSW
from .index_io import IoReader, IoWriter
from .quantized import IndexIVFFlat, IndexIVFPQ, IndexPQ, IndexScalarQuantizer, ProductQuantizer


class FaissFourcc:
    @staticmethod
    def of(s: str) -> int:
        if len(s) != 4:
            raise ValueError(f'Fourcc must be 4 chars, got "{s}"')
        return struct.unpack("<I", s.encode("ascii"))[0]

    @staticmethod
    def name(v: int) -> str:
        return struct.pack("<I", v).decode("ascii", errors="replace")


_F = FaissFourcc.of
_DUMMY = 1 << 20


class _W(IoWriter):
    def u64(self, v): self.i64(v)
    def tag(self, s): self.u32(_F(s))

    def vec(self, a, dtype):
        a = np.ascontiguousarray(a, dtype=dtype).reshape(-1)
        self.u64(len(a))
        self.raw(a.tobytes())


class _R(IoReader):
    def u64(self): return self.i64()

    def vec(self, dtype):
        n = self.u64()
        item = np.dtype(dtype).itemsize
        if n < 0 or n * item > self.remaining:
            raise ValueError(f"FAISS: vector of {n} x {item} bytes exceeds the remaining {self.remaining} bytes")
        return np.frombuffer(self.raw(n * item), dtype=dtype).copy()


# ---- headers ------------------------------------------------------------------------------------------------
def _w_header(w: _W, x: Index, ntotal=None):
    w.i32(x.d)
    w.i64(x.ntotal if ntotal is None else ntotal)
    w.i64(_DUMMY)
    w.i64(_DUMMY)
    w.u8(1 if x.is_trained else 0)
    w.i32(1 if x.metric == Metric.l2 else 0)


def _r_header(r: _R):
    d, ntotal = r.i32(), r.i64()
    r.i64()
    r.i64()
    trained, mt = r.u8() != 0, r.i32()
    if mt > 1:
        r.f32()
        raise ValueError(f"FAISS: unsupported metric_type {mt}")
    return d, ntotal, trained, (Metric.l2 if mt == 1 else Metric.inner_product)


# ---- transforms ---------------------------------------------------------------------------------------------
def _w_lt_body(w: _W, have_bias: bool, a, b):
    w.u8(1 if have_bias else 0)
    w.vec(a, "<f4")
    w.vec(b, "<f4")


def _w_vt_tail(w: _W, t: VectorTransform):
    w.i32(t.d_in)
    w.i32(t.d_out)
    w.u8(1 if t.is_trained else 0)


def write_faiss_transform(w: _W, t: VectorTransform) -> None:
    if isinstance(t, L2NormTransform):
        w.tag("VNrm")
        w.f32(2.0)
    elif isinstance(t, RandomRotationTransform):
        w.tag("rrot")
        _w_lt_body(w, False, t.matrix, np.zeros(0, np.float32))
    elif isinstance(t, PCATransform):
        w.tag("Pcam")
        w.f32(t.eigen_power)
        w.f32(0.0)                    # epsilon
        w.u8(0)                       # random_rotation
        w.i32(0)                      # balanced_bins
        w.vec(t.mean, "<f4")
        w.vec(t.eigenvalues, "<f4")
        w.vec(np.zeros(0, np.float32), "<f4")          # full eigenbasis is not retained
        _w_lt_body(w, True, t.matrix, t.bias)
    else:
        raise NotImplementedError(f"writeFaissTransform: {type(t).__name__} not yet supported.")
    _w_vt_tail(w, t)


def read_faiss_transform(r: _R) -> VectorTransform:
    tag = r.u32()
    name = FaissFourcc.name(tag)
    if name == "VNrm":
        norm = r.f32()
        d_in, d_out, _ = r.i32(), r.i32(), r.u8()
        if norm != 2.0 or d_in != d_out:
            raise ValueError(f"VNrm: only the L2 norm on equal widths is supported (norm={norm})")
        return L2NormTransform(d_in)
    if name == "rrot":
        _have_bias = r.u8()
        a, _b = r.vec("<f4"), r.vec("<f4")
        d_in, d_out, trained = r.i32(), r.i32(), r.u8() != 0
        if d_in != d_out or len(a) != d_in * d_in:
            raise ValueError(f"rrot: expected a square {d_in}x{d_in} matrix, got {len(a)} floats")
        t = RandomRotationTransform(d_in, matrix=a.reshape(d_in, d_in))
        t.is_trained = trained
        return t
    if name in ("Pcam", "PCAm"):
        power = r.f32()
        r.f32()
        r.u8()
        r.i32()
        mean, eig, _pcamat = r.vec("<f4"), r.vec("<f4"), r.vec("<f4")
        _have_bias = r.u8()
        a, _b = r.vec("<f4"), r.vec("<f4")
        d_in, d_out, trained = r.i32(), r.i32(), r.u8() != 0
        if len(a) != d_in * d_out:
            raise ValueError(f"Pcam: A has {len(a)} floats, expected {d_in * d_out}.")
        if len(mean) != d_in:
            raise ValueError(f"Pcam: mean has {len(mean)} floats, expected {d_in}.")
        t = PCATransform(d_in, d_out, eigen_power=float(power))
        t.mean, t.matrix, t.eigenvalues, t.is_trained = mean, a.reshape(d_out, d_in), eig[:d_out], trained
        return t
    raise ValueError(f'readFaissTransform: unsupported transform fourcc "{name}"')


# ---- shared payloads ----------------------------------------------------------------------------------------
def _w_pq(w: _W, pq: ProductQuantizer):
    w.u64(pq.d)
    w.u64(pq.m)
    w.u64(pq.nbits)
    w.vec(pq.codebooks, "<f4")


def _r_pq(r: _R) -> ProductQuantizer:
    d, m, nbits = r.u64(), r.u64(), r.u64()
    cent = r.vec("<f4")
    pq = ProductQuantizer(d, m, nbits)
    if len(cent) != m * pq.ksub * pq.dsub:
        raise ValueError(f"ProductQuantizer: {len(cent)} centroid floats, expected {m * pq.ksub * pq.dsub}")
    pq.codebooks, pq.is_trained = cent.reshape(m, pq.ksub, pq.dsub), True
    return pq


def _w_direct_map_none(w: _W):
    w.u8(0)
    w.vec(np.zeros(0, np.int64), "<i8")


def _r_direct_map(r: _R):
    kind = r.u8()
    if kind != 0:
        raise NotImplementedError(f"DirectMap: only NoMap (type=0) supported, got type={kind}")
    if len(r.vec("<i8")):
        raise ValueError("DirectMap: NoMap should carry an empty array")


def _w_inv_lists(w: _W, nlist: int, code_size: int, codes: List[np.ndarray], ids: List[np.ndarray]):
    w.tag("ilar")
    w.u64(nlist)
    w.u64(code_size)
    sizes = [len(i) for i in ids]
    nonempty = sum(1 for s in sizes if s)
    if nonempty * 2 < nlist:                       # upstream picks the sparse layout when most lists are empty
        w.tag("sprs")
        pairs = [v for c, s in enumerate(sizes) if s for v in (c, s)]
        w.vec(pairs, "<u8")
    else:
        w.tag("full")
        w.vec(sizes, "<u8")
    for c in range(nlist):
        if sizes[c]:
            w.raw(np.ascontiguousarray(codes[c], dtype=np.uint8).tobytes())
            w.raw(np.ascontiguousarray(ids[c], dtype="<i8").tobytes())


def _r_inv_lists(r: _R) -> Tuple[int, int, List[np.ndarray], List[np.ndarray]]:
    tag = FaissFourcc.name(r.u32())
    if tag == "il00":
        return 0, 0, [], []
    if tag != "ilar":
        raise ValueError(f'InvertedLists: unsupported container fourcc "{tag}"')
    nlist, code_size = r.u64(), r.u64()
    layout = FaissFourcc.name(r.u32())
    sizes = [0] * nlist
    if layout == "full":
        v = r.vec("<u8")
        if len(v) != nlist:
            raise ValueError(f"ilar/full: {len(v)} sizes for nlist={nlist}")
        sizes = [int(s) for s in v]
    elif layout == "sprs":
        v = r.vec("<u8")
        for c, s in zip(v[0::2], v[1::2]):
            sizes[int(c)] = int(s)
    else:
        raise ValueError(f'ilar: unknown list_type "{layout}"')
    codes, ids = [], []
    for s in sizes:
        codes.append(np.frombuffer(r.raw(s * code_size), dtype=np.uint8).copy())
        ids.append(np.frombuffer(r.raw(s * 8), dtype="<i8").astype(np.int64))
    return nlist, code_size, codes, ids


def _hnsw_default_probas(M: int, level_mult: float):
    probas, cum, nn, level = [], [0], 0, 0
    while True:
        p = math.exp(-level / level_mult) * (1 - math.exp(-1 / level_mult))
        if p < 1e-9:
            break
        probas.append(p)
        nn += M * 2 if level == 0 else M
        cum.append(nn)
        level += 1
    return probas, cum


# ---- writers ------------------------------------------------------------------------------------------------
def _write(w: _W, x) -> None:
    if isinstance(x, IndexIVFFlat):
        w.tag("IwFl")
        _w_header(w, x)
        w.u64(x.nlist)
        w.u64(x.nprobe)
        _write(w, x.quantizer)
        _w_direct_map_none(w)
        ids = [np.asarray(l, dtype=np.int64) for l in x.inv_lists]
        codes = [np.ascontiguousarray(x.storage[i], dtype="<f4").view(np.uint8).reshape(-1) for i in ids]
        _w_inv_lists(w, x.nlist, x.d * 4, codes, ids)
    elif isinstance(x, IndexIVFPQ):
        w.tag("IwPQ")
        _w_header(w, x)
        w.u64(x.nlist)
        w.u64(x.nprobe)
        _write(w, x.quantizer)
        _w_direct_map_none(w)
        w.u8(1)                                    # by_residual
        w.u64(x.m)                                 # code_size (nbits <= 8: one byte per sub-quantizer)
        _w_pq(w, x.pq)
        _w_inv_lists(w, x.nlist, x.m, [x.cell_codes(c).reshape(-1) for c in range(x.nlist)],
                     [np.asarray(l, dtype=np.int64) for l in x.inv_lists_ids])
    elif isinstance(x, IndexPQ):
        w.tag("IxPq")
        _w_header(w, x)
        _w_pq(w, x.pq)
        w.vec(x.codes, np.uint8)
        w.i32(0)                                   # search_type = ST_PQ
        w.u8(0)                                    # encode_signs
        w.i32(0)                                   # polysemous_ht
    elif isinstance(x, IndexScalarQuantizer):
        w.tag("IxSQ")
        _w_header(w, x)
        w.i32(0)                                   # QT_8bit
        w.i32(0)                                   # RS_minmax
        w.f32(0.0)
        w.u64(x.d)
        w.u64(x.d)
        w.vec(np.concatenate([x.vmin, x.scale]), "<f4")
        w.vec(x.codes, np.uint8)
    elif isinstance(x, IndexRefineFlat):
        w.tag("IxRF")
        _w_header(w, x)
        _write(w, x.base)
        _write(w, x.refine)
        w.f32(float(x.k_factor))
    elif isinstance(x, IndexIDMap):
        w.tag("IxMp")
        _w_header(w, x)
        _write(w, x.inner)
        w.vec([x.id_of(i) for i in range(x.size)], "<i8")
    elif isinstance(x, IndexPreTransform):
        w.tag("IxPT")
        _w_header(w, x, ntotal=x.inner.ntotal)
        w.i32(len(x.chain))
        for t in x.chain:
            write_faiss_transform(w, t)
        _write(w, x.inner)
    elif isinstance(x, IndexLSH):
        w.tag("IxHe")
        _w_header(w, x)
        w.i32(x.nbits)
        w.u8(1)                                    # rotate_data
        w.u8(0)                                    # train_thresholds
        w.vec(np.zeros(0, np.float32), "<f4")
        w.i32(x.code_size)
        w.tag("rrot")
        _w_lt_body(w, False, x.projection, np.zeros(0, np.float32))
        w.i32(x.d)
        w.i32(x.nbits)
        w.u8(1 if x.is_trained else 0)
        w.vec(x.codes, np.uint8)
    elif isinstance(x, IndexHNSW):
        w.tag("IHNf")
        _w_header(w, x)
        probas, cum = _hnsw_default_probas(x.M, 1.0 / math.log(x.M))
        while len(cum) < max(x.top_level + 1, 0) + 1:
            cum.append(cum[-1] + x.M)
        n = x.ntotal
        levels = [x.node_level(i) + 1 for i in range(n)]
        offsets = np.zeros(n + 1, dtype=np.int64)
        for i in range(n):
            offsets[i + 1] = offsets[i] + cum[levels[i]]
        nbrs = np.full(int(offsets[n]), -1, dtype=np.int32)
        for i in range(n):
            for l in range(levels[i]):
                adj = x.node_neighbors(i, l)
                lo, hi = int(offsets[i]) + cum[l], int(offsets[i]) + cum[l + 1]
                if len(adj) > hi - lo:
                    raise RuntimeError(f"HNSW node {i} layer {l} has {len(adj)} neighbors, but slot budget is {hi - lo}")
                nbrs[lo:lo + len(adj)] = adj
        w.vec(probas, "<f8")
        w.vec(cum, "<i4")
        w.vec(levels, "<i4")
        w.vec(offsets, "<u8")
        w.vec(nbrs, "<i4")
        for v in (x.entry_point, x.top_level, x.ef_construction, x.ef_search, 1):
            w.i32(v)
        storage = IndexFlat(x.d, x.metric)
        if n:
            storage.add(x.storage)
        _write(w, storage)
    elif isinstance(x, IndexFlat):
        w.tag("IxF2" if x.metric == Metric.l2 else "IxFI")
        _w_header(w, x)
        w.vec(x.storage, "<f4")
    else:
        raise NotImplementedError(f"writeFaissIndex: {type(x).__name__} not yet supported.")


def _w_binary_header(w: _W, x: IndexBinary):
    w.i32(x.d)
    w.i32(x.code_size)
    w.i64(x.ntotal)
    w.u8(1 if x.is_trained else 0)
    w.i32(1)


def _write_binary(w: _W, x: IndexBinary) -> None:
    if isinstance(x, IndexBinaryIVF):
        w.tag("IBwF")
        _w_binary_header(w, x)
        w.u64(x.nlist)
        w.u64(x.nprobe)
        _write_binary(w, x.quantizer)
        _w_direct_map_none(w)
        _w_inv_lists(w, x.nlist, x.code_size, [x.inv_list_codes(c).reshape(-1) for c in range(x.nlist)],
                     [np.asarray(x.inv_list_ids(c), dtype=np.int64) for c in range(x.nlist)])
    elif isinstance(x, IndexBinaryFlat):
        w.tag("IBxF")
        _w_binary_header(w, x)
        w.vec(x.codes, np.uint8)
    else:
        raise NotImplementedError(f"writeFaissBinaryIndex: {type(x).__name__} not yet supported.")


# ---- readers ------------------------------------------------------------------------------------------------
def _read(r: _R) -> Index:
    name = FaissFourcc.name(r.u32())
    if name in ("IxF2", "IxFI", "IxFl"):
        d, ntotal, trained, metric = _r_header(r)
        if name != "IxFl":
            metric = Metric.l2 if name == "IxF2" else Metric.inner_product
        xb = r.vec("<f4")
        if len(xb) != ntotal * d:
            raise ValueError(f"{name}: {len(xb)} floats for ntotal={ntotal}, d={d}")
        x = IndexFlat(d, metric)
        if ntotal:
            x.add(xb.reshape(ntotal, d))
        x.is_trained = trained
        return x
    if name in ("IxMp", "IxM2"):
        d, ntotal, trained, metric = _r_header(r)
        x = IndexIDMap(_read(r))
        ids = r.vec("<i8")
        x._ext = [int(i) for i in ids]
        x.ntotal, x.is_trained = len(ids), trained
        return x
    if name == "IxPT":
        _d, _ntotal, trained, _metric = _r_header(r)
        chain = [read_faiss_transform(r) for _ in range(r.i32())]
        x = IndexPreTransform(chain, _read(r))
        x.is_trained = trained
        return x
    if name == "IxPq":
        d, ntotal, trained, metric = _r_header(r)
        pq = _r_pq(r)
        codes = r.vec(np.uint8)
        r.i32()
        r.u8()
        r.i32()
        x = IndexPQ(d, pq.m, nbits=pq.nbits, metric=metric)
        x.pq = pq
        if ntotal:
            x._codes.append(codes.reshape(ntotal, pq.m))
        x.ntotal, x.is_trained = ntotal, trained
        return x
    if name == "IxSQ":
        d, ntotal, trained, metric = _r_header(r)
        qtype, rangestat = r.i32(), r.i32()
        r.f32()
        sq_d, _code_size = r.u64(), r.u64()
        t = r.vec("<f4")
        if qtype != 0:
            raise NotImplementedError(f"IxSQ: only QT_8bit (qtype=0) is supported, got qtype={qtype}.")
        if len(t) != 2 * sq_d:
            raise ValueError(f"IxSQ: trained has {len(t)} floats, expected {2 * sq_d}")
        x = IndexScalarQuantizer(d, metric=metric)
        x.vmin, x.scale = t[:d].astype(np.float32), t[d:].astype(np.float32)
        codes = r.vec(np.uint8)
        if ntotal:
            x._codes.append(codes.reshape(ntotal, d))
        x.ntotal, x.is_trained = ntotal, trained
        return x
    if name == "IxRF":
        d, ntotal, trained, metric = _r_header(r)
        base, refine = _read(r), _read(r)
        if not isinstance(refine, IndexFlat):
            raise ValueError(f"IxRF: refine index is {type(refine).__name__}, expected IndexFlat")
        x = IndexRefineFlat(base, k_factor=max(1, int(round(r.f32()))), refine=refine)
        x.ntotal, x.is_trained = ntotal, trained
        return x
    if name in ("IwFl", "IwPQ"):
        d, ntotal, trained, metric = _r_header(r)
        nlist, nprobe = r.u64(), r.u64()
        quantizer = _read(r)
        if not isinstance(quantizer, IndexFlat):
            raise ValueError(f"{name}: coarse quantizer is {type(quantizer).__name__}, expected IndexFlat")
        _r_direct_map(r)
        if name == "IwFl":
            _, code_size, codes, ids = _r_inv_lists(r)
            if code_size != d * 4:
                raise ValueError(f"IwFl: code_size {code_size} != 4 * d ({4 * d})")
            x = IndexIVFFlat(d, nlist, nprobe=nprobe, metric=metric)
            x.quantizer = quantizer
            storage = np.zeros((ntotal, d), dtype=np.float32)
            for c in range(nlist):
                if len(ids[c]):
                    if ids[c].min() < 0 or ids[c].max() >= ntotal:
                        raise ValueError(f"IwFl: list {c} holds ids outside [0, {ntotal})")
                    storage[ids[c]] = codes[c].view("<f4").reshape(-1, d)
            x.io_set(storage, [i.tolist() for i in ids])
        else:
            by_residual, code_size = r.u8(), r.u64()
            pq = _r_pq(r)
            if not by_residual:
                raise NotImplementedError("IwPQ: only by_residual=1 is supported")
            _, _, codes, ids = _r_inv_lists(r)
            x = IndexIVFPQ(d, nlist, pq.m, nbits=pq.nbits, nprobe=nprobe, metric=metric)
            x.quantizer, x.pq = quantizer, pq
            x.io_set([i.tolist() for i in ids], codes, ntotal)
        x.is_trained = trained
        return x
    if name == "IxHe":
        d, ntotal, trained, _metric = _r_header(r)
        nbits, rotate, train_thr = r.i32(), r.u8(), r.u8()
        r.vec("<f4")
        r.i32()
        if FaissFourcc.name(r.u32()) != "rrot":
            raise ValueError("IxHe: expected an inline rrot transform")
        r.u8()
        a, _b = r.vec("<f4"), r.vec("<f4")
        d_in, d_out, _t = r.i32(), r.i32(), r.u8()
        if not rotate or train_thr:
            raise NotImplementedError("IxHe: only rotate_data=1, train_thresholds=0 is supported")
        if d_in != d or d_out != nbits or len(a) != nbits * d:
            raise ValueError(f"IxHe: projection is {len(a)} floats, expected {nbits} x {d}")
        x = IndexLSH(d, nbits)
        x.projection = a.reshape(nbits, d)
        codes = r.vec(np.uint8)
        if ntotal:
            x._codes.append(codes.reshape(ntotal, x.code_size))
        x.ntotal, x.is_trained = ntotal, trained
        return x
    if name == "IHNf":
        d, ntotal, trained, metric = _r_header(r)
        probas, cum, levels = r.vec("<f8"), r.vec("<i4"), r.vec("<i4")
        offsets, nbrs = r.vec("<u8"), r.vec("<i4")
        entry, top, efc, efs, _beam = (r.i32() for _ in range(5))
        if len(cum) == 0 or cum[0] != 0:
            raise ValueError("IHNf: cum_nneighbor_per_level must start with 0")
        if len(probas) + 1 != len(cum):
            raise ValueError("IHNf: assign_probas length inconsistent with cum_nneighbor_per_level")
        if len(levels) != ntotal or len(offsets) != ntotal + 1:
            raise ValueError("IHNf: levels / offsets do not match ntotal")
        m0 = int(cum[1]) if len(cum) >= 2 else 0
        M = max(2, m0 // 2)
        storage = _read(r)
        if not isinstance(storage, IndexFlat):
            raise ValueError(f"IHNf: storage index is {type(storage).__name__}, expected IndexFlat")
        x = IndexHNSW(d, M=M, ef_construction=efc, ef_search=efs, metric=metric)
        per_node = []
        for i in range(ntotal):
            layers = []
            for l in range(int(levels[i])):
                lo, hi = int(offsets[i]) + int(cum[l]), int(offsets[i]) + int(cum[l + 1])
                layers.append([int(v) for v in nbrs[lo:hi] if v >= 0])
            per_node.append(layers)
        x.io_set(storage.storage, [int(l) - 1 for l in levels], per_node, entry, top)
        x.is_trained = trained
        return x
    raise ValueError(f'readFaissIndex: unsupported index fourcc "{name}"')


def _r_binary_header(r: _R):
    d, code_size, ntotal, trained, _metric = r.i32(), r.i32(), r.i64(), r.u8() != 0, r.i32()
    if d != code_size * 8:
        raise ValueError(f"binary header: d={d} != 8 * code_size ({code_size})")
    return code_size, ntotal, trained


def _read_binary(r: _R) -> IndexBinary:
    name = FaissFourcc.name(r.u32())
    if name == "IBxF":
        code_size, ntotal, trained = _r_binary_header(r)
        xb = r.vec(np.uint8)
        x = IndexBinaryFlat(code_size)
        if ntotal:
            x.add(xb.reshape(ntotal, code_size))
        x.is_trained = trained
        return x
    if name == "IBwF":
        code_size, ntotal, trained = _r_binary_header(r)
        nlist, nprobe = r.u64(), r.u64()
        quantizer = _read_binary(r)
        _r_direct_map(r)
        _, _, codes, ids = _r_inv_lists(r)
        x = IndexBinaryIVF(code_size, nlist, nprobe=nprobe)
        x.quantizer = quantizer
        x.io_set_inverted_lists([i.tolist() for i in ids], codes, ntotal)
        x.is_trained = trained
        return x
    raise ValueError(f'readFaissBinaryIndex: unsupported index fourcc "{name}"')


# ---- public entry points ------------------------------------------------------------------------------------
def write_faiss_index_bytes(x: Index) -> bytes:
    w = _W()
    _write(w, x)
    return w.take_bytes()


def read_faiss_index_bytes(data: bytes) -> Index:
    return _read(_R(data))


def write_faiss_binary_index_bytes(x: IndexBinary) -> bytes:
    w = _W()
    _write_binary(w, x)
    return w.take_bytes()


def read_faiss_binary_index_bytes(data: bytes) -> IndexBinary:
    return _read_binary(_R(data))


def write_faiss_index(x: Index, path: str) -> None:
    with open(path, "wb") as f:
        f.write(write_faiss_index_bytes(x))


def read_faiss_index(path: str) -> Index:
    with open(path, "rb") as f:
        return read_faiss_index_bytes(f.read())


def write_faiss_binary_index(x: IndexBinary, path: str) -> None:
    with open(path, "wb") as f:
        f.write(write_faiss_binary_index_bytes(x))


def read_faiss_binary_index(path: str) -> IndexBinary:
    with open(path, "rb") as f:
        return read_faiss_binary_index_bytes(f.read())


def faiss_describe(data: bytes) -> str:
    """One line per nested index: fourcc, d, ntotal, metric (the ``faiss_describe`` tool's summary)."""
    x = read_faiss_index_bytes(data)
    lines = []

    def walk(ix, depth):
        lines.append(f"{'  ' * depth}{type(ix).__name__} d={ix.d} ntotal={ix.ntotal} metric={ix.metric.name} "
                     f"trained={ix.is_trained}")
        for attr in ("inner", "base", "refine", "quantizer"):
            child = getattr(ix, attr, None)
            if isinstance(child, Index):
                walk(child, depth + 1)
    walk(x, 0)
    return "\n".join(lines)


def faiss_strip(data: bytes) -> bytes:
    """Re-encode an index with its vectors removed but training state kept (the ``faiss_strip`` tool): flat stores are
    emptied, trained quantizers and transforms survive."""
    x = read_faiss_index_bytes(data)

    def strip(ix):
        if isinstance(ix, IndexPreTransform):
            return IndexPreTransform(ix.chain, strip(ix.inner))
        if isinstance(ix, IndexIDMap):
            return IndexIDMap(strip(ix.inner))
        if isinstance(ix, IndexIVFFlat):
            y = IndexIVFFlat(ix.d, ix.nlist, nprobe=ix.nprobe, metric=ix.metric)
            y.quantizer, y.is_trained = ix.quantizer, ix.is_trained
            return y
        if isinstance(ix, IndexIVFPQ):
            y = IndexIVFPQ(ix.d, ix.nlist, ix.m, nbits=ix.pq.nbits, nprobe=ix.nprobe, metric=ix.metric)
            y.quantizer, y.pq, y.is_trained = ix.quantizer, ix.pq, ix.is_trained
            return y
        if isinstance(ix, IndexPQ):
            y = IndexPQ(ix.d, ix.m, nbits=ix.pq.nbits, metric=ix.metric)
            y.pq, y.is_trained = ix.pq, ix.is_trained
            return y
        if isinstance(ix, IndexScalarQuantizer):
            y = IndexScalarQuantizer(ix.d, metric=ix.metric)
            y.vmin, y.scale, y.is_trained = ix.vmin, ix.scale, ix.is_trained
            return y
        if isinstance(ix, IndexFlat):
            return IndexFlat(ix.d, ix.metric)
        raise NotImplementedError(f"faissStrip: {type(ix).__name__} not supported")
    return write_faiss_index_bytes(strip(x))


writeFaissIndex, readFaissIndex = write_faiss_index, read_faiss_index
writeFaissBinaryIndex, readFaissBinaryIndex = write_faiss_binary_index, read_faiss_binary_index
# the reference's names for the file / byte entry points
saveFaissIndex, loadFaissIndex = write_faiss_index, read_faiss_index
saveFaissBinaryIndex, loadFaissBinaryIndex = write_faiss_binary_index, read_faiss_binary_index
writeFaissIndexToBytes, readFaissIndexFromBytes = write_faiss_index_bytes, read_faiss_index_bytes
writeFaissBinaryIndexToBytes, readFaissBinaryIndexFromBytes = (write_faiss_binary_index_bytes,
                                                               read_faiss_binary_index_bytes)
FaissFourcc.toStr = FaissFourcc.name
