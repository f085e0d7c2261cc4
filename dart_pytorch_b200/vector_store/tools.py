"""Index factory strings, flat -> approximate conversions, benchmark harness and parameter auto-tuning
(reference: lib/core/vector_store/index_factory.dart:39-167, index_convert.dart:1-233, bench.dart:1-400,
auto_tune.dart:1-425).
"""
from __future__ import annotations

import re
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import numpy as np

from .base import Index, Metric, SearchResult, as_rows
from .composite import (IndexLSH, IndexPreTransform, IndexRefineFlat, L2NormTransform, PCATransform,
                        RandomRotationTransform, VectorTransform)
from .flat import IndexFlat
from .hnsw import IndexHNSW
from .quantized import IndexIVFFlat, IndexIVFPQ, IndexPQ, IndexScalarQuantizer


# --------------------------------------------------------------------------------------------------- factory --
def _parse_transform(tok: str, d_in: int) -> Optional[VectorTransform]:
    if tok == "L2Norm":
        return L2NormTransform(d_in)
    if tok == "RR":
        return RandomRotationTransform(d_in)
    m = re.fullmatch(r"PCA(W?)(\d+)", tok)
    if m:
        return PCATransform(d_in, int(m.group(2)), eigen_power=-0.5 if m.group(1) == "W" else 0.0)
    return None


def _pq_args(tok: str):
    m = re.fullmatch(r"PQ(\d+)(?:x(\d+))?", tok)
    return None if m is None else (int(m.group(1)), int(m.group(2)) if m.group(2) else 8)


def _parse_index(d: int, tokens: List[str], metric: Metric) -> Index:
    head = tokens[0]

    def alone(name):
        if len(tokens) != 1:
            raise ValueError(f"indexFactory: {name} takes no trailing tokens (got {tokens})")
    if head == "Flat":
        alone("Flat")
        return IndexFlat(d, metric)
    if head == "SQ8":
        alone("SQ8")
        return IndexScalarQuantizer(d, metric=metric)
    m = re.fullmatch(r"HNSW(\d+)", head)
    if m:
        alone("HNSW")
        return IndexHNSW(d, M=int(m.group(1)), metric=metric)
    m = re.fullmatch(r"LSH(\d+)", head)
    if m:
        alone("LSH")
        return IndexLSH(d, int(m.group(1)))
    pq = _pq_args(head)
    if pq:
        alone("PQ")
        return IndexPQ(d, pq[0], nbits=pq[1], metric=metric)
    m = re.fullmatch(r"IVF(\d+)", head)
    if m:
        if len(tokens) != 2:
            raise ValueError(f"indexFactory: IVF must be followed by Flat or PQ (got {tokens})")
        nlist = int(m.group(1))
        if tokens[1] == "Flat":
            return IndexIVFFlat(d, nlist, metric=metric)
        pq = _pq_args(tokens[1])
        if pq:
            return IndexIVFPQ(d, nlist, pq[0], nbits=pq[1], metric=metric)
        raise ValueError(f'indexFactory: unknown IVF tail "{tokens[1]}"')
    raise ValueError(f'indexFactory: unknown index specifier "{head}" in {tokens}')


def index_factory(d: int, description: str, metric: Metric = Metric.l2) -> Index:
    """``"PCA32,IVF64,Flat"``-style strings: leading transforms (``L2Norm``, ``RR``, ``PCA<n>``, ``PCAW<n>``) then one
    of ``Flat``, ``SQ8``, ``HNSW<M>``, ``LSH<bits>``, ``PQ<m>[x<bits>]``, ``IVF<nlist>,Flat``, ``IVF<nlist>,PQ<m>[x<bits>]``."""
    tokens = [t.strip() for t in description.split(",") if t.strip()]
    if not tokens:
        raise ValueError("indexFactory: empty description")
    chain: List[VectorTransform] = []
    cur = d
    while tokens:
        tr = _parse_transform(tokens[0], cur)
        if tr is None:
            break
        chain.append(tr)
        cur = tr.d_out
        tokens.pop(0)
    if not tokens:
        raise ValueError(f'indexFactory: no index specifier in "{description}"')
    inner = _parse_index(cur, tokens, metric)
    return IndexPreTransform(chain, inner) if chain else inner


indexFactory = index_factory


# ----------------------------------------------------------------------------------------------- conversions --
def reconstruct_all(src: IndexFlat) -> np.ndarray:
    return np.array(src.storage, copy=True)


def _auto_nlist(ntotal: int) -> int:
    k = 1
    while k * k < ntotal:
        k += 1
    return max(1, k)


def _subsample(x: np.ndarray, cap: Optional[int], seed: int) -> np.ndarray:
    if cap is None or cap >= len(x):
        return x
    return x[np.random.default_rng(seed).permutation(len(x))[:cap]]


def flat_to_ivf_flat(src: IndexFlat, nlist: Optional[int] = None, nprobe: Optional[int] = None,
                     train_size: Optional[int] = None, kmeans_iters: int = 20, seed: int = 1234) -> IndexIVFFlat:
    if src.ntotal == 0:
        raise ValueError("flatToIvfFlat: source index is empty")
    k = nlist or _auto_nlist(src.ntotal)
    x = reconstruct_all(src)
    ivf = IndexIVFFlat(src.d, k, nprobe=nprobe or min(k, 8), kmeans_iters=kmeans_iters, seed=seed, metric=src.metric)
    ivf.train(_subsample(x, train_size, seed))
    ivf.add(x)
    return ivf


def flat_to_ivf_pq(src: IndexFlat, m: int, nbits: int = 8, nlist: Optional[int] = None,
                   nprobe: Optional[int] = None, train_size: Optional[int] = None, seed: int = 1234) -> IndexIVFPQ:
    if src.ntotal == 0:
        raise ValueError("flatToIvfPq: source index is empty")
    if src.d % m:
        raise ValueError(f"flatToIvfPq: d={src.d} not divisible by m={m}")
    k = nlist or _auto_nlist(src.ntotal)
    x = reconstruct_all(src)
    ivf = IndexIVFPQ(src.d, k, m, nbits=nbits, nprobe=nprobe or min(k, 8), seed=seed, metric=src.metric)
    ivf.train(_subsample(x, train_size, seed))
    ivf.add(x)
    return ivf


def flat_to_hnsw(src: IndexFlat, M: int = 16, ef_construction: int = 100, ef_search: int = 32,
                 seed: int = 1234) -> IndexHNSW:
    h = IndexHNSW(src.d, M=M, ef_construction=ef_construction, ef_search=ef_search, seed=seed, metric=src.metric)
    h.add(reconstruct_all(src))
    return h


def wrap_with_refine(base: Index, src: IndexFlat, k_factor: int = 4) -> IndexRefineFlat:
    if base.d != src.d:
        raise ValueError(f"wrapWithRefine: base.d={base.d} != src.d={src.d}")
    if base.metric != src.metric:
        raise ValueError("wrapWithRefine: metric mismatch")
    if base.ntotal != src.ntotal:
        raise ValueError(f"wrapWithRefine: base.ntotal={base.ntotal} != src.ntotal={src.ntotal}")
    if not base.is_trained:
        raise ValueError("wrapWithRefine: base index is not trained")
    refined = IndexRefineFlat(base, k_factor=k_factor)
    refined.refine.add(reconstruct_all(src))
    refined.ntotal = refined.refine.ntotal
    return refined


reconstructAll, flatToIvfFlat, flatToIvfPq, flatToHnsw, wrapWithRefine = (reconstruct_all, flat_to_ivf_flat,
                                                                          flat_to_ivf_pq, flat_to_hnsw,
                                                                          wrap_with_refine)


# ---------------------------------------------------------------------------------------------------- bench --
@dataclass
class BenchResult:
    label: str
    nq: int
    k: int
    recall: float
    mean_us: float
    p50_us: float
    p95_us: float
    p99_us: float
    ntotal: int


@dataclass
class BenchOptions:
    warmup: int = 1
    repeats: int = 3
    per_query: bool = True


def recall_at_k(result: SearchResult, truth: SearchResult, k: int) -> float:
    """Mean fraction of the true top-``k`` ids found in the returned top-``k``."""
    hits = total = 0
    for got, want in zip(result.ids[:, :k], truth.ids[:, :k]):
        want = set(int(i) for i in want if i >= 0)
        total += len(want)
        hits += len(want & set(int(i) for i in got if i >= 0))
    return hits / total if total else 0.0


def _percentile(sorted_us: Sequence[float], p: float) -> float:
    if not sorted_us:
        return 0.0
    return float(sorted_us[min(len(sorted_us) - 1, int(p * (len(sorted_us) - 1) + 0.5))])


def bench_index(index: Index, queries, k: int, truth: SearchResult, label: str = "index",
                options: Optional[BenchOptions] = None) -> BenchResult:
    options = options or BenchOptions()
    q = as_rows(queries, index.d)
    if len(q) == 0:
        raise ValueError("benchIndex: queries is empty")
    if truth.nq != len(q):
        raise ValueError(f"benchIndex: truth.nq={truth.nq} != queries.length={len(q)}")
    if truth.k < k:
        raise ValueError(f"benchIndex: truth.k={truth.k} is smaller than requested k={k}")
    for _ in range(options.warmup):
        index.search(q, k)
    best_us, last = None, None
    for _ in range(max(1, options.repeats)):
        if options.per_query:
            us, rows_d, rows_i = [], [], []
            for i in range(len(q)):
                t0 = time.perf_counter()
                r = index.search(q[i:i + 1], k)
                us.append((time.perf_counter() - t0) * 1e6)
                rows_d.append(r.distances[0])
                rows_i.append(r.ids[0])
            res = SearchResult(np.stack(rows_d), np.stack(rows_i))
        else:
            t0 = time.perf_counter()
            res = index.search(q, k)
            us = [(time.perf_counter() - t0) * 1e6 / len(q)] * len(q)
        if best_us is None or sum(us) < sum(best_us):
            best_us, last = us, res
    s = sorted(best_us)
    return BenchResult(label, len(q), k, recall_at_k(last, truth, k), sum(best_us) / len(best_us),
                       _percentile(s, 0.50), _percentile(s, 0.95), _percentile(s, 0.99), index.ntotal)


def bench_index_sweep(index: Index, queries, k: int, truth: SearchResult, values: Iterable,
                      apply: Callable[[object], None], label_for: Callable[[object], str] = str,
                      options: Optional[BenchOptions] = None) -> List[BenchResult]:
    out = []
    for v in values:
        apply(v)
        out.append(bench_index(index, queries, k, truth, label=label_for(v), options=options))
    return out


def _csv_escape(s: str) -> str:
    return '"' + s.replace('"', '""') + '"' if any(c in s for c in ',"\n') else s


def to_bench_csv(rows: Iterable[BenchResult]) -> str:
    out = ["label,ntotal,nq,k,recall,mean_us,p50_us,p95_us,p99_us"]
    for r in rows:
        out.append(f"{_csv_escape(r.label)},{r.ntotal},{r.nq},{r.k},{r.recall:.6f},{r.mean_us:.3f},{r.p50_us:.3f},"
                   f"{r.p95_us:.3f},{r.p99_us:.3f}")
    return "\n".join(out) + "\n"


def format_bench_table(rows: Iterable[BenchResult]) -> str:
    rows = list(rows)
    lw = max([12] + [len(r.label) for r in rows])
    lines = [f"{'label':<{lw}} {'ntotal':>8} {'nq':>6} {'k':>4} {'recall':>8} {'mean us':>10} {'p50':>9} {'p95':>9} "
             f"{'p99':>9}"]
    for r in rows:
        lines.append(f"{r.label:<{lw}} {r.ntotal:>8} {r.nq:>6} {r.k:>4} {r.recall:>8.4f} {r.mean_us:>10.1f} "
                     f"{r.p50_us:>9.1f} {r.p95_us:>9.1f} {r.p99_us:>9.1f}")
    return "\n".join(lines) + "\n"


def to_bench_markdown(rows: Iterable[BenchResult]) -> str:
    out = ["| label | ntotal | nq | k | recall | mean us | p50 | p95 | p99 |", "|---|---|---|---|---|---|---|---|---|"]
    for r in rows:
        out.append(f"| {r.label} | {r.ntotal} | {r.nq} | {r.k} | {r.recall:.4f} | {r.mean_us:.1f} | {r.p50_us:.1f} | "
                   f"{r.p95_us:.1f} | {r.p99_us:.1f} |")
    return "\n".join(out) + "\n"


def pareto_frontier(rows: Iterable[BenchResult]) -> List[BenchResult]:
    """Rows not dominated in (higher recall, lower mean latency), by ascending latency."""
    out: List[BenchResult] = []
    best = -1.0
    for r in sorted(rows, key=lambda r: (r.mean_us, -r.recall)):
        if r.recall > best:
            out.append(r)
            best = r.recall
    return out


benchIndex, benchIndexSweep, toBenchCsv, formatBenchTable, toBenchMarkdown, paretoFrontier = (
    bench_index, bench_index_sweep, to_bench_csv, format_bench_table, to_bench_markdown, pareto_frontier)


# ------------------------------------------------------------------------------------------------ auto-tune --
@dataclass
class OperatingPoint:
    param_value: int
    param_label: str
    recall: float
    mean_us: float


class OperatingPoints:
    def __init__(self, points: Sequence[OperatingPoint]):
        self.points = list(points)

    def pareto(self) -> List[OperatingPoint]:
        out, best = [], -1.0
        for p in sorted(self.points, key=lambda p: (p.mean_us, -p.recall)):
            if p.recall > best:
                out.append(p)
                best = p.recall
        return out

    def pick_for_recall(self, min_recall: float) -> Optional[OperatingPoint]:
        ok = [p for p in self.points if p.recall >= min_recall]
        return min(ok, key=lambda p: p.mean_us) if ok else None

    def pick_for_latency(self, max_mean_us: float) -> Optional[OperatingPoint]:
        ok = [p for p in self.points if p.mean_us <= max_mean_us]
        return max(ok, key=lambda p: (p.recall, -p.mean_us)) if ok else None

    pickForRecall, pickForLatency = pick_for_recall, pick_for_latency


def _tune(index: Index, attr_owner, attr: str, label: str, queries, k, truth, values, limit, min_recall, apply_best,
          options) -> OperatingPoints:
    rows, seen = [], set()
    original = getattr(attr_owner, attr)
    for raw in values:
        v = int(raw) if limit is None else max(1, min(int(raw), limit))
        if v in seen:
            continue
        seen.add(v)
        setattr(attr_owner, attr, v)
        r = bench_index(index, queries, k, truth, label=f"{label}={v}", options=options)
        rows.append(OperatingPoint(v, f"{label}={v}", r.recall, r.mean_us))
    points = OperatingPoints(rows)
    chosen = points.pick_for_recall(min_recall) if (apply_best and min_recall is not None) else None
    setattr(attr_owner, attr, chosen.param_value if chosen is not None else original)
    return points


def _unwrap(index: Index, kinds) -> Index:
    cur = index
    while not isinstance(cur, kinds):
        nxt = getattr(cur, "inner", None) or getattr(cur, "base", None)
        if nxt is None:
            raise ValueError(f"autoTune: {type(index).__name__} does not wrap a tunable index")
        cur = nxt
    return cur


def auto_tune_nprobe(target: Index, queries, k: int, truth: SearchResult, values: Sequence[int] = (1, 2, 4, 8, 16, 32),
                     min_recall: Optional[float] = None, apply_best: bool = True,
                     options: Optional[BenchOptions] = None) -> OperatingPoints:
    """Sweep ``nprobe`` of an IVF index (possibly inside IDMap / PreTransform / RefineFlat wrappers)."""
    ivf = _unwrap(target, (IndexIVFFlat, IndexIVFPQ))
    return _tune(target, ivf, "nprobe", "nprobe", queries, k, truth, values, ivf.nlist, min_recall, apply_best, options)


def auto_tune_ef_search(target: Index, queries, k: int, truth: SearchResult,
                        values: Sequence[int] = (8, 16, 32, 64, 128, 256), min_recall: Optional[float] = None,
                        apply_best: bool = True, options: Optional[BenchOptions] = None) -> OperatingPoints:
    hnsw = _unwrap(target, (IndexHNSW,))
    return _tune(target, hnsw, "ef_search", "efSearch", queries, k, truth, values, None, min_recall, apply_best,
                 options)


@dataclass
class TuneMResult:
    points: OperatingPoints
    built: Dict[int, IndexIVFPQ]
    chosen: Optional[OperatingPoint]
    chosen_index: Optional[IndexIVFPQ]


def auto_tune_m(source_vectors, queries, k: int, truth: SearchResult, values: Sequence[int] = (4, 8, 16),
                nbits: int = 8, nlist: Optional[int] = None, nprobe: Optional[int] = None,
                metric: Metric = Metric.l2, min_recall: Optional[float] = None, seed: int = 1234,
                options: Optional[BenchOptions] = None) -> TuneMResult:
    """Build one IVFPQ per candidate ``m`` (sub-quantizer count) and report recall / latency of each."""
    x = np.asarray(source_vectors, dtype=np.float32)
    if x.ndim != 2 or len(x) == 0:
        raise ValueError("autoTuneM: sourceVectors is empty")
    d = x.shape[1]
    k0 = nlist or _auto_nlist(len(x))
    p0 = nprobe or min(k0, 8)
    rows, built = [], {}
    for m in values:
        if d % m:
            continue
        idx = IndexIVFPQ(d, k0, m, nbits=nbits, nprobe=p0, seed=seed, metric=metric)
        idx.train(x)
        idx.add(x)
        built[m] = idx
        r = bench_index(idx, queries, k, truth, label=f"m={m}", options=options)
        rows.append(OperatingPoint(m, f"m={m}", r.recall, r.mean_us))
    points = OperatingPoints(rows)
    chosen = points.pick_for_recall(min_recall) if min_recall is not None else None
    return TuneMResult(points, built, chosen, built.get(chosen.param_value) if chosen else None)


def auto_tune_m_from_flat(source: IndexFlat, queries, k: int, truth: SearchResult, values: Sequence[int] = (4, 8, 16),
                          **kw) -> TuneMResult:
    """``auto_tune_m`` over the vectors (and metric) already held by a flat index
    (reference: lib/core/vector_store/auto_tune.dart:343-378)."""
    if source.ntotal == 0:
        raise ValueError("autoTuneMFromFlat: source index is empty")
    return auto_tune_m(reconstruct_all(source), queries, k, truth, values=values, metric=source.metric, **kw)


autoTuneNprobe, autoTuneEfSearch, autoTuneM = auto_tune_nprobe, auto_tune_ef_search, auto_tune_m
autoTuneMFromFlat = auto_tune_m_from_flat
