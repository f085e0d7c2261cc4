"""Vector store: exactness of flat search, recall of the approximate indexes, wrappers, transforms, factory strings,
persistence round trips (FAISDART and FAISS layouts), bench / auto-tune helpers."""
import itertools
import struct

import numpy as np
import pytest

from dart_pytorch_b200 import vector_store as vs
from dart_pytorch_b200.vector_store import Metric


def _data(n=400, d=16, seed=0, clusters=8):
    rng = np.random.default_rng(seed)
    cent = rng.standard_normal((clusters, d)).astype(np.float32) * 4
    x = cent[rng.integers(clusters, size=n)] + rng.standard_normal((n, d)).astype(np.float32) * 0.5
    q = cent[rng.integers(clusters, size=20)] + rng.standard_normal((20, d)).astype(np.float32) * 0.5
    return x.astype(np.float32), q.astype(np.float32)


def _truth(x, q, k, metric=Metric.l2):
    f = vs.IndexFlat(x.shape[1], metric)
    f.add(x)
    return f, f.search(q, k)


def test_flat_search_exact_range_and_remove():
    x, q = _data()
    for metric in (Metric.l2, Metric.inner_product):
        f, r = _truth(x, q, 5, metric)
        if metric == Metric.l2:
            want = ((q[:, None, :] - x[None]) ** 2).sum(-1)
            order = np.argsort(want, 1)[:, :5]
        else:
            want = q @ x.T
            order = np.argsort(-want, 1)[:, :5]
        assert np.array_equal(r.ids, order)
        assert np.allclose(r.distances, np.take_along_axis(want, order, 1), atol=1e-3)
    f, _ = _truth(x, q, 5)
    rr = f.range_search(q[:3], 4.0)
    assert rr.nq == 3 and rr.total_matches == sum(rr.length_for(i) for i in range(3))
    ds, ids = rr.to_rows()
    assert all((d < 4.0).all() for d in ds)
    assert f.remove_ids({0, 1, 10 ** 6}) == 2 and f.ntotal == len(x) - 2
    assert np.allclose(f.reconstruct(0), x[2])
    small = vs.IndexFlat(4)
    small.add_rows([[0, 0, 0, 0], [1, 1, 1, 1]])
    r = small.search_rows([[0.1, 0, 0, 0]], 4)
    assert r.ids[0].tolist() == [0, 1, -1, -1] and np.isinf(r.distances[0, 2])
    with pytest.raises(ValueError):
        small.add_rows([[1, 2, 3]])


def test_topk_heap_and_kmeans():
    t = vs.TopK(3, max_is_worst=True)
    for s, i in [(5, 0), (1, 1), (4, 2), (0.5, 3), (9, 4)]:
        t.push(s, i)
    sc, ids = t.sorted()
    assert ids.tolist() == [3, 1, 2] and t.worst == 4 and t.worse_than_worst(4.0)
    t = vs.TopK(2, max_is_worst=False)
    t.push(1.0, 7)
    sc, ids = t.sorted()
    assert ids.tolist() == [7, -1] and sc[1] == -np.inf
    x, _ = _data(300, 8, clusters=4)
    res = vs.Kmeans(8, 4, niter=15, seed=3).train(x)
    assert res.centroids.shape == (4, 8) and len(set(res.assignments.tolist())) == 4
    assert res.objective / len(x) < 8 * 0.5 ** 2 * 2.5          # close to the within-cluster noise
    with pytest.raises(ValueError):
        vs.Kmeans(8, 400).train(x)


@pytest.mark.parametrize("desc,min_recall,setup", [
    ("IVF16,Flat", 0.95, lambda ix: setattr(ix, "nprobe", 8)),
    ("IVF8,PQ4", 0.5, lambda ix: setattr(ix, "nprobe", 8)),
    ("PQ8", 0.5, None),
    ("SQ8", 0.9, None),
    ("HNSW8", 0.9, None),
    ("PCA8,Flat", 0.5, None),
    ("L2Norm,Flat", 0.0, None),
    ("RR,IVF4,Flat", 0.5, lambda ix: setattr(ix.inner, "nprobe", 4)),
])
def test_factory_indexes_reach_recall(desc, min_recall, setup):
    x, q = _data()
    ix = vs.index_factory(16, desc)
    if setup:
        setup(ix)
    assert not ix.is_trained or desc in ("HNSW8", "L2Norm,Flat")
    ix.train(x)
    ix.add(x)
    assert ix.is_trained and ix.ntotal == len(x)
    _, truth = _truth(x, q, 10)
    r = ix.search(q, 10)
    assert r.ids.shape == (20, 10)
    assert vs.recall_at_k(r, truth, 10) >= min_recall


def test_factory_rejects_bad_descriptions():
    for bad in ("", "Flat,Flat", "IVF8", "IVF8,Bogus", "Wat", "PCA4"):
        with pytest.raises(ValueError):
            vs.index_factory(16, bad)
    assert isinstance(vs.index_factory(16, "LSH32"), vs.IndexLSH)
    assert vs.index_factory(16, "PQ4x6").pq.ksub == 64


def test_ivf_flat_full_probe_is_exact_and_remove_ids():
    x, q = _data()
    ivf = vs.IndexIVFFlat(16, 8, nprobe=8)
    with pytest.raises(RuntimeError):
        ivf.add(x)
    ivf.train(x)
    ivf.add(x)
    f, truth = _truth(x, q, 5)
    assert np.array_equal(ivf.search(q, 5).ids, truth.ids)
    assert sum(ivf.list_sizes()) == len(x)
    assert ivf.remove_ids({3, 4}) == 2 and ivf.ntotal == len(x) - 2
    f.remove_ids({3, 4})
    assert np.array_equal(ivf.search(q, 5).ids, f.search(q, 5).ids)


def test_wrappers_idmap_refine_shards_replicas():
    x, q = _data(200, 8)
    idm = vs.IndexIDMap(vs.IndexFlat(8))
    idm.add_with_ids(x, [1000 + 2 * i for i in range(len(x))])
    f, truth = _truth(x, q, 3)
    assert np.array_equal(idm.search(q, 3).ids, 1000 + 2 * truth.ids)
    assert idm.internal_of(1004) == 2 and idm.internal_of(7) == -1
    assert idm.remove_ids({1000, 1002}) == 2 and idm.id_of(0) == 1004
    with pytest.raises(ValueError):
        idm.add_with_ids(x[:1], [2 ** 40])
    base = vs.IndexPQ(8, 4, nbits=4)
    ref = vs.IndexRefineFlat(base, k_factor=8)
    ref.train(x)
    ref.add(x)
    assert vs.recall_at_k(ref.search(q, 3), truth, 3) >= vs.recall_at_k(base.search(q, 3), truth, 3)
    assert vs.recall_at_k(ref.search(q, 3), truth, 3) > 0.8
    sh = vs.IndexShards([vs.IndexFlat(8) for _ in range(3)])
    sh.add(x)
    assert [s.ntotal for s in sh.shards] == [67, 67, 66]
    assert np.array_equal(sh.search(q, 3).ids, truth.ids)
    rep = vs.IndexReplicas([vs.IndexFlat(8), vs.IndexFlat(8)])
    rep.add(x)
    assert np.array_equal(rep.search(q, 3).ids, truth.ids) and np.array_equal(rep.search(q, 3).ids, truth.ids)
    with pytest.raises(ValueError):
        vs.IndexShards([vs.IndexFlat(8), vs.IndexFlat(4)])


def test_binary_indexes_and_lsh():
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 256, size=(300, 8), dtype=np.uint8)
    q = codes[:5].copy()
    q[:, 0] ^= 1
    bf = vs.IndexBinaryFlat(8)
    bf.add(codes)
    r = bf.search(q, 2)
    assert r.ids[:, 0].tolist() == [0, 1, 2, 3, 4] and (r.distances[:, 0] == 1).all() and bf.d == 64
    assert vs.hamming_distance(codes[0], codes[1]) == int(np.unpackbits(codes[0] ^ codes[1]).sum())
    biv = vs.IndexBinaryIVF(8, 4, nprobe=4)
    biv.train(codes)
    biv.add(codes)
    assert np.array_equal(biv.search(q, 2).ids, r.ids)
    x, qq = _data(300, 16)
    lsh = vs.IndexLSH(16, 64)
    lsh.add(x)
    _, truth = _truth(x, qq, 10)
    assert vs.recall_at_k(lsh.search(qq, 10), truth, 10) > 0.3


def test_transforms():
    x, _ = _data(200, 6)
    rr = vs.RandomRotationTransform(6, seed=5)
    assert np.allclose(rr.matrix @ rr.matrix.T, np.eye(6), atol=1e-5)
    assert np.allclose(np.linalg.norm(rr.apply(x), axis=1), np.linalg.norm(x, axis=1), atol=1e-4)
    assert np.allclose(np.linalg.norm(vs.L2NormTransform(6).apply(x), axis=1), 1.0, atol=1e-5)
    pca = vs.PCATransform(6, 3)
    pca.train(x)
    y = pca.apply(x)
    w = np.linalg.eigvalsh(np.cov(x.T))[::-1][:3]
    assert np.allclose(pca.eigenvalues, w, rtol=1e-3) and np.allclose(y.var(0, ddof=1), w, rtol=1e-3)
    white = vs.PCATransform(6, 3, eigen_power=-0.5)
    white.train(x)
    assert np.allclose(white.apply(x).var(0, ddof=1), 1.0, atol=1e-3)
    assert np.allclose(pca.apply(x), x @ pca.matrix.T + pca.bias, atol=1e-4)
    wv, vv = vs.jacobi_eigh(np.array([[2.0, 1.0], [1.0, 2.0]]))
    assert np.allclose(wv, [3.0, 1.0])


def _roundtrip_all(x, q):
    d = x.shape[1]
    made = {}
    for desc in ("Flat", "IVF8,Flat", "PQ4x4", "IVF4,PQ4x4", "SQ8", "HNSW8", "LSH32", "PCA8,IVF4,Flat", "L2Norm,Flat",
                 "RR,Flat"):
        ix = vs.index_factory(d, desc)
        ix.train(x)
        ix.add(x)
        made[desc] = ix
    idm = vs.IndexIDMap(vs.IndexFlat(d))
    idm.add_with_ids(x, list(range(5, 5 + len(x))))
    made["idmap"] = idm
    ref = vs.IndexRefineFlat(vs.index_factory(d, "PQ4x4"), k_factor=4)
    ref.train(x)
    ref.add(x)
    made["refine"] = ref
    return made


def test_faisdart_round_trip_every_kind(tmp_path):
    x, q = _data(200, 16)
    made = _roundtrip_all(x, q)
    sh = vs.IndexShards([vs.IndexFlat(16), vs.IndexFlat(16)])
    sh.add(x)
    made["shards"] = sh
    rep = vs.IndexReplicas([vs.IndexFlat(16), vs.IndexFlat(16)])
    rep.add(x)
    made["replicas"] = rep
    for name, ix in made.items():
        blob = vs.write_index_bytes(ix)
        assert blob[:8] == b"FAISDART" and struct.unpack("<I", blob[8:12])[0] == 1
        back = vs.read_index_bytes(blob)
        assert type(back) is type(ix) and back.ntotal == ix.ntotal, name
        a, b = ix.search(q, 5), back.search(q, 5)
        assert np.array_equal(a.ids, b.ids) and np.allclose(a.distances, b.distances, atol=1e-5), name
        assert vs.write_index_bytes(back) == blob, name
    p = tmp_path / "sub" / "flat.idx"
    vs.write_index(made["Flat"], str(p))
    assert vs.read_index(str(p)).ntotal == 200
    with pytest.raises(ValueError):
        vs.read_index_bytes(b"NOTMAGIC" + bytes(20))
    with pytest.raises(ValueError):
        vs.read_index_bytes(vs.write_index_bytes(made["Flat"])[:40])
    rng = np.random.default_rng(1)
    codes = rng.integers(0, 256, size=(50, 4), dtype=np.uint8)
    for b in (vs.IndexBinaryFlat(4), vs.IndexBinaryIVF(4, 4, nprobe=4)):
        b.train(codes)
        b.add(codes)
        back = vs.read_binary_index_bytes(vs.write_index_bytes(b))
        assert np.array_equal(back.search(codes[:3], 2).ids, b.search(codes[:3], 2).ids)
    with pytest.raises(ValueError):
        vs.read_binary_index_bytes(vs.write_index_bytes(made["Flat"]))


def test_faiss_layout_round_trip_and_header_bytes():
    x, q = _data(200, 16)
    made = _roundtrip_all(x, q)
    for name, ix in made.items():
        blob = vs.write_faiss_index_bytes(ix)
        back = vs.read_faiss_index_bytes(blob)
        assert type(back) is type(ix) and back.ntotal == ix.ntotal, name
        a, b = ix.search(q, 5), back.search(q, 5)
        assert np.array_equal(a.ids, b.ids) and np.allclose(a.distances, b.distances, atol=1e-4), name
    blob = vs.write_faiss_index_bytes(made["Flat"])
    assert blob[:4] == b"IxF2"
    d, ntotal, dummy1, dummy2, trained, metric = struct.unpack("<iqqqBi", blob[4:37])
    assert (d, ntotal, dummy1, dummy2, trained, metric) == (16, 200, 1 << 20, 1 << 20, 1, 1)
    assert struct.unpack("<Q", blob[37:45])[0] == 200 * 16
    assert np.array_equal(np.frombuffer(blob[45:], dtype="<f4").reshape(200, 16), x)
    ip = vs.IndexFlat(16, Metric.inner_product)
    ip.add(x)
    assert vs.write_faiss_index_bytes(ip)[:4] == b"IxFI"
    assert vs.FaissFourcc.of("IxF2") == 0x32467849
    with pytest.raises(ValueError):
        vs.read_faiss_index_bytes(b"Zzzz" + bytes(64))
    rng = np.random.default_rng(1)
    codes = rng.integers(0, 256, size=(50, 4), dtype=np.uint8)
    for b in (vs.IndexBinaryFlat(4), vs.IndexBinaryIVF(4, 4, nprobe=4)):
        b.train(codes)
        b.add(codes)
        back = vs.read_faiss_binary_index_bytes(vs.write_faiss_binary_index_bytes(b))
        assert np.array_equal(back.search(codes[:3], 2).ids, b.search(codes[:3], 2).ids)
    assert "IndexIVFFlat" in vs.faiss_describe(vs.write_faiss_index_bytes(made["PCA8,IVF4,Flat"]))
    stripped = vs.read_faiss_index_bytes(vs.faiss_strip(vs.write_faiss_index_bytes(made["IVF8,Flat"])))
    assert stripped.ntotal == 0 and stripped.is_trained and stripped.quantizer.ntotal == 8


def test_conversions_bench_and_autotune():
    x, q = _data(300, 16)
    f, truth = _truth(x, q, 10)
    ivf = vs.flat_to_ivf_flat(f, nlist=8)
    assert ivf.ntotal == 300 and ivf.nprobe == 8
    assert vs.flat_to_ivf_pq(f, m=4, nlist=4).ntotal == 300
    h = vs.flat_to_hnsw(f, M=8)
    assert vs.recall_at_k(h.search(q, 10), truth, 10) > 0.9
    wrapped = vs.wrap_with_refine(vs.flat_to_ivf_pq(f, m=4, nlist=4), f)
    assert wrapped.refine.ntotal == 300
    with pytest.raises(ValueError):
        vs.flat_to_ivf_pq(f, m=5)
    res = vs.bench_index(ivf, q, 10, truth, label="ivf", options=vs.BenchOptions(warmup=0, repeats=1))
    assert res.recall > 0.99 and res.mean_us > 0 and res.p50_us <= res.p99_us
    csv = vs.to_bench_csv([res])
    assert csv.splitlines()[0] == "label,ntotal,nq,k,recall,mean_us,p50_us,p95_us,p99_us" and "ivf,300,20,10" in csv
    assert "recall" in vs.format_bench_table([res]) and vs.to_bench_markdown([res]).startswith("| label")
    pts = vs.auto_tune_nprobe(ivf, q, 10, truth, values=(1, 2, 8, 64), min_recall=0.99,
                              options=vs.BenchOptions(warmup=0, repeats=1))
    assert [p.param_value for p in pts.points] == [1, 2, 8]           # 64 clamps to nlist=8, deduplicated
    assert pts.pick_for_recall(0.99) is not None and ivf.nprobe == pts.pick_for_recall(0.99).param_value
    assert pts.pareto()[0].mean_us <= pts.pareto()[-1].mean_us
    ef = vs.auto_tune_ef_search(h, q, 10, truth, values=(4, 64), options=vs.BenchOptions(warmup=0, repeats=1))
    assert ef.points[1].recall >= ef.points[0].recall
    tm = vs.auto_tune_m(x, q, 10, truth, values=(2, 4, 5), nlist=4, options=vs.BenchOptions(warmup=0, repeats=1))
    assert sorted(tm.built) == [2, 4]
    frontier = vs.pareto_frontier([vs.BenchResult("a", 1, 1, 0.5, 10, 0, 0, 0, 1), vs.BenchResult("b", 1, 1, 0.4, 20, 0, 0, 0, 1),
                                   vs.BenchResult("c", 1, 1, 0.9, 30, 0, 0, 0, 1)])
    assert [r.label for r in frontier] == ["a", "c"]


def test_gpu_index_flat_cpu_fallback_matches_flat():
    x, q = _data(100, 8)
    g = vs.GpuIndexFlat.l2(8, device="cpu")
    g.add(x)
    _, truth = _truth(x, q, 4)
    assert np.array_equal(g.search(q, 4).ids, truth.ids)           # below the 2^18 threshold: CPU scan
    big_x, big_q = _data(2000, 32, seed=2)
    g2 = vs.GpuIndexFlat.wrap(_truth(big_x, big_q, 1)[0], device="cpu")
    _, t2 = _truth(big_x, big_q, 5)
    assert np.array_equal(g2.search(big_q, 5).ids, t2.ids)         # matmul path (fp32 on CPU)
