"""CPU tests of the FAISS-file probe, the ``IxDT`` tuning-metadata wrapper and its command-line tools, plus further
vector-store cases (id maps, range search, binary indexes, golden FAISS bytes), after the corresponding groups of the
reference's test/vector_store_test.dart."""
import json
import struct
from datetime import datetime, timezone

import numpy as np
import pytest

from dart_pytorch_b200 import vector_store as vs
from dart_pytorch_b200.apps.__main__ import main as cli
from dart_pytorch_b200.vector_store import Metric


def _data(n=300, d=16, nq=12, seed=0):
    rng = np.random.default_rng(seed)
    cent = rng.standard_normal((8, d)).astype(np.float32) * 3
    x = (cent[rng.integers(8, size=n)] + rng.standard_normal((n, d))).astype(np.float32)
    q = (cent[rng.integers(8, size=nq)] + rng.standard_normal((nq, d))).astype(np.float32)
    return x, q


def _ivf(x, nlist=8, nprobe=1):
    ix = vs.IndexIVFFlat(x.shape[1], nlist, nprobe=nprobe)
    ix.train(x)
    ix.add(x)
    return ix


def _meta(chosen=4, label="nprobe"):
    pts = [vs.OperatingPoint(1, f"{label}=1", 0.61, 10.5), vs.OperatingPoint(4, f"{label}=4", 0.93, 31.25),
           vs.OperatingPoint(8, f"{label}=8 ✓", 1.0, 64.0)]
    return vs.TuningMetadata(datetime(2024, 5, 6, 7, 8, 9, 123456, tzinfo=timezone.utc), Metric.l2, pts, chosen)


# --------------------------------------------------------------------------------------------------- wrapper ---
def test_ixdt_wrapper_round_trips_metadata_and_keeps_the_inner_blob_byte_for_byte():
    x, q = _data()
    ix = _ivf(x)
    plain = vs.write_faiss_index_bytes(ix)
    blob = vs.write_tuned_faiss_index_bytes(ix, _meta())
    assert blob[:4] == b"IxDT" and struct.unpack_from("<I", blob, 4)[0] == 1
    tuning_len = struct.unpack_from("<Q", blob, 8)[0]
    assert blob[16 + tuning_len:] == plain and vs.strip_tuning_wrapper(blob) == plain
    assert vs.is_tuned_faiss_blob(blob) and not vs.is_tuned_faiss_blob(plain) and not vs.is_tuned_faiss_blob(b"Ix")
    back, meta = vs.read_tuned_faiss_index_bytes(blob)
    assert isinstance(back, vs.IndexIVFFlat) and back.ntotal == 300 and back.nprobe == 1
    assert meta.created_at == _meta().created_at and meta.metric == Metric.l2 and meta.chosen_param_value == 4
    assert [(p.param_value, p.param_label, p.recall, p.mean_us) for p in meta.points] == \
        [(1, "nprobe=1", 0.61, 10.5), (4, "nprobe=4", 0.93, 31.25), (8, "nprobe=8 ✓", 1.0, 64.0)]
    assert np.array_equal(back.search(q, 5).ids, ix.search(q, 5).ids)
    # golden layout of the tuning block
    t = blob[16:16 + tuning_len]
    micros, metric_code, n = struct.unpack_from("<qiI", t, 0)
    assert micros == 1714979289123456 and metric_code == 1 and n == 3
    assert struct.unpack_from("<iI", t, 16) == (1, 8) and t[24:32] == b"nprobe=1"
    assert struct.unpack_from("<dd", t, 32) == (0.61, 10.5) and t[-5:] == b"\x01" + struct.pack("<i", 4)


def test_ixdt_wrapper_with_no_points_and_no_choice():
    x, _ = _data(50)
    flat = vs.IndexFlatIP(16)
    flat.add(x)
    empty = vs.TuningMetadata(datetime(2020, 1, 1, tzinfo=timezone.utc), Metric.inner_product, [], None)
    blob = vs.write_tuned_faiss_index_bytes(flat, empty)
    back, meta = vs.read_tuned_faiss_index_bytes(blob, apply_tuning=True)
    assert meta.points == [] and meta.chosen_param_value is None and meta.metric == Metric.inner_product
    assert back.ntotal == 50 and struct.unpack_from("<Q", blob, 8)[0] == 8 + 4 + 4 + 1


def test_ixdt_rejections():
    x, _ = _data(40)
    plain = vs.write_faiss_index_bytes(_ivf(x, 4))
    blob = vs.write_tuned_faiss_index_bytes(_ivf(x, 4), _meta())
    for fn in (vs.read_tuned_faiss_index_bytes, vs.strip_tuning_wrapper):
        with pytest.raises(ValueError, match="not a tuned"):
            fn(plain)
        with pytest.raises(ValueError):
            fn(b"Ix")
        with pytest.raises(ValueError, match="version"):
            fn(blob[:4] + struct.pack("<I", 2) + blob[8:])
        with pytest.raises(ValueError, match="declares"):
            fn(blob[:8] + struct.pack("<Q", 1 << 40) + blob[16:])
        with pytest.raises(ValueError, match="truncated"):
            fn(blob[:10])


def test_apply_tuning_to_index():
    x, _ = _data()
    ivf = _ivf(x)
    assert vs.apply_tuning_to_index(ivf, _meta(4)) and ivf.nprobe == 4
    refined = vs.wrap_with_refine(_ivf(x), _flat(x))
    assert vs.apply_tuning_to_index(refined, _meta(8)) and refined.base.nprobe == 8
    hnsw = vs.IndexHNSW(16, M=8)
    hnsw.add(x[:100])
    assert vs.apply_tuning_to_index(hnsw, _meta(8, "efSearch")) and hnsw.ef_search == 8
    assert vs.apply_tuning_to_index(ivf, _meta(None)) is False and ivf.nprobe == 4
    assert vs.apply_tuning_to_index(ivf, _meta(4, "m")) is False              # not a search-time parameter
    with pytest.raises(ValueError):
        vs.apply_tuning_to_index(hnsw, _meta(4))                              # nprobe on a graph index
    with pytest.raises(ValueError):
        vs.apply_tuning_to_index(ivf, _meta(8, "efSearch"))
    with pytest.raises(ValueError):
        vs.apply_tuning_to_index(ivf, _meta(5))                               # chosen value not among the points


def _flat(x, metric=Metric.l2):
    f = vs.IndexFlat(x.shape[1], metric)
    f.add(x)
    return f


def test_tuning_metadata_from_sweeps_and_load_with_apply(tmp_path):
    x, q = _data(400)
    truth = _flat(x).search(q, 5)
    ivf = _ivf(x, nlist=8, nprobe=1)
    sweep = vs.auto_tune_nprobe(ivf, q, 5, truth, values=(1, 2, 8), min_recall=0.99)
    chosen = sweep.pick_for_recall(0.99)
    meta = vs.TuningMetadata.from_operating_points(sweep, Metric.l2, chosen_param_value=chosen.param_value)
    assert len(meta.points) == len(sweep.points) and meta.created_at.tzinfo is not None
    ivf.nprobe = 1
    path = tmp_path / "tuned.faiss"
    vs.save_tuned_faiss_index(str(path), ivf, meta)
    cold, _ = vs.load_tuned_faiss_index(str(path))
    warm, m2 = vs.load_tuned_faiss_index(str(path), apply_tuning=True)
    assert cold.nprobe == 1 and warm.nprobe == chosen.param_value == m2.chosen_param_value
    assert vs.recall_at_k(warm.search(q, 5), truth, 5) >= 0.99
    res = vs.auto_tune_m(x, q, 5, truth, values=(4, 8), nlist=4, nprobe=4)
    mm = vs.TuningMetadata.from_tune_m_result(res, Metric.l2)
    assert [p.param_value for p in mm.points] == [4, 8]
    assert mm.chosen_param_value == (None if res.chosen is None else res.chosen.param_value)


# ----------------------------------------------------------------------------------------------------- probe ---
def test_probe_float_binary_wrapped_and_unknown(tmp_path):
    x, _ = _data(120)
    info = vs.probe_faiss_index(vs.write_faiss_index_bytes(_flat(x, Metric.inner_product)))
    assert (info.fourcc_str, info.kind, info.d, info.ntotal, info.metric, info.is_trained) == \
        ("IxFI", vs.FaissIndexKind.float_index, 16, 120, Metric.inner_product, True)
    assert info.fourcc == vs.FaissFourcc.of("IxFI") and info.tuning is None and info.inner is None and info.code_size is None
    empty_ivf = vs.IndexIVFFlat(16, 4)
    assert vs.probe_faiss_index(vs.write_faiss_index_bytes(empty_ivf)[:37]).is_trained is False
    codes = np.random.default_rng(0).integers(0, 256, size=(30, 8), dtype=np.uint8)
    b = vs.IndexBinaryFlat(8)
    b.add(codes)
    bi = vs.probe_faiss_index(vs.write_faiss_binary_index_bytes(b))
    assert (bi.fourcc_str, bi.kind, bi.d, bi.code_size, bi.ntotal) == ("IBxF", vs.FaissIndexKind.binary_index, 64, 8, 30)
    wrapped = vs.probe_faiss_index(vs.write_tuned_faiss_index_bytes(_ivf(x, 4), _meta()))
    assert wrapped.kind == vs.FaissIndexKind.tuned_wrapper and wrapped.fourcc_str == "IxDT"
    assert wrapped.inner.fourcc_str == "IwFl" and wrapped.d == 16 and wrapped.ntotal == 120
    assert wrapped.tuning.chosen_param_value == 4 and len(wrapped.tuning.points) == 3
    unk = vs.probe_faiss_index(b"Zzzz" + bytes(40))
    assert unk.kind == vs.FaissIndexKind.unknown and unk.fourcc_str == "Zzzz" and unk.d is None
    with pytest.raises(ValueError):
        vs.probe_faiss_index(b"Ix")
    with pytest.raises(ValueError):
        vs.probe_faiss_index(b"IxF2" + bytes(10))
    plain, tuned = tmp_path / "p.faiss", tmp_path / "t.faiss"
    vs.write_faiss_index(_flat(x), str(plain))
    vs.save_tuned_faiss_index(str(tuned), _ivf(x, 4), _meta())
    assert vs.probe_faiss_index_file(str(plain)).ntotal == 120
    assert vs.probe_faiss_index_file(str(tuned)).tuning.points[1].recall == 0.93


def test_describe_and_strip_tools(tmp_path, capsys):
    x, _ = _data(90)
    tuned = tmp_path / "tuned.faiss"
    vs.save_tuned_faiss_index(str(tuned), _ivf(x, 4), _meta())
    rec = cli(["faiss_describe", str(tuned), "--json"])
    printed = json.loads(capsys.readouterr().out.strip().splitlines()[0])
    assert printed == json.loads(json.dumps(rec)) and rec["fourcc"] == "IxDT" and rec["inner"] == "IwFl"
    assert rec["tuning"]["chosen"] == 4 and rec["ntotal"] == 90
    out = cli(["faiss_strip", str(tuned)])
    assert out == str(tmp_path / "tuned.stripped.faiss")
    plain = open(out, "rb").read()
    assert plain[:4] == b"IwFl" and vs.read_faiss_index_bytes(plain).ntotal == 90
    with pytest.raises(ValueError):
        cli(["faiss_strip", out])                                              # already plain
    emptied = cli(["faiss_strip", out, str(tmp_path / "empty.faiss"), "--vectors"])
    assert vs.read_faiss_index(emptied).ntotal == 0
    vs.strip_tuning_wrapper_file(str(tuned), str(tmp_path / "again.faiss"))
    assert open(tmp_path / "again.faiss", "rb").read() == plain
    cli(["faiss_describe", out, "--deep"])
    assert "IndexIVFFlat" in capsys.readouterr().out


# ------------------------------------------------------------------------------------- further index checks ---
def test_id_map_custom_ids_remove_and_faiss_round_trip():
    x, q = _data(60)
    m = vs.IndexIDMap(vs.IndexFlatL2(16))
    ids = np.arange(1000, 1060, dtype=np.int64) * 7
    m.add_with_ids(x, ids)
    res = m.search(x[:5], 1)
    assert res.ids[:, 0].tolist() == ids[:5].tolist() and np.allclose(res.distances[:, 0], 0, atol=1e-3)
    with pytest.raises(ValueError):
        m.add_with_ids(x[:1], np.array([1 << 40]))                             # ids must fit int32 (file format)
    assert m.remove_ids({int(ids[0]), int(ids[3])}) == 2 and m.ntotal == 58
    assert int(ids[0]) not in m.search(x[:1], 3).ids[0].tolist()
    assert m.search(x[1:2], 1).ids[0, 0] == ids[1]                             # external ids survive compaction
    back = vs.read_faiss_index_bytes(vs.write_faiss_index_bytes(m))
    assert isinstance(back, vs.IndexIDMap) and np.array_equal(back.search(q, 4).ids, m.search(q, 4).ids)
    blob = bytearray(vs.write_faiss_index_bytes(m))
    blob[:4] = b"IxM2"                                                         # IndexIDMap2 reads as an id map
    assert isinstance(vs.read_faiss_index_bytes(bytes(blob)), vs.IndexIDMap)


def test_range_search_agrees_with_filtered_search_and_unsupported_raises():
    x, q = _data(150)
    flat = _flat(x)
    full = flat.search(q, 150)
    radius = float(np.median(full.distances[:, 10]))
    rr = flat.range_search(q, radius)
    for i in range(len(q)):
        got = set(rr.ids[rr.limits[i]:rr.limits[i + 1]].tolist())
        assert got == set(full.ids[i][full.distances[i] < radius].tolist())
    ivf = _ivf(x, nlist=4, nprobe=4)
    r2 = ivf.range_search(q, radius)
    assert r2.total_matches == rr.total_matches
    with pytest.raises(NotImplementedError):
        vs.IndexHNSW(16).range_search(q, 1.0)


def test_binary_flat_hamming_ranking_and_ivf_accumulates():
    rng = np.random.default_rng(3)
    codes = rng.integers(0, 256, size=(80, 4), dtype=np.uint8)
    flat = vs.IndexBinaryFlat(4)
    flat.add(codes)
    res = flat.search(codes[:6], 5)
    assert res.ids[:, 0].tolist() == list(range(6)) and (res.distances[:, 0] == 0).all()
    assert (np.diff(res.distances, axis=1) >= 0).all()
    want = [vs.hamming_distance(codes[0], codes[int(j)]) for j in res.ids[0]]
    assert res.distances[0].tolist() == want
    ivf = vs.IndexBinaryIVF(4, 4, nprobe=4)
    ivf.train(codes)
    ivf.add(codes[:50])
    ivf.add(codes[50:])
    assert ivf.ntotal == 80
    assert np.array_equal(np.sort(ivf.search(codes[:6], 5).distances, 1), np.sort(res.distances, 1))


def test_faiss_flat_golden_fixture_parses():
    vecs = np.array([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], dtype="<f4")
    blob = b"IxF2" + struct.pack("<iqqqBi", 2, 3, 1 << 20, 1 << 20, 1, 1) + struct.pack("<Q", 6) + vecs.tobytes()
    ix = vs.read_faiss_index_bytes(blob)
    assert isinstance(ix, vs.IndexFlat) and ix.metric == Metric.l2 and ix.d == 2 and ix.ntotal == 3
    assert ix.search(np.array([[3.0, 4.0]], dtype=np.float32), 1).ids[0, 0] == 1
    assert vs.write_faiss_index_bytes(ix) == blob
    assert vs.FaissFourcc.name(vs.FaissFourcc.of("IwPQ")) == "IwPQ"
    with pytest.raises(ValueError):
        vs.FaissFourcc.of("toolong")
    with pytest.raises(ValueError, match="Zzzz"):
        vs.read_faiss_index_bytes(b"Zzzz" + blob[4:])
