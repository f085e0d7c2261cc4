"""CPU tests: cooperative training (checkpoint averaging, shards, HTTP star / gossip modes with injected failures),
tokenizers, datasets, safetensors.  Failures are injected on the host: stale rounds, garbled blobs, mismatched headers,
unreachable peers."""
import json
import os
import random
import struct

import numpy as np
import pytest
import torch

import dart_pytorch_b200 as dp
from dart_pytorch_b200 import nn
from dart_pytorch_b200.coop import (Coordinator, Peer, Worker, average_checkpoints, build_coop_lm, CharVocab,
                                    K_TOY_CORPUS, sample_window, shard_slice, train_phase0)
from dart_pytorch_b200.data import (BpeTokenizer, CharTokenizer, CsvDataset, DataLoader, ListDataset, TextTokenDataset)
from dart_pytorch_b200.io.safetensors import SafeTensors


def test_average_checkpoints_weights_and_rejections():
    a, b = nn.Linear(2, 2, seed=1), nn.Linear(2, 2, seed=2)
    ba, bb = dp.Checkpoint.save_bytes(a), dp.Checkpoint.save_bytes(b)
    avg = average_checkpoints([ba, bb])
    c = nn.Linear(2, 2, seed=3)
    dp.Checkpoint.load_into_bytes(c, avg)
    assert torch.allclose(c.weight, 0.5 * (a.weight + b.weight), atol=1e-7)
    w = average_checkpoints([ba, bb], [3.0, 1.0])
    dp.Checkpoint.load_into_bytes(c, w)
    assert torch.allclose(c.bias, 0.75 * a.bias + 0.25 * b.bias, atol=1e-7)
    assert avg[:12 + struct.unpack("<I", ba[8:12])[0]] == ba[:12 + struct.unpack("<I", ba[8:12])[0]]
    other = dp.Checkpoint.save_bytes(nn.Linear(3, 2))
    for bad in (lambda: average_checkpoints([]), lambda: average_checkpoints([ba, bb], [1.0]),
                lambda: average_checkpoints([ba, bb], [1.0, -1.0]), lambda: average_checkpoints([ba, bb], [0.0, 0.0]),
                lambda: average_checkpoints([ba, other]), lambda: average_checkpoints([b"XXXX" + ba[4:], bb]),
                lambda: average_checkpoints([ba, ba[:20] + b"!" + ba[21:]]),
                lambda: average_checkpoints([dp.Checkpoint.save_bytes(a, fp16=True) + b"\0"])):
        with pytest.raises(ValueError):
            bad()


def test_shards_windows_and_vocab():
    v = CharVocab.from_text("hello world")
    ids = v.encode("hello world")
    assert v.decode(ids) == "hello world" and v.encode("z") == [0.0]
    assert shard_slice(list(range(10)), 0, 3) == [0, 1, 2] and shard_slice(list(range(10)), 2, 3) == [6, 7, 8, 9]
    with pytest.raises(ValueError):
        shard_slice([1, 2], 2, 2)
    x, y = sample_window(ids, 4, random.Random(0))
    assert x.shape == (4,) and torch.equal(x[1:], y[:-1])
    with pytest.raises(ValueError):
        sample_window(ids, 20, random.Random(0))
    lm = build_coop_lm("gpt", "tiny", v.size)
    assert lm.max_len == 32 and lm.scalar_count == sum(p.numel() for p in lm.module.parameters())
    assert build_coop_lm("aft", "tiny", v.size)(torch.tensor([1, 2, 3])).shape == (3, v.size)
    with pytest.raises(ValueError):
        build_coop_lm("gpt", "huge", 10)


def test_coordinator_rounds_stale_and_poisoned_submissions():
    coord = Coordinator(target=2, seed=1)
    h = coord.serve()
    try:
        w0 = Worker(h.url, "w0", 0, 2, local_steps=3, seed=1)
        w1 = Worker(h.url, "w1", 1, 2, local_steps=3, seed=2)
        r0 = w0.run_round()
        assert r0["status"] == 200 and r0["accepted"] and not r0["aggregated"] and r0["queueSize"] == 1
        before = coord.global_bytes
        r1 = w1.run_round()
        assert r1["aggregated"] and r1["round"] == 1 and coord.global_bytes != before
        assert coord.status() == {"round": 1, "queueSize": 0, "target": 2, "workersSeen": ["w0", "w1"]}
        # stale round -> 409, nothing queued
        code, js = coord.submit("w0", 0, 3, dp.Checkpoint.save_bytes(w0.lm.module))
        assert code == 409 and js["reason"] == "stale round" and js["currentRound"] == 1
        # garbled blob and wrong architecture -> 400
        good = dp.Checkpoint.save_bytes(w0.lm.module)
        for bad in (good[:-8], b"junk", dp.Checkpoint.save_bytes(nn.Linear(2, 2))):
            code, js = coord.submit("evil", 1, 3, bad)
            assert code == 400 and not js["accepted"]
        assert coord.status()["queueSize"] == 0 and "evil" not in coord.status()["workersSeen"]
        cfg = json.loads(coord.config_json())
        assert cfg["arch"] == "gpt" and cfg["maxLen"] == 32 and cfg["target"] == 2
    finally:
        h.close()


def test_gossip_peer_survives_unreachable_peer():
    a = Peer([], local_steps=2, seed=1)
    ha = a.serve()
    try:
        b = Peer([ha.url, "http://127.0.0.1:9"], local_steps=2, seed=2, connect_timeout=0.5, read_timeout=0.5)
        outcomes = [b.run_round()["gossiped"] for _ in range(6)]
        assert ha.url in outcomes          # merged with the live peer at least once
        assert any("failed" in line for line in b.log) or None not in outcomes
        assert all(torch.isfinite(p).all() for p in b.lm.module.parameters())
    finally:
        ha.close()


def test_phase0_average_tracks_baseline():
    hist = train_phase0(num_replicas=2, rounds=3, local_steps_per_round=8, seed=0)
    assert len(hist["coop"]) == 3 and hist["coop"][-1] < hist["coop"][0] + 0.05
    assert all(np.isfinite(hist["baseline"]))


def test_tokenizers():
    ct = CharTokenizer.from_text("banana")
    assert ct.chars == ["a", "b", "n"] and ct.encode("nab?") == [2, 0, 1, 0] and ct.decode([1, 0, 2, 9]) == "ban"
    assert CharTokenizer.from_json(ct.to_json()).chars == ct.chars
    with pytest.raises(ValueError):
        CharTokenizer.from_vocab(["a", "a"])
    with pytest.raises(ValueError):
        CharTokenizer.from_json('{"kind":"bpe","chars":[]}')
    bpe = BpeTokenizer.train("abababab abab", 259)
    assert bpe.merges[0] == [97, 98] and bpe.vocab_size <= 259
    text = "abab ba"
    assert bpe.decode(bpe.encode(text)) == text and len(bpe.encode(text)) < len(text)
    again = BpeTokenizer.from_json(bpe.save_json())
    assert again.encode(text) == bpe.encode(text)
    assert json.loads(bpe.save_json())["kind"] == "byte-bpe"
    with pytest.raises(ValueError):
        BpeTokenizer.train("abc", 100)
    with pytest.raises(ValueError):
        bpe.decode([100000])
    assert BpeTokenizer.train("héllo héllo", 260).decode(BpeTokenizer.train("héllo héllo", 260).encode("héllo")) == "héllo"


def test_datasets_and_loader():
    ds = TextTokenDataset.from_tokens(list(range(10)), 4)
    assert len(ds) == 6 and ds[2].input.tolist() == [2, 3, 4, 5] and ds[2].target.tolist() == [3, 4, 5, 6]
    with pytest.raises(IndexError):
        ds[6]
    with pytest.raises(ValueError):
        TextTokenDataset.from_tokens([1, 2, 3], 3)
    assert len(TextTokenDataset.from_text("hello world", CharTokenizer.from_text("hello world"), 3)) == 8
    dl = DataLoader(ListDataset(list(range(10))), batch_size=4, shuffle=True, drop_last=True, seed=3)
    b1, b2 = list(dl.batches()), list(dl.batches())
    assert len(dl) == 2 and all(len(b) == 4 for b in b1) and b1 != b2          # reshuffles on every call
    assert [len(b) for b in DataLoader(ListDataset(list(range(10))), batch_size=4).batches()] == [4, 4, 2]
    with pytest.raises(ValueError):
        DataLoader(ListDataset([1]), batch_size=0)
    xs, ys = next(DataLoader(ds, batch_size=3).pinned_batches())
    assert xs.shape == (3, 4) and torch.equal(xs[:, 1:], ys[:, :-1])
    csv = CsvDataset.from_lines(["a,b,label", "1,2,cat", "3,x,dog", ""], label_column=2, class_map={"cat": 0, "dog": 1})
    assert csv.num_features == 2 and csv[1].features.tolist() == [3.0, 0.0] and csv[1].label == 1.0
    assert csv.headers == ["a", "b", "label"]
    for bad in (lambda: CsvDataset.from_lines([]), lambda: CsvDataset.from_lines(["a,b"]),
                lambda: CsvDataset.from_lines(["a,b", "1,2", "1"]),
                lambda: CsvDataset.from_lines(["a,b", "1,zz"], label_column=1),
                lambda: CsvDataset.from_lines(["a,b", "1,2"], label_column=5)):
        with pytest.raises(ValueError):
            bad()


def test_safetensors_dtypes_metadata_shards(tmp_path):
    def blob(entries, meta=None):
        header, data, off = {}, b"", 0
        if meta:
            header["__metadata__"] = meta
        for name, (dt, shape, raw) in entries.items():
            header[name] = {"dtype": dt, "shape": shape, "data_offsets": [off, off + len(raw)]}
            data += raw
            off += len(raw)
        hj = json.dumps(header).encode()
        return struct.pack("<Q", len(hj)) + hj + data

    bf = (np.array([1.5, -2.0], dtype=np.float32).view(np.uint32) >> 16).astype("<u2").tobytes()
    raw = blob({"f32": ("F32", [2, 2], np.arange(4, dtype="<f4").tobytes()),
                "f16": ("F16", [2], np.array([0.5, 2.0], dtype="<f2").tobytes()),
                "bf16": ("BF16", [2], bf),
                "i64": ("I64", [2], np.array([7, -3], dtype="<i8").tobytes()),
                "u8": ("U8", [3], bytes([1, 2, 255])),
                "bool": ("BOOL", [2], bytes([0, 1])),
                "scalar": ("F64", [], np.array([3.25], dtype="<f8").tobytes())}, meta={"format": "pt"})
    t = SafeTensors.load_bytes(raw)
    assert t["f32"].tolist() == [[0.0, 1.0], [2.0, 3.0]] and t["f16"].tolist() == [0.5, 2.0]
    assert t["bf16"].tolist() == [1.5, -2.0] and t["i64"].tolist() == [7.0, -3.0] and t["u8"].tolist() == [1.0, 2.0, 255.0]
    assert t["bool"].tolist() == [0.0, 1.0] and t["scalar"].shape == (1,) and float(t["scalar"]) == 3.25
    assert all(v.dtype == torch.float32 for v in t.values())
    assert SafeTensors.load_bytes(raw, keep_fp16=True)["f16"].dtype == torch.float16
    assert SafeTensors.read_metadata(raw) == {"format": "pt"} and "__metadata__" not in t
    for bad in (b"123", struct.pack("<Q", 999) + b"{}", struct.pack("<Q", 2) + b"[]",
                blob({"x": ("F99", [1], b"\0\0\0\0")}), blob({"x": ("F32", [2], b"\0\0\0\0")})):
        with pytest.raises(ValueError):
            SafeTensors.load_bytes(bad)
    # round trip through the writer, and a two-shard index
    w = {"a": torch.randn(3, 2), "b": torch.randn(4)}
    p1, p2 = tmp_path / "model-00001.safetensors", tmp_path / "model-00002.safetensors"
    SafeTensors.save_file({"a": w["a"]}, str(p1))
    SafeTensors.save_file({"b": w["b"]}, str(p2), dtype="BF16")
    idx = tmp_path / "model.safetensors.index.json"
    idx.write_text(json.dumps({"metadata": {"total_size": 40}, "weight_map": {"a": p1.name, "b": p2.name}}))
    merged = SafeTensors.load_sharded(str(idx))
    assert torch.equal(merged["a"], w["a"]) and torch.allclose(merged["b"], w["b"], atol=2e-2)
    seen = []
    SafeTensors.stream_sharded(str(idx), lambda m: seen.append(sorted(m)))
    assert seen == [["a"], ["b"]]
    assert [e.name for e in SafeTensors.list_entries(str(p1))] == ["a"]
    (tmp_path / "bad.json").write_text("[]")
    with pytest.raises(ValueError):
        SafeTensors.read_shard_index(str(tmp_path / "bad.json"))


def test_image_folder_dataset(tmp_path):
    import numpy as np
    from PIL import Image
    from dart_pytorch_b200.data.image_folder import ImageFolderDataset
    from dart_pytorch_b200.models.vit import patchify
    rng = np.random.default_rng(0)
    for cname, n in (("b_cat", 5), ("a_dog", 4), ("c_empty", 0)):
        os.makedirs(tmp_path / cname)
        for i in range(n):
            arr = rng.integers(0, 256, size=(12, 10, 3), dtype=np.uint8)
            Image.fromarray(arr).save(tmp_path / cname / f"img{i}.png")
    (tmp_path / "a_dog" / "broken.jpg").write_bytes(b"not an image")
    (tmp_path / "a_dog" / "notes.txt").write_text("skip me")
    ds = ImageFolderDataset(str(tmp_path), image_size=8, patch_size=4, val_split=0.25, seed=3)
    assert ds.classes == ["a_dog", "b_cat"] and ds.num_patches == 4 and ds.patch_pixels == 48
    assert ds.num_train + ds.num_val == 9 and ds.num_val in (1, 2)   # the unreadable file is skipped wherever it falls
    s = ds[0]
    assert s.patches.shape == (4, 48) and 0.0 <= float(s.patches.min()) and float(s.patches.max()) <= 1.0
    val = ds.val_split()
    assert len(val) == ds.num_val and val.val_split() is val and len(ds) == ds.num_train
    # patch order agrees with the model-side patchify of the same image
    flat = ds._train[0][0]
    want = patchify(torch.from_numpy(flat).permute(2, 0, 1).unsqueeze(0), 4)[0]
    assert torch.allclose(ds[0].patches, want)
    t = ds.sample_triplet()
    assert t.anchor.shape == (4, 48) and t.anchor_class != t.negative_class
    with pytest.raises(ValueError):
        ImageFolderDataset(str(tmp_path), image_size=9, patch_size=4)
    with pytest.raises(ValueError):
        ImageFolderDataset(str(tmp_path / "missing"), image_size=8, patch_size=4)
