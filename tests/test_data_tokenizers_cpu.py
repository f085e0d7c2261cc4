"""CPU tests of the datasets, the loader and the three trainable / file-based tokenizers, case by case after the
reference's test/dataloader_test.dart, test/char_tokenizer_test.dart, test/bpe_tokenizer_test.dart and
test/wordpiece_tokenizer_test.dart."""
import json
import random

import pytest
import torch

from dart_pytorch_b200.data import (CsvDataset, DataLoader, ImageFolderDataset, ListDataset, TextTokenDataset)
from dart_pytorch_b200.data.hf_tokenizers import WordPieceTokenizer
from dart_pytorch_b200.data.tokenizers import BpeTokenizer, CharTokenizer


# --------------------------------------------------------------------------------------------------- loader ---
def test_list_dataset_and_loader_order_drop_last_shuffle():
    ds = ListDataset([10, 11, 12, 13, 14, 15, 16])
    assert len(ds) == 7 and ds.length == 7 and ds[3] == 13
    assert list(DataLoader(ds, batch_size=3).batches()) == [[10, 11, 12], [13, 14, 15], [16]]
    assert list(DataLoader(ds, batch_size=3, drop_last=True).batches()) == [[10, 11, 12], [13, 14, 15]]
    assert len(DataLoader(ds, batch_size=3)) == 3 and len(DataLoader(ds, batch_size=3, drop_last=True)) == 2
    a = list(DataLoader(ds, batch_size=2, shuffle=True, seed=5).batches())
    b = list(DataLoader(ds, batch_size=2, shuffle=True, seed=5).batches())
    c = list(DataLoader(ds, batch_size=2, shuffle=True, seed=6).batches())
    flat = [x for batch in a for x in batch]
    assert a == b and a != c and sorted(flat) == list(range(10, 17)) and flat != list(range(10, 17))
    # one generator per loader: every pass draws a new order, and equal seeds give equal sequences of passes
    l1, l2 = DataLoader(ds, batch_size=7, shuffle=True, seed=1), DataLoader(ds, batch_size=7, shuffle=True, seed=1)
    e1, e2 = list(l1.batches()), list(l1.batches())
    assert e1 != e2 and [e1, e2] == [list(l2.batches()), list(l2.batches())]
    assert list(DataLoader(ds, batch_size=7, shuffle=True).batches()) == list(DataLoader(ds, 7, True, seed=0).batches())
    with pytest.raises(ValueError):
        DataLoader(ds, batch_size=0)


def _image_folder(root, classes=("ann", "ben", "cy"), per_class=5, size=16):
    from PIL import Image
    g = random.Random(0)
    for c in classes:
        (root / c).mkdir()
        for k in range(per_class):
            px = bytes(g.randrange(256) for _ in range(size * size * 3))
            Image.frombytes("RGB", (size, size), px).save(root / c / f"img{k}.png")
    (root / "notes.txt").write_text("ignored")
    return root


def test_image_folder_dataset_split_patches_loader_and_triplets(tmp_path):
    root = _image_folder(tmp_path)
    ds = ImageFolderDataset(str(root), 16, 8, val_split=0.2, seed=7)
    assert ds.classes == ["ann", "ben", "cy"] and ds.num_classes == 3
    assert ds.num_train + ds.num_val == 15 and ds.num_val == 3 and len(ds) == ds.num_train
    s = ds[0]
    assert s.patches.shape == (4, 8 * 8 * 3) and 0 <= s.label < 3
    assert float(s.patches.min()) >= 0.0 and float(s.patches.max()) <= 1.0
    val = ds.val_split()
    assert len(val) == 3 and val[0].patches.shape == (4, 192)
    batches = list(DataLoader(ds, batch_size=5, shuffle=True, seed=1).batches())
    assert [len(b) for b in batches] == [5, 5, 2] and all(hasattr(x, "patches") for x in batches[0])
    t = ds.sample_triplet()
    assert t.anchor.shape == t.positive.shape == t.negative.shape == (4, 192)
    assert t.anchor_class != t.negative_class
    capped = ImageFolderDataset(str(root), 16, 8, max_per_class=2, max_classes=2, val_split=0.0)
    assert capped.num_classes == 2 and capped.num_train == 4
    with pytest.raises(ValueError):
        ImageFolderDataset(str(root), 16, 5)                        # patch size must divide the image size


def test_patchify_order_is_row_major_patches_of_dy_dx_c(tmp_path):
    from PIL import Image
    (tmp_path / "a").mkdir()
    px = bytearray()
    for y in range(4):
        for x in range(4):
            px += bytes([y * 4 + x, 100 + y * 4 + x, 200 + (y * 4 + x) % 50])
    for k in range(2):
        Image.frombytes("RGB", (4, 4), bytes(px)).save(tmp_path / "a" / f"{k}.png")
    ds = ImageFolderDataset(str(tmp_path), 4, 2, val_split=0.0)
    p = ds[0].patches * 255.0
    assert p.shape == (4, 12)
    # patch 1 = top-right 2x2 block; inside a patch: (dy, dx, c) with c fastest
    want = [2, 102, 202, 3, 103, 203, 6, 106, 206, 7, 107, 207]
    assert torch.allclose(p[1], torch.tensor(want, dtype=torch.float32), atol=1e-3)


def test_text_token_dataset_windows():
    text = "hello world, hello there"
    tok = CharTokenizer.from_text(text)
    ds = TextTokenDataset.from_text(text, tok, 5)
    ids = tok.encode(text)
    assert len(ds) == len(ids) - 5 and ds.num_tokens == len(ids)
    s = ds[3]
    assert s.input.tolist() == ids[3:8] and s.target.tolist() == ids[4:9]
    pre = TextTokenDataset.from_tokens(list(range(10)), 4)
    assert len(pre) == 6 and pre[5].target.tolist() == [6, 7, 8, 9]
    with pytest.raises(IndexError):
        pre[6]
    with pytest.raises(ValueError):
        TextTokenDataset.from_tokens([1, 2, 3], 3)
    with pytest.raises(ValueError):
        TextTokenDataset.from_text(text, object(), 4)


def test_csv_dataset_numeric_classmap_no_label_and_errors():
    ds = CsvDataset.from_lines(["f1,f2,y", "1.5,2,0", "3,4.25,1"], label_column=2)
    assert len(ds) == 2 and ds[1].features.tolist() == [3.0, 4.25] and ds[1].label == 1.0
    cm = CsvDataset.from_lines(["a,kind", "1,cat", "2,dog", "3,cat"], label_column=1, class_map={"cat": 0, "dog": 1})
    assert [cm[i].label for i in range(3)] == [0.0, 1.0, 0.0] and cm[0].features.tolist() == [1.0]
    nl = CsvDataset.from_lines(["a,b", "1,2"])
    assert nl[0].label == -1.0 and nl[0].features.tolist() == [1.0, 2.0]
    for bad in (["a,b", "1,2", "3,4,5"], ["a,b"], [], ["a,kind", "1,cat"]):     # width is set by the first data row
        with pytest.raises(ValueError):
            CsvDataset.from_lines(bad, label_column=1 if bad and "kind" in bad[0] else None)


# ----------------------------------------------------------------------------------------------- tokenizers ---
def test_char_tokenizer(tmp_path):
    tok = CharTokenizer.from_text("banana band")
    assert tok.chars == [" ", "a", "b", "d", "n"] and tok.vocab_size == 5
    ids = tok.encode("band an")
    assert tok.decode(ids) == "band an"
    assert tok.encode("bxa") == [2, 0, 1] and tok.decode([2, 99, -1, 1]) == "ba"
    again = CharTokenizer.from_json(tok.to_json())
    assert again.chars == tok.chars and json.loads(tok.to_json())["kind"] == "char"
    tok.save_file(str(tmp_path / "tok.json"))
    assert CharTokenizer.load_file(str(tmp_path / "tok.json")).encode("band") == tok.encode("band")
    with pytest.raises(ValueError):
        CharTokenizer(["a", "a"])
    with pytest.raises(ValueError):
        CharTokenizer.from_json('{"kind":"byte-bpe","chars":[]}')


def test_bpe_tokenizer_training_rules():
    with pytest.raises(ValueError):
        BpeTokenizer.train("abc", 255)
    with pytest.raises(ValueError):
        BpeTokenizer.train("", 300)
    corpus = "the cat sat on the mat. the cat ate the rat. " * 20
    tok = BpeTokenizer.train(corpus, 300)
    assert 256 < tok.vocab_size <= 300 and tok.vocab_size == 256 + len(tok.merges)
    again = BpeTokenizer.train(corpus, 300)
    assert again.merges == tok.merges                                   # deterministic
    tiny = BpeTokenizer.train("abcdefg", 400)
    assert tiny.vocab_size == 256                                       # no pair occurs twice: stops at once
    some = BpeTokenizer.train("ababab xyz", 400, min_count=3)
    assert some.vocab_size == 257 and some.merges[0] == [ord("a"), ord("b")]
    tie = BpeTokenizer.train("zyzy abab", 257)                          # equal counts: the smaller packed pair wins
    assert tie.merges[0] == [ord("a"), ord("b")]


def test_bpe_tokenizer_encode_decode_and_persistence(tmp_path):
    base = BpeTokenizer(256, [])
    assert base.encode("hi!") == list(b"hi!") and base.decode(list("héllo".encode())) == "héllo"
    corpus = "low lower lowest newer newest wide wider widest " * 30
    tok = BpeTokenizer.train(corpus, 320)
    for text in ("lower and wider", "naïve café ☕ 漢字", ""):
        assert tok.decode(tok.encode(text)) == text
    assert len(tok.encode(corpus)) < 0.6 * len(corpus.encode())
    again = BpeTokenizer.from_json(tok.save_json())
    assert again.merges == tok.merges and again.encode("lowest wide") == tok.encode("lowest wide")
    saved = json.loads(tok.save_json())
    assert saved["version"] == 1 and saved["kind"] == "byte-bpe" and saved["vocabSize"] == tok.vocab_size
    tok.save_file(str(tmp_path / "bpe.json"))
    assert BpeTokenizer.load_file(str(tmp_path / "bpe.json")).encode("newest") == tok.encode("newest")
    for bad in ({"version": 1, "kind": "char", "vocabSize": 256, "merges": []},
                {"version": 2, "kind": "byte-bpe", "vocabSize": 256, "merges": []}):
        with pytest.raises(ValueError):
            BpeTokenizer.from_json(json.dumps(bad))
    assert tok.decode([0xFF, 0xFE]) != ""                               # malformed UTF-8 decodes to replacement chars


def test_wordpiece_tokenizer(tmp_path):
    vocab = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "hello", "world", "un", "##aff", "##able", ",", "!", "play", "##ing",
             "cafe"]
    path = tmp_path / "vocab.txt"
    path.write_text("\n".join(vocab) + "\n")
    tok = WordPieceTokenizer.from_vocab_file(str(path))
    assert tok.vocab_size == len(vocab) and (tok.pad_id, tok.unk_id, tok.cls_id, tok.sep_id) == (0, 1, 2, 3)
    assert tok.encode("Hello, WORLD!") == [2, 4, 9, 5, 10, 3]                    # lowercase + punctuation split
    assert tok.tokenize("unaffable playing") == ["un", "##aff", "##able", "play", "##ing"]
    assert tok.encode("hello", add_special_tokens=False) == [4]
    assert tok.encode("Café") == [2, 13, 3]                                      # accents stripped
    assert tok.encode("hello xyzzy") == [2, 4, 1, 3]                             # whole word -> [UNK]
    assert tok.encode_pair("hello", "world !") == [2, 4, 3, 5, 10, 3]
    long = tok.encode("hello world hello world hello", max_length=4)
    assert long == [2, 4, 5, 3]                                                  # truncation keeps [CLS] ... [SEP]
    assert tok.decode([2, 6, 7, 8, 11, 12, 3, 0, 0]) == "unaffable playing"
    with pytest.raises(ValueError):
        WordPieceTokenizer(["hello", "world"])                                   # no special tokens
