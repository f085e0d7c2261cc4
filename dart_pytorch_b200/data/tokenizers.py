"""Character and byte-level BPE tokenizers (reference: lib/core/data/char_tokenizer.dart, bpe_tokenizer.dart).

JSON formats are the reference's: ``{"version":1,"kind":"char","chars":[...]}`` and
``{"version":1,"kind":"byte-bpe","vocabSize":N,"merges":[[a,b],...]}``.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence, Tuple


class CharTokenizer:
    def __init__(self, chars: Sequence[str]):
        self.chars: List[str] = list(chars)
        self._stoi: Dict[str, int] = {c: i for i, c in enumerate(self.chars)}
        if len(self._stoi) != len(self.chars):
            raise ValueError("CharTokenizer.fromVocab: chars must be unique")

    @property
    def vocab_size(self) -> int:
        return len(self.chars)

    vocabSize = vocab_size

    @classmethod
    def from_text(cls, text: str) -> "CharTokenizer":
        return cls(sorted(set(text)))

    @classmethod
    def from_vocab(cls, chars: Sequence[str]) -> "CharTokenizer":
        return cls(chars)

    def encode(self, s: str) -> List[int]:
        """Unknown characters map to id 0."""
        return [self._stoi.get(ch, 0) for ch in s]

    def decode(self, ids: Sequence[int]) -> str:
        return "".join(self.chars[int(i)] for i in ids if 0 <= int(i) < len(self.chars))

    def to_json(self) -> str:
        return json.dumps({"version": 1, "kind": "char", "chars": self.chars}, separators=(",", ":"),
                          ensure_ascii=False)

    @classmethod
    def from_json(cls, s: str) -> "CharTokenizer":
        obj = json.loads(s)
        if obj.get("kind") != "char":
            raise ValueError(f"CharTokenizer.fromJson: kind is {obj.get('kind')}")
        return cls(obj["chars"])

    def save_file(self, path: str) -> None:
        with open(path, "w", encoding="utf-8") as f:
            f.write(self.to_json())

    @classmethod
    def load_file(cls, path: str) -> "CharTokenizer":
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_json(f.read())

    fromText, fromVocab, toJson, fromJson, saveFile, loadFile = from_text, from_vocab, to_json, from_json, save_file, load_file


def _pair_key(a: int, b: int) -> int:
    return (a << 20) | (b & 0xFFFFF)


class BpeTokenizer:
    """Byte-level BPE trained on the whole corpus as one sequence (no pre-tokenisation).

    Training picks the most frequent adjacent pair, ties going to the smaller packed key ``(a << 20) | b``, stops when the
    best count drops below ``min_count`` or the vocabulary is full, and applies each merge left to right without
    overlaps.  Encoding repeatedly merges the adjacent pair of lowest rank (leftmost on ties), one occurrence per pass.
    """

    def __init__(self, vocab_size: int, merges: Sequence[Sequence[int]]):
        self.vocab_size = int(vocab_size)
        self.merges: List[List[int]] = [[int(a), int(b)] for a, b in merges]
        self._rank: Dict[int, int] = {_pair_key(a, b): r for r, (a, b) in enumerate(self.merges)}

    vocabSize = property(lambda self: self.vocab_size)

    @classmethod
    def train(cls, corpus: str, target_vocab_size: int, min_count: int = 2) -> "BpeTokenizer":
        if target_vocab_size < 256:
            raise ValueError(f"BpeTokenizer.train: targetVocabSize must be >= 256; got {target_vocab_size}")
        seq = list(corpus.encode("utf-8"))
        if not seq:
            raise ValueError("BpeTokenizer.train: corpus is empty")
        merges: List[List[int]] = []
        next_id = 256
        while next_id < target_vocab_size:
            counts: Dict[int, int] = {}
            for i in range(len(seq) - 1):
                k = _pair_key(seq[i], seq[i + 1])
                counts[k] = counts.get(k, 0) + 1
            if not counts:
                break
            best_key, best_count = -1, 0
            for k, c in counts.items():
                if c > best_count or (c == best_count and (best_key == -1 or k < best_key)):
                    best_count, best_key = c, k
            if best_count < min_count:
                break
            a, b = best_key >> 20, best_key & 0xFFFFF
            merges.append([a, b])
            merged, i = [], 0
            while i < len(seq):
                if i + 1 < len(seq) and seq[i] == a and seq[i + 1] == b:
                    merged.append(next_id)
                    i += 2
                else:
                    merged.append(seq[i])
                    i += 1
            seq = merged
            next_id += 1
        return cls(next_id, merges)

    def encode(self, text: str) -> List[int]:
        seq = list(text.encode("utf-8"))
        while len(seq) >= 2:
            best_rank, best_i = 1 << 30, -1
            for i in range(len(seq) - 1):
                r = self._rank.get(_pair_key(seq[i], seq[i + 1]))
                if r is not None and r < best_rank:
                    best_rank, best_i = r, i
            if best_i == -1:
                break
            seq = seq[:best_i] + [256 + best_rank] + seq[best_i + 2:]
        return seq

    def _expand(self, out: List[int], tid: int) -> None:
        if tid < 256:
            out.append(tid)
            return
        rank = tid - 256
        if rank >= len(self.merges):
            raise ValueError(f"BpeTokenizer.decode: unknown token id {tid}")
        self._expand(out, self.merges[rank][0])
        self._expand(out, self.merges[rank][1])

    def decode(self, tokens: Sequence[int]) -> str:
        out: List[int] = []
        for t in tokens:
            self._expand(out, int(t))
        return bytes(out).decode("utf-8", errors="replace")

    def save_json(self) -> str:
        return json.dumps({"version": 1, "kind": "byte-bpe", "vocabSize": self.vocab_size, "merges": self.merges},
                          separators=(",", ":"))

    def save_file(self, path: str) -> None:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w", encoding="utf-8") as f:
            f.write(self.save_json())

    @classmethod
    def from_json(cls, s: str) -> "BpeTokenizer":
        data = json.loads(s)
        if data.get("kind") != "byte-bpe":
            raise ValueError(f'BpeTokenizer.fromJson: expected kind "byte-bpe", got {data.get("kind")}')
        if data.get("version") != 1:
            raise ValueError(f"BpeTokenizer.fromJson: unsupported version {data.get('version')}")
        return cls(int(data["vocabSize"]), data["merges"])

    @classmethod
    def load_file(cls, path: str) -> "BpeTokenizer":
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_json(f.read())

    saveJson, saveFile, fromJson, loadFile = save_json, save_file, from_json, load_file
