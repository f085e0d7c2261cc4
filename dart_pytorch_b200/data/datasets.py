"""Datasets and the batching loader (reference: lib/core/data/dataset.dart, text_token_dataset.dart, csv_dataset.dart).

Samples are ``torch`` tensors.  ``DataLoader.batches()`` reshuffles with its own seeded generator on every call, as the
reference does; ``DataLoader.pinned_batches()`` is the device-feeding variant: it stacks each batch into pinned host
memory so the host-to-device copy of the next batch overlaps the current step.
"""
from __future__ import annotations

import random
from dataclasses import dataclass
from typing import Dict, Generic, Iterator, List, Optional, Sequence, TypeVar

import torch

T = TypeVar("T")


class Dataset(Generic[T]):
    def __len__(self) -> int:
        raise NotImplementedError

    def __getitem__(self, index: int) -> T:
        raise NotImplementedError

    @property
    def length(self) -> int:
        return len(self)


class ListDataset(Dataset[T]):
    def __init__(self, items: Sequence[T]):
        self._items = list(items)

    def __len__(self):
        return len(self._items)

    def __getitem__(self, index):
        return self._items[index]


class DataLoader(Generic[T]):
    def __init__(self, dataset: Dataset[T], batch_size: int = 1, shuffle: bool = False, drop_last: bool = False,
                 seed: Optional[int] = None):
        if batch_size < 1:
            raise ValueError(f"batchSize must be >= 1, got {batch_size}")
        self.dataset, self.batch_size, self.shuffle, self.drop_last = dataset, batch_size, shuffle, drop_last
        self._rng = random.Random(seed or 0)

    def __len__(self) -> int:
        n = len(self.dataset)
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size

    length = property(__len__)

    def batches(self) -> Iterator[List[T]]:
        n = len(self.dataset)
        order = list(range(n))
        if self.shuffle:
            self._rng.shuffle(order)
        for start in range(0, n, self.batch_size):
            end = min(start + self.batch_size, n)
            if self.drop_last and end - start < self.batch_size:
                break
            yield [self.dataset[order[k]] for k in range(start, end)]

    __iter__ = batches

    def pinned_batches(self):
        """Yield ``(inputs, targets)`` stacked into pinned host tensors (for ``LmSample``-like datasets)."""
        for batch in self.batches():
            xs = torch.stack([b.input for b in batch])
            ys = torch.stack([b.target for b in batch])
            if torch.cuda.is_available():
                xs, ys = xs.pin_memory(), ys.pin_memory()
            yield xs, ys


@dataclass
class LmSample:
    input: torch.Tensor    # [blockSize] token ids
    target: torch.Tensor   # [blockSize] the same window shifted by one


class TextEncoder:
    """What ``TextTokenDataset.from_text`` needs of a tokenizer: ``encode(str) -> list[int]``; every tokenizer of the
    package satisfies it (reference: lib/core/data/text_token_dataset.dart:27-29)."""

    def encode(self, text: str) -> List[int]:
        raise NotImplementedError


class TextTokenDataset(Dataset[LmSample]):
    """Sliding next-token windows over a token stream; ``len = numTokens - blockSize``."""

    def __init__(self, tokens: Sequence[int], block_size: int, device=None):
        if block_size < 1:
            raise ValueError(f"blockSize must be >= 1, got {block_size}")
        if len(tokens) <= block_size:
            raise ValueError(f"need > blockSize tokens for at least one example, got {len(tokens)} tokens with "
                             f"blockSize={block_size}")
        self.tokens = torch.tensor(list(tokens), dtype=torch.long)
        self.block_size, self.device = block_size, device

    @property
    def num_tokens(self) -> int:
        return int(self.tokens.numel())

    numTokens = num_tokens

    @classmethod
    def from_text(cls, text: str, tokenizer, block_size: int, device=None):
        if not hasattr(tokenizer, "encode"):
            raise ValueError(f"tokenizer must expose `encode(str) -> list[int]`; got {type(tokenizer).__name__}")
        return cls(tokenizer.encode(text), block_size, device)

    @classmethod
    def from_file(cls, path: str, tokenizer, block_size: int, device=None):
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_text(f.read(), tokenizer, block_size, device)

    @classmethod
    def from_tokens(cls, tokens: Sequence[int], block_size: int, device=None):
        return cls(tokens, block_size, device)

    fromText, fromFile, fromTokens = from_text, from_file, from_tokens

    def __len__(self):
        return self.num_tokens - self.block_size

    def __getitem__(self, index: int) -> LmSample:
        if index < 0 or index >= len(self):
            raise IndexError(f"index {index} out of range [0, {len(self) - 1}]")
        x = self.tokens[index:index + self.block_size]
        y = self.tokens[index + 1:index + 1 + self.block_size]
        if self.device is not None:
            x, y = x.to(self.device), y.to(self.device)
        return LmSample(x, y)


@dataclass
class CsvSample:
    features: torch.Tensor   # [numFeatures]
    label: float             # -1 when there is no label column


class CsvDataset(Dataset[CsvSample]):
    def __init__(self, rows: List[List[float]], labels: List[float], num_features: int, headers: List[str], device=None):
        self._rows = torch.tensor(rows, dtype=torch.float32)
        self._labels = labels
        self.num_features, self.headers, self.device = num_features, headers, device

    @property
    def num_examples(self) -> int:
        return self._rows.shape[0]

    numExamples = num_examples

    @classmethod
    def from_file(cls, path: str, **kw):
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_lines(f.read().splitlines(), **kw)

    @classmethod
    def from_lines(cls, lines: Sequence[str], label_column: Optional[int] = None,
                   class_map: Optional[Dict[str, int]] = None, has_header: bool = True, delimiter: str = ",",
                   device=None):
        if not lines:
            raise ValueError("CsvDataset: empty input")
        headers: List[str] = []
        start = 0
        if has_header:
            headers = lines[0].split(delimiter)
            start = 1
        if start >= len(lines):
            raise ValueError("CsvDataset: no data rows")
        total_cols = len(lines[start].split(delimiter))
        if label_column is not None and not (0 <= label_column < total_cols):
            raise ValueError(f"labelColumn={label_column} out of range [0, {total_cols})")
        num_features = total_cols if label_column is None else total_cols - 1
        rows, labels = [], []
        for i in range(start, len(lines)):
            line = lines[i].strip()
            if not line:
                continue
            cells = line.split(delimiter)
            if len(cells) != total_cols:
                raise ValueError(f"row {i}: expected {total_cols} columns, got {len(cells)}")
            feats, label = [], -1.0
            for c, cell in enumerate(cells):
                raw = cell.strip()
                if c == label_column:
                    if class_map is not None:
                        if raw not in class_map:
                            raise ValueError(f'row {i} col {c}: label "{raw}" not in classMap')
                        label = float(class_map[raw])
                    else:
                        try:
                            label = float(raw)
                        except ValueError:
                            raise ValueError(f'row {i} col {c}: label "{raw}" is not numeric (pass a classMap for '
                                             f"categorical labels)") from None
                else:
                    try:
                        feats.append(float(raw))
                    except ValueError:
                        feats.append(0.0)
            rows.append(feats)
            labels.append(label)
        if not rows:
            raise ValueError("CsvDataset: parsed 0 data rows")
        return cls(rows, labels, num_features, headers, device)

    fromFile, fromLines = from_file, from_lines

    def __len__(self):
        return self._rows.shape[0]

    def __getitem__(self, index: int) -> CsvSample:
        f = self._rows[index]
        return CsvSample(f.to(self.device) if self.device is not None else f, self._labels[index])
