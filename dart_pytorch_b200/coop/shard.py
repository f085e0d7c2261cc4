"""Corpus helpers of cooperative training: a character vocabulary, random training windows and contiguous,
non-overlapping corpus shards (reference: lib/core/coop/shard.dart:14-97)."""
from __future__ import annotations

import random
from typing import Dict, List, Sequence, Tuple

import torch

K_TOY_CORPUS = (
    "to be or not to be that is the question "
    "whether tis nobler in the mind to suffer "
    "the slings and arrows of outrageous fortune "
    "or to take arms against a sea of troubles "
    "and by opposing end them to die to sleep "
    "no more and by a sleep to say we end "
    "the heart ache and the thousand natural shocks "
    "that flesh is heir to tis a consummation "
    "devoutly to be wished to die to sleep "
    "to sleep perchance to dream ay theres the rub "
    "for in that sleep of death what dreams may come "
    "when we have shuffled off this mortal coil "
    "must give us pause theres the respect "
    "that makes calamity of so long life ")
kToyCorpus = K_TOY_CORPUS


class CharVocab:
    def __init__(self, itos: Sequence[str]):
        self.itos: List[str] = list(itos)
        self.stoi: Dict[str, int] = {c: i for i, c in enumerate(self.itos)}

    @property
    def size(self) -> int:
        return len(self.itos)

    @classmethod
    def from_text(cls, text: str) -> "CharVocab":
        return cls(sorted(set(text)))

    @classmethod
    def from_itos(cls, itos: Sequence[str]) -> "CharVocab":
        return cls(itos)

    fromText, fromItos = from_text, from_itos

    def encode(self, s: str) -> List[float]:
        return [float(self.stoi.get(c, 0)) for c in s]

    def decode(self, ids: Sequence[float]) -> str:
        return "".join(self.itos[min(max(int(v), 0), self.size - 1)] for v in ids)


def sample_window(ids: Sequence[float], block_size: int, rng: random.Random, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """A random ``(x, y)`` pair of ``block_size`` ids with ``y`` shifted by one."""
    max_start = len(ids) - block_size - 1
    if max_start <= 0:
        raise ValueError(f"sampleWindow: corpus ({len(ids)}) too short for blockSize {block_size}")
    start = rng.randrange(max_start)
    x = torch.tensor([int(v) for v in ids[start:start + block_size]], dtype=torch.long, device=device)
    y = torch.tensor([int(v) for v in ids[start + 1:start + 1 + block_size]], dtype=torch.long, device=device)
    return x, y


def shard_slice(ids: Sequence[float], shard_index: int, num_shards: int) -> List[float]:
    """Shard ``shard_index`` of ``num_shards`` equal contiguous pieces; the last shard takes the remainder."""
    if num_shards <= 0 or shard_index < 0 or shard_index >= num_shards:
        raise ValueError(f"shardSlice: shardIndex={shard_index}, numShards={num_shards}")
    size = len(ids) // num_shards
    start = shard_index * size
    end = len(ids) if shard_index == num_shards - 1 else start + size
    return list(ids[start:end])


sampleWindow, shardSlice = sample_window, shard_slice
