"""Helpers shared by the training demos (reference: bin/shakespeare_util.dart:1-190).

``load_corpus`` reads ``data/tiny_shakespeare.txt`` relative to the working directory when it exists and otherwise
falls back to the built-in toy corpus, so every demo runs offline.
"""
from __future__ import annotations

import os
import random
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from ..coop.shard import K_TOY_CORPUS
from ..ops.reference import sample_from_logits as _sample_row

SHAKESPEARE_PATH = "data/tiny_shakespeare.txt"
kShakespearePath = SHAKESPEARE_PATH


def load_corpus(max_chars: Optional[int] = None, path: Optional[str] = None) -> str:
    path = path or SHAKESPEARE_PATH
    if os.path.exists(path):
        with open(path, "r", encoding="utf-8") as f:
            text = f.read()
    else:
        text = K_TOY_CORPUS
    return text if max_chars is None or max_chars >= len(text) else text[:max_chars]


def get_window(ids: Sequence[int], block_size: int, rng: random.Random, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Random ``(x, y)`` with ``y`` the next-token shift of ``x``; ``start`` uniform in ``[0, len - block - 1)``."""
    max_start = len(ids) - block_size - 1
    if max_start <= 0:
        raise ValueError(f"getWindow: corpus ({len(ids)}) too short for blockSize {block_size}")
    start = rng.randrange(max_start)
    x = torch.tensor(ids[start:start + block_size], dtype=torch.long, device=device)
    y = torch.tensor(ids[start + 1:start + block_size + 1], dtype=torch.long, device=device)
    return x, y


def sample_from_logits(logits: Sequence[float], temperature: float = 1.0, top_k: Optional[int] = None,
                       rng: Optional[random.Random] = None) -> int:
    return _sample_row(torch.as_tensor(logits, dtype=torch.float32), temperature, top_k, rng or random.Random())


def last_row_logits(logits: torch.Tensor, vocab_size: int) -> List[float]:
    return logits.detach().float().reshape(-1, logits.shape[-1])[-1, :vocab_size].cpu().tolist()


def generate_text(prompt: Sequence[int], max_new_tokens: int, max_ctx: int, vocab_size: int,
                  step_fn: Callable[[List[int]], Sequence[float]], temperature: float = 1.0,
                  top_k: Optional[int] = None, rng: Optional[random.Random] = None) -> List[int]:
    """Model-agnostic sampling loop: ``step_fn(context ids)`` returns logits whose last ``vocab_size`` entries are the
    next-token row; the context slides over the last ``max_ctx`` tokens."""
    out = [int(t) for t in prompt]
    rng = rng or random.Random()
    for _ in range(max_new_tokens):
        logits = list(step_fn(out[-max_ctx:]))
        row = logits if len(logits) == vocab_size else logits[-vocab_size:]
        out.append(sample_from_logits(row, temperature, top_k, rng))
    return out


def param_scalar_count(params) -> int:
    return sum(p.numel() for p in params)


loadCorpus, getWindow, sampleFromLogits, lastRowLogits, generateText, paramScalarCount = (
    load_corpus, get_window, sample_from_logits, last_row_logits, generate_text, param_scalar_count)
