"""Weighted averaging of DPTC checkpoints: the merge step of cooperative (DiLoCo-style) training
(reference: lib/core/coop/param_avg.dart:20-123).

All inputs must be fp32 DPTC blobs of equal length whose preamble + JSON header are byte-identical; weights must be
non-negative and are renormalised to sum to one (uniform by default).  The output is the first blob's header followed
by the weighted mean of the data, accumulated in float32 in input order (the reference's arithmetic)."""
from __future__ import annotations

import struct
from typing import List, Optional, Sequence

import numpy as np


def average_checkpoints(checkpoints: Sequence[bytes], weights: Optional[Sequence[float]] = None) -> bytes:
    if not checkpoints:
        raise ValueError("averageCheckpoints: no inputs")
    if weights is not None and len(weights) != len(checkpoints):
        raise ValueError(f"averageCheckpoints: weights length {len(weights)} != checkpoints length {len(checkpoints)}")
    if weights is None:
        ws = [1.0 / len(checkpoints)] * len(checkpoints)
    else:
        for w in weights:
            if w < 0:
                raise ValueError(f"averageCheckpoints: negative weight {w}")
        total = float(sum(weights))
        if total <= 0:
            raise ValueError(f"averageCheckpoints: weights sum to {total}")
        ws = [float(w) / total for w in weights]
    first = bytes(checkpoints[0])
    if len(first) < 12:
        raise ValueError("averageCheckpoints: checkpoint 0 too small")
    if first[:4] != b"DPTC":
        raise ValueError("averageCheckpoints: bad DPTC magic")
    (header_len,) = struct.unpack("<I", first[8:12])
    header_end = 12 + header_len
    if len(first) < header_end:
        raise ValueError("averageCheckpoints: checkpoint 0 truncated header")
    data_len = len(first) - header_end
    if data_len % 4:
        raise ValueError("averageCheckpoints: checkpoint 0 data blob not float32-aligned")
    n = data_len // 4
    head = first[:header_end]
    for i, c in enumerate(checkpoints[1:], start=1):
        c = bytes(c)
        if len(c) != len(first):
            raise ValueError(f"averageCheckpoints: checkpoint {i} has length {len(c)} but checkpoint 0 has {len(first)}")
        if c[:header_end] != head:
            b = next(k for k in range(header_end) if c[k] != head[k])
            raise ValueError(f"averageCheckpoints: checkpoint {i} header differs at byte {b}")
    acc = np.zeros(n, dtype=np.float32)
    for w, c in zip(ws, checkpoints):
        acc += np.frombuffer(bytes(c), dtype="<f4", count=n, offset=header_end) * np.float32(w)
    return head + acc.astype("<f4").tobytes()


averageCheckpoints = average_checkpoints
