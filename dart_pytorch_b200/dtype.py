"""IEEE half-precision codec with the reference's conventions: round to nearest even, overflow saturates to +-Inf,
NaN encodes as 0x7e00 (reference: lib/core/tensor/dtype.dart:32-170)."""
from __future__ import annotations

from typing import Iterable, List

import torch


def fp32_to_fp16_bits(x: torch.Tensor) -> torch.Tensor:
    """fp32 tensor -> int16 tensor of half bit patterns."""
    h = x.detach().float().cpu().to(torch.float16)  # RNE, saturates to inf
    bits = h.view(torch.int16).clone()
    nan = torch.isnan(x.detach().float().cpu())
    bits[nan] = 0x7E00
    return bits


def fp16_bits_to_fp32(bits: torch.Tensor) -> torch.Tensor:
    return bits.to(torch.int16).view(torch.float16).float()


def fp32ToFp16Bits(value: float) -> int:
    return int(fp32_to_fp16_bits(torch.tensor([value]))[0].item()) & 0xFFFF


def fp16BitsToFp32(bits: int) -> float:
    b = bits & 0xFFFF
    if b >= 0x8000:
        b -= 0x10000
    return float(fp16_bits_to_fp32(torch.tensor([b], dtype=torch.int16))[0].item())


def fp32ListToFp16Bits(values: Iterable[float]) -> List[int]:
    t = fp32_to_fp16_bits(torch.tensor(list(values), dtype=torch.float32))
    return [int(v) & 0xFFFF for v in t.tolist()]


def fp16BitsListToFp32(bits: Iterable[int]) -> List[float]:
    arr = [(b & 0xFFFF) - (0x10000 if (b & 0xFFFF) >= 0x8000 else 0) for b in bits]
    return fp16_bits_to_fp32(torch.tensor(arr, dtype=torch.int16)).tolist()


def decodeFp16Bulk(bits) -> torch.Tensor:
    """Half bit patterns (tensor, array or list of ints) -> fp32 tensor, the bulk form of ``fp16BitsToFp32``
    (reference: lib/core/tensor/dtype.dart:122-170)."""
    if not isinstance(bits, torch.Tensor):
        bits = torch.as_tensor(list(bits), dtype=torch.int32)
    return fp16_bits_to_fp32((bits.to(torch.int32) & 0xFFFF).to(torch.int16))


decode_fp16_bulk = decodeFp16Bulk
