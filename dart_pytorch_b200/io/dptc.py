"""DPTC checkpoints, bit-compatible with the reference (lib/core/nn/serialize.dart:37-227).

Layout: ``"DPTC"`` | u32 LE version (1) | u32 LE header length | UTF-8 JSON header | data.  The header is the compact
JSON ``{"version":1,"params":[{"shape":[...]}...],"totalScalars":N}`` (with ``"dtype":"F16"`` per parameter when saved
in half precision); the data block holds the parameters back to back in ``module.reference_parameters()`` order as
little-endian fp32 (or IEEE half).  Loading validates magic, version, parameter count, every shape, every dtype and
the exact data length before it writes anything, then copies in place so tensor identity (and optimizer state) is kept.
"""
from __future__ import annotations

import json
import os
import struct
from typing import List

import numpy as np
import torch

from ..dtype import fp32_to_fp16_bits

MAGIC = b"DPTC"
VERSION = 1


def _ref_params(module) -> List[torch.Tensor]:
    if hasattr(module, "reference_parameters"):
        return list(module.reference_parameters())
    return [p.data for p in module.parameters()]


def _master_values(view: torch.Tensor, module) -> torch.Tensor:
    """fp32 values for a checkpoint view: the arena's fp32 master copy when the view lives in a bf16 arena."""
    arena = None
    for p in module.parameters():
        arena = getattr(p, "_dptb_arena", None)
        break
    if arena is not None and arena.master is not None and view.dtype != torch.float32:
        base = arena.flat.data_ptr()
        off = (view.data_ptr() - base) // arena.flat.element_size()
        if 0 <= off < arena.numel:
            m = torch.as_strided(arena.master, view.shape, view.stride(), off)
            return m.detach().float().cpu().contiguous()
    return view.detach().float().cpu().contiguous()


class Checkpoint:
    @staticmethod
    def save_bytes(module, fp16: bool = False) -> bytes:
        params = _ref_params(module)
        entries, total = [], 0
        for p in params:
            e = {"shape": [int(s) for s in p.shape]}
            if fp16:
                e["dtype"] = "F16"
            entries.append(e)
            total += p.numel()
        header = json.dumps({"version": VERSION, "params": entries, "totalScalars": total},
                            separators=(",", ":")).encode("utf-8")
        chunks = [MAGIC, struct.pack("<I", VERSION), struct.pack("<I", len(header)), header]
        for p in params:
            vals = _master_values(p, module).reshape(-1)
            if fp16:
                chunks.append(fp32_to_fp16_bits(vals).numpy().astype("<i2").tobytes())
            else:
                chunks.append(vals.numpy().astype("<f4").tobytes())
        return b"".join(chunks)

    @staticmethod
    def save_file(module, path: str, fp16: bool = False) -> None:
        parent = os.path.dirname(os.path.abspath(path))
        os.makedirs(parent, exist_ok=True)
        with open(path, "wb") as f:
            f.write(Checkpoint.save_bytes(module, fp16=fp16))

    @staticmethod
    def parse_header(data: bytes):
        """Validate the preamble and return ``(header_dict, data_offset)``."""
        if len(data) < 12:
            raise ValueError("Checkpoint: buffer too small for a DPTC preamble")
        if data[:4] != MAGIC:
            raise ValueError("Checkpoint: bad magic (not a DPTC file)")
        version, hlen = struct.unpack("<II", data[4:12])
        if version != VERSION:
            raise ValueError(f"Checkpoint: unsupported version {version}")
        if 12 + hlen > len(data):
            raise ValueError("Checkpoint: truncated header")
        try:
            header = json.loads(data[12:12 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise ValueError(f"Checkpoint: malformed header: {e}") from e
        return header, 12 + hlen

    @staticmethod
    def load_into_bytes(module, data: bytes) -> None:
        header, off = Checkpoint.parse_header(data)
        params = _ref_params(module)
        entries = header.get("params")
        if not isinstance(entries, list) or len(entries) != len(params):
            raise ValueError(f"Checkpoint: parameter count mismatch (file {len(entries) if isinstance(entries, list) else '?'}"
                             f", module {len(params)})")
        sizes, halfs = [], []
        expected = 0
        for i, (e, p) in enumerate(zip(entries, params)):
            shape = e.get("shape")
            if not isinstance(shape, list) or [int(s) for s in shape] != [int(s) for s in p.shape]:
                raise ValueError(f"Checkpoint: shape mismatch at parameter {i}: file {shape}, module {list(p.shape)}")
            dt = e.get("dtype", "F32")
            if dt not in ("F32", "F16"):
                raise ValueError(f"Checkpoint: unsupported dtype {dt!r} at parameter {i}")
            half = dt == "F16"
            n = p.numel()
            sizes.append(n)
            halfs.append(half)
            expected += n * (2 if half else 4)
        if len(data) - off != expected:
            raise ValueError(f"Checkpoint: data length {len(data) - off} != expected {expected}")
        touched_arena = None
        with torch.no_grad():
            for p, n, half in zip(params, sizes, halfs):
                if half:
                    arr = np.frombuffer(data, dtype="<f2", count=n, offset=off).astype(np.float32)
                    off += 2 * n
                else:
                    arr = np.frombuffer(data, dtype="<f4", count=n, offset=off)
                    off += 4 * n
                src = torch.from_numpy(arr.copy()).reshape(p.shape)
                p.copy_(src.to(device=p.device, dtype=p.dtype))
                _write_master(module, p, src)
        for q in module.parameters():
            touched_arena = getattr(q, "_dptb_arena", None)
            break

    @staticmethod
    def load_into_file(module, path: str) -> None:
        with open(path, "rb") as f:
            Checkpoint.load_into_bytes(module, f.read())

    # camelCase names of the reference
    saveBytes = save_bytes
    saveFile = save_file
    loadIntoBytes = load_into_bytes
    loadIntoFile = load_into_file


def _write_master(module, view: torch.Tensor, src_f32: torch.Tensor) -> None:
    """Keep the arena's fp32 master copy exact when loading into a bf16 model."""
    arena = None
    for p in module.parameters():
        arena = getattr(p, "_dptb_arena", None)
        break
    if arena is None or arena.master is None:
        return
    base = arena.flat.data_ptr()
    off = (view.data_ptr() - base) // arena.flat.element_size()
    if 0 <= off < arena.numel:
        m = torch.as_strided(arena.master, view.shape, view.stride(), off)
        m.copy_(src_f32.to(m.device))
