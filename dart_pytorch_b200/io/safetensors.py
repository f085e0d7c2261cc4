"""Safetensors reader (and a small writer for fixtures / exports) with shard-index support
(reference: lib/core/nn/safetensors.dart:92-530).

File layout: ``u64 LE header length`` | JSON header ``{name: {dtype, shape, data_offsets:[begin,end]}, "__metadata__":
{...}}`` | data.  Every supported dtype (F32, F64, F16, BF16, U8, BOOL, I8, I32, U32, I64, U64) is converted to fp32;
``keep_fp16=True`` keeps F16 tensors as half storage.  Scalars ``[]`` become shape ``[1]``.  The file is memory-mapped,
so loading a shard never copies it whole (the reference reads the file into RAM and decodes element by element).
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import numpy as np
import torch

METADATA_KEY = "__metadata__"

_NP_DTYPES = {"F32": "<f4", "F64": "<f8", "F16": "<f2", "U8": "u1", "BOOL": "u1", "I8": "i1", "I32": "<i4",
              "U32": "<u4", "I64": "<i8", "U64": "<u8", "BF16": "<u2", "I16": "<i2", "U16": "<u2"}


@dataclass
class SafeTensorEntry:
    name: str
    dtype: str
    shape: List[int]
    begin: int
    end: int

    @property
    def num_elements(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


@dataclass
class ShardIndex:
    weight_map: Dict[str, str]
    metadata: Dict[str, object]
    index_path: str

    @property
    def shards(self) -> List[str]:
        seen, out = set(), []
        for v in self.weight_map.values():
            if v not in seen:
                seen.add(v)
                out.append(v)
        return out

    shardFiles = shard_files = shards


def _data_offset(buf) -> int:
    if len(buf) < 8:
        raise ValueError(f"safetensors: buffer too small ({len(buf)} bytes)")
    (hlen,) = struct.unpack("<Q", bytes(buf[:8]))
    if 8 + hlen > len(buf):
        raise ValueError(f"safetensors: invalid headerLen={hlen} for buffer {len(buf)}")
    return 8 + hlen


def _header_json(buf) -> dict:
    off = _data_offset(buf)
    try:
        decoded = json.loads(bytes(buf[8:off]).decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise ValueError(f"safetensors: malformed header: {e}") from e
    if not isinstance(decoded, dict):
        raise ValueError(f"safetensors: header is not a JSON object (got {type(decoded).__name__})")
    return decoded


def _parse_header(buf) -> List[SafeTensorEntry]:
    entries = []
    for name, v in _header_json(buf).items():
        if name == METADATA_KEY:
            continue
        if not isinstance(v, dict):
            raise ValueError(f'safetensors: entry "{name}" is not an object')
        if "dtype" not in v:
            raise ValueError(f'safetensors: entry "{name}" missing "dtype"')
        shape = v.get("shape")
        offs = v.get("data_offsets")
        if not isinstance(shape, list) or not isinstance(offs, list) or len(offs) != 2:
            raise ValueError(f'safetensors: entry "{name}" has malformed shape / data_offsets')
        entries.append(SafeTensorEntry(name, str(v["dtype"]), [int(s) for s in shape], int(offs[0]), int(offs[1])))
    return entries


def _read_tensor(buf, data_off: int, e: SafeTensorEntry, keep_fp16: bool) -> torch.Tensor:
    if e.dtype not in _NP_DTYPES:
        raise ValueError(f'safetensors: unsupported dtype "{e.dtype}" for "{e.name}"')
    npdt = np.dtype(_NP_DTYPES[e.dtype])
    n = e.num_elements
    if e.end - e.begin != n * npdt.itemsize or data_off + e.end > len(buf):
        raise ValueError(f'safetensors: entry "{e.name}" has inconsistent byte range')
    arr = np.frombuffer(buf, dtype=npdt, count=n, offset=data_off + e.begin)
    shape = e.shape if e.shape else [1]
    if e.dtype == "BF16":
        t = torch.from_numpy(arr.astype(np.int32) << 16).view(torch.float32)
    elif e.dtype == "F16" and keep_fp16:
        t = torch.from_numpy(arr.copy())
    elif e.dtype in ("U64", "U32"):
        t = torch.from_numpy(arr.astype(np.float64)).to(torch.float32)
    else:
        t = torch.from_numpy(arr.astype(np.float32))
    return t.reshape(shape)


class SafeTensors:
    metadataKey = METADATA_KEY

    @staticmethod
    def load_bytes(data, keep_fp16: bool = False) -> Dict[str, torch.Tensor]:
        buf = memoryview(data)
        off = _data_offset(buf)
        return {e.name: _read_tensor(buf, off, e, keep_fp16) for e in _parse_header(buf)}

    @staticmethod
    def load_file(path: str, keep_fp16: bool = False) -> Dict[str, torch.Tensor]:
        mm = np.memmap(path, dtype=np.uint8, mode="r")
        return SafeTensors.load_bytes(mm, keep_fp16=keep_fp16)

    @staticmethod
    def list_entries(path: str) -> List[SafeTensorEntry]:
        mm = np.memmap(path, dtype=np.uint8, mode="r")
        return _parse_header(memoryview(mm))

    @staticmethod
    def read_metadata(data) -> Dict[str, str]:
        meta = _header_json(memoryview(data)).get(METADATA_KEY)
        return {str(k): str(v) for k, v in meta.items()} if isinstance(meta, dict) else {}

    @staticmethod
    def read_shard_index(index_path: str) -> ShardIndex:
        with open(index_path, "r", encoding="utf-8") as f:
            decoded = json.load(f)
        if not isinstance(decoded, dict):
            raise ValueError(f"safetensors: shard index is not a JSON object (got {type(decoded).__name__})")
        wm = decoded.get("weight_map")
        if not isinstance(wm, dict):
            raise ValueError('safetensors: shard index missing "weight_map" object')
        md = decoded.get("metadata")
        return ShardIndex({str(k): str(v) for k, v in wm.items()}, dict(md) if isinstance(md, dict) else {}, index_path)

    @staticmethod
    def load_sharded(index_path: str, keep_fp16: bool = False) -> Dict[str, torch.Tensor]:
        merged: Dict[str, torch.Tensor] = {}
        SafeTensors.stream_sharded(index_path, merged.update, keep_fp16=keep_fp16)
        return merged

    @staticmethod
    def stream_sharded(index_path: str, on_shard: Callable[[Dict[str, torch.Tensor]], None],
                       keep_fp16: bool = False) -> None:
        """Load one shard at a time and hand it to ``on_shard``: peak memory is one shard, not the model."""
        index = SafeTensors.read_shard_index(index_path)
        base = os.path.dirname(os.path.abspath(index_path))
        for shard in index.shards:
            on_shard(SafeTensors.load_file(os.path.join(base, shard), keep_fp16=keep_fp16))

    @staticmethod
    def save_bytes(tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None,
                   dtype: str = "F32") -> bytes:
        """Serialise tensors as F32, F16 or BF16 (used for exports and for synthetic test fixtures)."""
        header, chunks, off = {}, [], 0
        if metadata:
            header[METADATA_KEY] = {str(k): str(v) for k, v in metadata.items()}
        for name, t in tensors.items():
            t = t.detach().cpu()
            if dtype == "F32":
                raw = t.float().contiguous().numpy().astype("<f4").tobytes()
            elif dtype == "F16":
                raw = t.to(torch.float16).contiguous().numpy().astype("<f2").tobytes()
            elif dtype == "BF16":
                raw = (t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().astype("<i2")).tobytes()
            else:
                raise ValueError(f"safetensors: cannot write dtype {dtype}")
            header[name] = {"dtype": dtype, "shape": [int(s) for s in t.shape], "data_offsets": [off, off + len(raw)]}
            chunks.append(raw)
            off += len(raw)
        hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
        hj += b" " * ((8 - len(hj) % 8) % 8)
        return struct.pack("<Q", len(hj)) + hj + b"".join(chunks)

    @staticmethod
    def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata=None, dtype: str = "F32") -> None:
        with open(path, "wb") as f:
            f.write(SafeTensors.save_bytes(tensors, metadata, dtype))

    # camelCase names of the reference
    loadBytes = load_bytes
    loadFile = load_file
    listEntries = list_entries
    readMetadata = read_metadata
    readShardIndex = read_shard_index
    loadSharded = load_sharded
    streamSharded = stream_sharded
