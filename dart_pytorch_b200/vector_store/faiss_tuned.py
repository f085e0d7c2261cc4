"""Cheap header inspection of FAISS-layout files and the tuning-metadata wrapper around them.

``probe_faiss_index`` reads the fourcc and the common header (37 bytes for float indexes, 25 for binary ones) without
decoding the payload.  The ``IxDT`` wrapper stores the operating points of an auto-tune sweep in front of an ordinary
FAISS blob, so that a loader can restore the chosen ``nprobe`` / ``efSearch``; ``strip_tuning_wrapper`` gives the plain
blob back for consumers that do not know the wrapper.

Wrapper layout (little endian): ``u32 "IxDT" | u32 version = 1 | u64 tuning_len | tuning | inner FAISS blob``;
tuning block: ``i64 created_at_us | i32 metric (0 = inner product, 1 = L2) | u32 n | n x {i32 value, u32 len, utf-8
label, f64 recall, f64 mean_us} | u8 has_chosen [| i32 chosen]``
(reference: lib/core/vector_store/faiss_io.dart:2105-2415 probe, :2752-3143 wrapper).
"""
from __future__ import annotations

import enum
import struct
from dataclasses import dataclass, field
from datetime import datetime, timedelta, timezone
from typing import List, Optional, Tuple

from .base import Index, Metric
from .faiss_io import FaissFourcc, read_faiss_index_bytes, write_faiss_index_bytes
from .hnsw import IndexHNSW
from .composite import IndexRefineFlat
from .quantized import IndexIVFFlat, IndexIVFPQ
from .tools import OperatingPoint, OperatingPoints, TuneMResult

IXDT = FaissFourcc.of("IxDT")
IXDT_VERSION = 1
_EPOCH = datetime(1970, 1, 1, tzinfo=timezone.utc)
FLOAT_FOURCCS = ("IxF2", "IxFI", "IxFl", "IxMp", "IxM2", "IxPT", "IxPq", "IxSQ", "IxRF", "IwFl", "IwPQ", "IxHe", "IHNf")
BINARY_FOURCCS = ("IBxF", "IBwF")


class FaissIndexKind(enum.Enum):
    float_index = "floatIndex"
    binary_index = "binaryIndex"
    tuned_wrapper = "tunedWrapper"
    unknown = "unknown"


@dataclass
class TuningMetadata:
    created_at: datetime
    metric: Metric
    points: List[OperatingPoint] = field(default_factory=list)
    chosen_param_value: Optional[int] = None

    @classmethod
    def from_operating_points(cls, points: OperatingPoints, metric: Metric, chosen_param_value: Optional[int] = None,
                              created_at: Optional[datetime] = None) -> "TuningMetadata":
        return cls(created_at or datetime.now(timezone.utc), metric, list(points.points), chosen_param_value)

    @classmethod
    def from_tune_m_result(cls, result: TuneMResult, metric: Metric,
                           created_at: Optional[datetime] = None) -> "TuningMetadata":
        chosen = None if result.chosen is None else result.chosen.param_value
        return cls(created_at or datetime.now(timezone.utc), metric, list(result.points.points), chosen)

    fromOperatingPoints, fromTuneMResult = from_operating_points, from_tune_m_result


@dataclass
class FaissIndexInfo:
    fourcc: int
    fourcc_str: str
    kind: FaissIndexKind
    d: Optional[int] = None
    ntotal: Optional[int] = None
    metric: Optional[Metric] = None
    is_trained: Optional[bool] = None
    code_size: Optional[int] = None
    tuning: Optional[TuningMetadata] = None
    inner: Optional["FaissIndexInfo"] = None


# ---------------------------------------------------------------------------------------------- tuning block ---
def _micros(t: datetime) -> int:
    if t.tzinfo is None:
        t = t.replace(tzinfo=timezone.utc)
    delta = t - _EPOCH
    return (delta.days * 86400 + delta.seconds) * 1_000_000 + delta.microseconds


def _encode_tuning(meta: TuningMetadata) -> bytes:
    out = [struct.pack("<qiI", _micros(meta.created_at), 0 if meta.metric == Metric.inner_product else 1,
                       len(meta.points))]
    for p in meta.points:
        label = p.param_label.encode("utf-8")
        out.append(struct.pack("<iI", int(p.param_value), len(label)) + label + struct.pack("<dd", p.recall, p.mean_us))
    out.append(b"\x00" if meta.chosen_param_value is None else b"\x01" + struct.pack("<i", meta.chosen_param_value))
    return b"".join(out)


def _decode_tuning(data: bytes) -> TuningMetadata:
    try:
        micros, metric_code, n = struct.unpack_from("<qiI", data, 0)
        off = 16
        points = []
        for _ in range(n):
            value, ln = struct.unpack_from("<iI", data, off)
            off += 8
            if off + ln > len(data):
                raise struct.error("label runs past the tuning block")
            label = data[off:off + ln].decode("utf-8")
            off += ln
            recall, mean_us = struct.unpack_from("<dd", data, off)
            off += 16
            points.append(OperatingPoint(value, label, recall, mean_us))
        (flag,) = struct.unpack_from("<B", data, off)
        chosen = struct.unpack_from("<i", data, off + 1)[0] if flag == 1 else None
    except (struct.error, UnicodeDecodeError) as e:
        raise ValueError(f"IxDT: malformed tuning block: {e}") from e
    created = _EPOCH + timedelta(microseconds=micros)
    return TuningMetadata(created, Metric.inner_product if metric_code == 0 else Metric.l2, points, chosen)


def _split_wrapper(data: bytes, who: str) -> Tuple[bytes, int]:
    """Validate the wrapper header; returns (tuning bytes, offset of the inner blob)."""
    if len(data) < 4:
        raise ValueError(f"{who}: blob is {len(data)} bytes, need at least 4 for the fourcc")
    (tag,) = struct.unpack_from("<I", data, 0)
    if tag != IXDT:
        raise ValueError(f'{who}: expected fourcc "IxDT" but got "{FaissFourcc.name(tag)}": this blob is not a tuned '
                         f'wrapper')
    if len(data) < 16:
        raise ValueError(f"{who}: IxDT wrapper header truncated: need 4 (version) + 8 (tuning length) bytes after "
                         f"the fourcc")
    version, tuning_len = struct.unpack_from("<IQ", data, 4)
    if version != IXDT_VERSION:
        raise ValueError(f"{who}: unsupported IxDT wrapper version {version} (this build handles {IXDT_VERSION})")
    if len(data) - 16 < tuning_len:
        raise ValueError(f"{who}: tuning block declares {tuning_len} bytes but only {len(data) - 16} remain")
    return bytes(data[16:16 + tuning_len]), 16 + tuning_len


# --------------------------------------------------------------------------------------------------- wrapper ---
def is_tuned_faiss_blob(data: bytes) -> bool:
    return len(data) >= 4 and struct.unpack_from("<I", data, 0)[0] == IXDT


def write_tuned_faiss_index_bytes(inner: Index, meta: TuningMetadata) -> bytes:
    tuning = _encode_tuning(meta)
    return struct.pack("<IIQ", IXDT, IXDT_VERSION, len(tuning)) + tuning + write_faiss_index_bytes(inner)


def read_tuned_faiss_index_bytes(data: bytes, apply_tuning: bool = False) -> Tuple[Index, TuningMetadata]:
    tuning, start = _split_wrapper(data, "readTunedFaissIndex")
    meta = _decode_tuning(tuning)
    index = read_faiss_index_bytes(bytes(data[start:]))
    if apply_tuning:
        apply_tuning_to_index(index, meta)
    return index, meta


def save_tuned_faiss_index(path: str, inner: Index, meta: TuningMetadata) -> None:
    with open(path, "wb") as f:
        f.write(write_tuned_faiss_index_bytes(inner, meta))


def load_tuned_faiss_index(path: str, apply_tuning: bool = False) -> Tuple[Index, TuningMetadata]:
    with open(path, "rb") as f:
        return read_tuned_faiss_index_bytes(f.read(), apply_tuning=apply_tuning)


def strip_tuning_wrapper(data: bytes) -> bytes:
    """The inner FAISS blob, byte for byte; the tuning block is discarded."""
    _, start = _split_wrapper(data, "stripTuningWrapper")
    return bytes(data[start:])


def strip_tuning_wrapper_file(in_path: str, out_path: str) -> None:
    with open(in_path, "rb") as f:
        plain = strip_tuning_wrapper(f.read())
    with open(out_path, "wb") as f:
        f.write(plain)


def apply_tuning_to_index(index: Index, meta: TuningMetadata) -> bool:
    """Set the chosen ``nprobe`` / ``efSearch`` on ``index`` (through an ``IndexRefineFlat`` wrapper if need be).
    Returns False when nothing was chosen or the swept parameter is not a search-time one (e.g. PQ ``m``)."""
    chosen = meta.chosen_param_value
    if chosen is None:
        return False
    point = next((p for p in meta.points if p.param_value == chosen), None)
    if point is None:
        raise ValueError(f"applyTuningToIndex: chosen paramValue {chosen} is not present in TuningMetadata.points")
    label = point.param_label.lower()
    if label.startswith("nprobe"):
        target = index.base if isinstance(index, IndexRefineFlat) else index
        if not isinstance(target, (IndexIVFFlat, IndexIVFPQ)):
            raise ValueError(f"applyTuningToIndex: no nprobe setter for {type(index).__name__}")
        target.nprobe = chosen
        return True
    if label.startswith("efsearch"):
        if not isinstance(index, IndexHNSW):
            raise ValueError(f"applyTuningToIndex: no efSearch setter for {type(index).__name__}")
        index.ef_search = chosen
        return True
    return False


# ----------------------------------------------------------------------------------------------------- probe ---
def probe_faiss_index(data: bytes) -> FaissIndexInfo:
    if len(data) < 4:
        raise ValueError(f"probeFaissIndex: blob is {len(data)} bytes, need at least 4 for the fourcc")
    (tag,) = struct.unpack_from("<I", data, 0)
    name = FaissFourcc.name(tag)
    if tag == IXDT:
        tuning, start = _split_wrapper(data, "probeFaissIndex")
        inner = probe_faiss_index(bytes(data[start:]))
        return FaissIndexInfo(tag, name, FaissIndexKind.tuned_wrapper, inner.d, inner.ntotal, inner.metric,
                              inner.is_trained, inner.code_size, _decode_tuning(tuning), inner)
    if name in FLOAT_FOURCCS:
        if len(data) < 37:
            raise ValueError(f'probeFaissIndex: blob is {len(data)} bytes but the float "{name}" header needs 4 + 33')
        d, ntotal, _, _, trained, mt = struct.unpack_from("<iqqqBi", data, 4)
        metric = Metric.l2 if mt == 1 else (Metric.inner_product if mt == 0 else None)
        return FaissIndexInfo(tag, name, FaissIndexKind.float_index, d, ntotal, metric, trained != 0)
    if name in BINARY_FOURCCS:
        if len(data) < 25:
            raise ValueError(f'probeFaissIndex: blob is {len(data)} bytes but the binary "{name}" header needs 4 + 21')
        d, code_size, ntotal, trained, mt = struct.unpack_from("<iiqBi", data, 4)
        metric = Metric.l2 if mt == 1 else (Metric.inner_product if mt == 0 else None)
        return FaissIndexInfo(tag, name, FaissIndexKind.binary_index, d, ntotal, metric, trained != 0, code_size)
    return FaissIndexInfo(tag, name, FaissIndexKind.unknown)


def probe_faiss_index_file(path: str) -> FaissIndexInfo:
    """Reads 37 bytes of a plain file; a wrapped file is read whole (its tuning block has no fixed size)."""
    with open(path, "rb") as f:
        head = f.read(37)
        if is_tuned_faiss_blob(head):
            head += f.read()
    return probe_faiss_index(head)


isTunedFaissBlob, writeTunedFaissIndexToBytes, readTunedFaissIndexFromBytes = (
    is_tuned_faiss_blob, write_tuned_faiss_index_bytes, read_tuned_faiss_index_bytes)
saveTunedFaissIndex, loadTunedFaissIndex, stripTuningWrapper, stripTuningWrapperFile = (
    save_tuned_faiss_index, load_tuned_faiss_index, strip_tuning_wrapper, strip_tuning_wrapper_file)
applyTuningToIndex, probeFaissIndex, probeFaissIndexFile = apply_tuning_to_index, probe_faiss_index, probe_faiss_index_file
