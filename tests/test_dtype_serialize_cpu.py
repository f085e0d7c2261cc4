"""CPU tests of the half-precision codec and storage tensors, DPTC checkpoints and the safetensors reader, case by
case after the reference's test/dtype_test.dart, test/serialize_test.dart and test/safetensors_test.dart."""
import json
import math
import os
import struct

import numpy as np
import pytest
import torch

import dart_pytorch_b200 as dp
from dart_pytorch_b200 import dtype as D
from dart_pytorch_b200 import nn
from dart_pytorch_b200 import ops as F
from dart_pytorch_b200.io.dptc import Checkpoint
from dart_pytorch_b200.io.safetensors import SafeTensors

T = dp.Tensor


# ------------------------------------------------------------------------------------------------ fp16 codec ---
def test_fp16_canonical_bit_patterns_both_ways():
    table = {0x0000: 0.0, 0x3C00: 1.0, 0xC000: -2.0, 0x7BFF: 65504.0, 0x0001: 2.0 ** -24, 0x0400: 2.0 ** -14,
             0x3555: 0.333251953125, 0x7C00: math.inf, 0xFC00: -math.inf}
    for bits, value in table.items():
        assert D.fp16BitsToFp32(bits) == value
        assert D.fp32ToFp16Bits(value) == bits
    assert math.isnan(D.fp16BitsToFp32(0x7E00)) and D.fp32ToFp16Bits(-0.0) == 0x8000
    assert D.fp32ToFp16Bits(70000.0) == 0x7C00 and D.fp32ToFp16Bits(1e-9) == 0            # saturate / flush
    assert D.fp32ToFp16Bits(1.0 + 2.0 ** -11) == 0x3C00 and D.fp32ToFp16Bits(1.0 + 3 * 2.0 ** -11) == 0x3C02   # ties to even


def test_fp16_round_trips_and_bulk_codec():
    g = torch.Generator().manual_seed(0)
    vals = (torch.randn(500, generator=g) * 50).tolist() + [1e-5, -1e-5, 60000.0, -60000.0]
    bits = D.fp32ListToFp16Bits(vals)
    back = D.fp16BitsListToFp32(bits)
    for v, b in zip(vals, back):
        assert abs(v - b) <= max(abs(v) * 2.0 ** -11, 2.0 ** -24)
    assert D.fp32ListToFp16Bits(back) == bits                                             # already representable
    assert bits == [D.fp32ToFp16Bits(v) for v in vals]
    want = torch.tensor(vals).half().view(torch.int16).to(torch.int32) & 0xFFFF
    assert bits == want.tolist()


# ------------------------------------------------------------------------------------- half storage tensors ---
def test_half_storage_tensor_construction_and_readonly_rules():
    h = T.fromFp16Bits([2, 2], [0x3C00, 0x4000, 0xC000, 0x3800])
    assert h.dtype == dp.DType.fp16 and h.shape == [2, 2] and h.toList() == [1.0, 2.0, -2.0, 0.5]
    with pytest.raises((ValueError, RuntimeError)):
        T.fromFp16Bits([2, 2], [0x3C00] * 3)
    f = T.fromList([2, 2], [1.0, 2.5, -3.0, 1000.0])
    r = f.toFp16().toFp32()
    assert r.dtype == dp.DType.fp32 and r.shape == [2, 2] and r.toList() == [1.0, 2.5, -3.0, 1000.0]
    with pytest.raises(RuntimeError):
        h.assign(f)
    with pytest.raises(RuntimeError):
        f.assign(h)
    c = h.clone()
    assert c.dtype == dp.DType.fp16 and c.t.data_ptr() != h.t.data_ptr() and c.toList() == h.toList()
    assert f.residentBytes == 16 and h.residentBytes == 8 and f.toFp16().residentBytes * 2 == f.residentBytes


def test_half_storage_operands_in_ops_match_fp32():
    g = torch.Generator().manual_seed(1)
    w32 = T(torch.randn(6, 4, generator=g))
    w16 = w32.toFp16()
    x = T(torch.randn(3, 6, generator=g))
    base = x.matmul(w16.toFp32())
    assert x.matmul(w16).dtype == dp.DType.fp32 and torch.equal(x.matmul(w16).t, base.t)
    assert torch.allclose(x.matmul(w16).t, x.matmul(w32).t, atol=2e-2)
    rhs = T(torch.randn(3, 6, generator=g))
    assert torch.equal((x + rhs.toFp16()).t, (x + rhs.toFp16().toFp32()).t)
    assert w16.transpose().dtype == dp.DType.fp16 and w16.transpose().shape == [4, 6]
    assert torch.equal(w16.transpose().toFp32().t, w16.toFp32().t.t())
    s = w16.sliceRows(1, 3)
    assert s.dtype == dp.DType.fp16 and s.shape == [2, 4] and torch.equal(s.toFp32().t, w16.toFp32().t[1:3])
    assert w32.sliceRows(0, 2).dtype == dp.DType.fp32
    with pytest.raises(IndexError):
        w16.sliceRows(4, 9)
    b16 = T(torch.randn(4, generator=g)).toFp16()
    y = F.linear(x.t, w16.t.t().contiguous(), b16.t)                       # Linear-style x @ W^T + b
    assert torch.allclose(y, x.t @ w16.toFp32().t + b16.toFp32().t, atol=1e-6)


def test_adopt_cpu_storage_swaps_in_half_weights_in_place():
    lin = nn.Linear(4, 3, seed=0)
    x = torch.ones(2, 4)
    want = lin(x).detach()
    p = T(lin.weight.data)
    half = T(lin.weight.data.clone()).toFp16()
    p.adoptCpuStorageFrom(half)
    assert p.dtype == dp.DType.fp16 and p.shape == [3, 4] and half.length == 0
    assert torch.allclose(F.linear(x, p.t, lin.bias.data), want, atol=1e-2)
    with pytest.raises(ValueError):
        p.adoptCpuStorageFrom(T.fromList([5], [0.0] * 5))


# ------------------------------------------------------------------------------------------------------ DPTC ---
def test_dptc_round_trip_is_byte_identical_and_header_lists_every_parameter(tmp_path):
    lin = nn.Linear(5, 3, seed=4)
    blob = Checkpoint.save_bytes(lin)
    assert blob[:4] == b"DPTC" and struct.unpack("<I", blob[4:8])[0] == 1
    hlen = struct.unpack("<I", blob[8:12])[0]
    header = json.loads(blob[12:12 + hlen])
    assert header["version"] == 1 and [p["shape"] for p in header["params"]] == [[3, 5], [1, 3]]
    assert header["totalScalars"] == 18 and len(blob) == 12 + hlen + 18 * 4
    other = nn.Linear(5, 3, seed=9)
    Checkpoint.load_into_bytes(other, blob)
    x = torch.randn(7, 5, generator=torch.Generator().manual_seed(0))
    assert torch.equal(other(x), lin(x)) and Checkpoint.save_bytes(other) == blob
    path = tmp_path / "deep" / "er" / "lin.dptc"                               # parent directories are created
    Checkpoint.save_file(lin, str(path))
    third = nn.Linear(5, 3, seed=11)
    Checkpoint.load_into_file(third, str(path))
    assert torch.equal(third.weight, lin.weight) and os.path.getsize(path) == len(blob)


def test_dptc_rejections_leave_the_module_untouched():
    lin = nn.Linear(2, 2, seed=1)
    blob = Checkpoint.save_bytes(lin)
    target = nn.Linear(2, 2, seed=2)
    before = [p.detach().clone() for p in target.parameters()]
    cases = [b"NOPE" + blob[4:],                                              # magic
             blob[:-3],                                                       # truncated data
             blob + b"\x00" * 4]                                              # trailing bytes
    for bad in cases:
        with pytest.raises(ValueError):
            Checkpoint.load_into_bytes(target, bad)
    with pytest.raises(ValueError):
        Checkpoint.load_into_bytes(nn.Linear(2, 2, bias=False), blob)         # parameter count
    with pytest.raises(ValueError):
        Checkpoint.load_into_bytes(nn.Linear(2, 3), Checkpoint.save_bytes(nn.Linear(3, 2)))   # shapes
    assert all(torch.equal(a, b) for a, b in zip(before, target.parameters()))


def test_dptc_fp16_halves_the_blob_and_old_headers_load():
    lin = nn.Linear(16, 8, seed=3)
    full, half = Checkpoint.save_bytes(lin), Checkpoint.save_bytes(lin, fp16=True)

    def data_len(b):
        return len(b) - 12 - struct.unpack("<I", b[8:12])[0]
    assert data_len(half) * 2 == data_len(full)
    other = nn.Linear(16, 8, seed=5)
    Checkpoint.load_into_bytes(other, half)
    assert other.weight.dtype == torch.float32 and torch.allclose(other.weight, lin.weight, atol=1e-3)
    assert torch.equal(other.weight, lin.weight.half().float())
    assert b'"dtype"' not in full[:12 + struct.unpack("<I", full[8:12])[0]]   # fp32 headers carry no dtype field
    Checkpoint.load_into_bytes(other, full)
    assert torch.equal(other.weight, lin.weight)


def test_dptc_model_generates_identically_after_reload(tmp_path):
    from dart_pytorch_b200 import GPT, GPTConfig
    a = GPT(GPTConfig(vocab_size=20, max_ctx=12, embed_dim=16, num_layers=1, num_heads=2, seed=1))
    Checkpoint.save_file(a, str(tmp_path / "gpt.dptc"))
    b = GPT(GPTConfig(vocab_size=20, max_ctx=12, embed_dim=16, num_layers=1, num_heads=2, seed=2))
    Checkpoint.load_into_file(b, str(tmp_path / "gpt.dptc"))
    assert a.generate([1, 2, 3], 8, temperature=0.0) == b.generate([1, 2, 3], 8, temperature=0.0)


# ----------------------------------------------------------------------------------------------- safetensors ---
def _st(entries, metadata=None) -> bytes:
    header, data = {}, b""
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, (dtype, shape, raw) in entries.items():
        header[name] = {"dtype": dtype, "shape": shape, "data_offsets": [len(data), len(data) + len(raw)]}
        data += raw
    h = json.dumps(header).encode()
    return struct.pack("<Q", len(h)) + h + data


def test_safetensors_reads_every_supported_dtype():
    f32 = np.arange(6, dtype="<f4").reshape(2, 3)
    blob = _st({
        "a": ("F32", [2, 3], f32.tobytes()),
        "b": ("F64", [2], np.array([1.5, -2.25], dtype="<f8").tobytes()),
        "c": ("BF16", [3], (np.array([1.0, -0.5, 3.140625], dtype="<f4").view("<u4") >> 16).astype("<u2").tobytes()),
        "d": ("I32", [2], np.array([7, -3], dtype="<i4").tobytes()),
        "e": ("I64", [1, 3], np.array([[0, 1, 2]], dtype="<i8").tobytes()),
        "f": ("F16", [2], np.array([0.5, 2.0], dtype="<f2").tobytes()),
    }, metadata={"format": "pt"})
    out = SafeTensors.load_bytes(blob)
    assert set(out) == {"a", "b", "c", "d", "e", "f"}                          # the metadata key is not a tensor
    assert out["a"].shape == (2, 3) and torch.equal(out["a"], torch.from_numpy(f32.copy()))
    assert out["b"].dtype == torch.float32 and out["b"].tolist() == [1.5, -2.25]
    assert out["c"].tolist() == [1.0, -0.5, 3.140625]
    assert out["d"].tolist() == [7.0, -3.0] and out["e"].shape == (1, 3) and out["e"].tolist() == [[0.0, 1.0, 2.0]]
    assert out["f"].dtype == torch.float32 and out["f"].tolist() == [0.5, 2.0]
    kept = SafeTensors.load_bytes(blob, keep_fp16=True)
    assert kept["f"].dtype == torch.float16 and kept["a"].dtype == torch.float32
    assert SafeTensors.read_metadata(blob) == {"format": "pt"}


def test_safetensors_rejections_and_entries(tmp_path):
    with pytest.raises(ValueError):
        SafeTensors.load_bytes(b"\x01\x02\x03")                               # short buffer
    with pytest.raises(ValueError):
        SafeTensors.load_bytes(struct.pack("<Q", 1000) + b"{}")               # header longer than the buffer
    with pytest.raises(ValueError, match="unsupported dtype"):
        SafeTensors.load_bytes(_st({"x": ("C64", [1], b"\0" * 8)}))
    with pytest.raises(ValueError):
        SafeTensors.load_bytes(_st({"x": ("F32", [3], b"\0" * 8)}))           # byte range does not match the shape
    blob = _st({"w": ("F32", [2, 2], np.ones(4, "<f4").tobytes()), "v": ("F16", [3], np.ones(3, "<f2").tobytes())})
    path = tmp_path / "m.safetensors"
    path.write_bytes(blob)
    entries = {e.name: e for e in SafeTensors.list_entries(str(path))}
    assert entries["w"].shape == [2, 2] and (entries["w"].begin, entries["w"].end) == (0, 16)
    assert entries["v"].dtype == "F16" and (entries["v"].begin, entries["v"].end) == (16, 22)
    assert entries["v"].num_elements == 3


def test_safetensors_sharded_loading(tmp_path):
    a = _st({"layer.0.w": ("F32", [2], np.array([1, 2], "<f4").tobytes())})
    b = _st({"layer.1.w": ("F16", [2], np.array([3, 4], "<f2").tobytes())})
    (tmp_path / "model-00001-of-00002.safetensors").write_bytes(a)
    (tmp_path / "model-00002-of-00002.safetensors").write_bytes(b)
    index = {"metadata": {"total_size": 12}, "weight_map": {"layer.0.w": "model-00001-of-00002.safetensors",
                                                            "layer.1.w": "model-00002-of-00002.safetensors"}}
    ipath = tmp_path / "model.safetensors.index.json"
    ipath.write_text(json.dumps(index))
    idx = SafeTensors.read_shard_index(str(ipath))
    assert idx.shards == ["model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors"]
    merged = SafeTensors.load_sharded(str(ipath), keep_fp16=True)
    assert merged["layer.0.w"].tolist() == [1.0, 2.0] and merged["layer.1.w"].dtype == torch.float16
    seen = []
    SafeTensors.stream_sharded(str(ipath), lambda part: seen.append(sorted(part)))
    assert seen == [["layer.0.w"], ["layer.1.w"]]


def test_small_api_parity_items(tmp_path, monkeypatch):
    from dart_pytorch_b200 import _native
    from dart_pytorch_b200.data import TextEncoder, debugPreview
    from dart_pytorch_b200.io import BertLoadReport, ClipLoadReport, GPT2LoadReport, LoadReport
    assert dp.DType.fp16.itemBytes == 2 and dp.DType.fp32.itemBytes == 4
    assert D.decodeFp16Bulk([0x3C00, 0xC000, 0x7BFF]).tolist() == [1.0, -2.0, 65504.0]
    a = T.fromList([2, 3], [1, 2, 3, 4, 5, 6], requiresGrad=True)
    b = T.fromList([3, 2], [1, 0, 0, 1, 1, 1], requiresGrad=True)
    assert a.matmul(b).debugChildShapes == [[2, 3], [3, 2]] and a.debugChildShapes == []
    assert debugPreview(range(10), 3) == "[0,1,2] ...(10 total)" and debugPreview([1, 2], 3) == "[1,2]"
    assert GPT2LoadReport is LoadReport and BertLoadReport is ClipLoadReport
    assert hasattr(TextEncoder, "encode")
    monkeypatch.setenv("DPTB200_NATIVE_LIB", str(tmp_path / "missing.so"))
    with pytest.raises(_native.NativeLibraryError):
        _native.ensureNativeLib()


def test_debug_backward_hook_fires_after_every_closure():
    """``Tensor.debug_backward_hook`` is called with a running index and a view of each backward node, in execution
    order, and is silent once removed."""
    from dart_pytorch_b200.tensor import Tensor
    a = Tensor.fromList([2, 3], [1, 2, 3, 4, 5, 6], requiresGrad=True)
    w = Tensor.fromList([3, 2], [0.5, -1, 2, 0.25, 1, 1], requiresGrad=True)
    seen = []
    Tensor.debug_backward_hook = lambda i, t: seen.append((i, t.debug_node, list(t.shape)))
    try:
        (a.matmul(w).tanh() * 2.0).sum().backward()
    finally:
        Tensor.debug_backward_hook = None
    assert [i for i, _, _ in seen] == list(range(len(seen))) and len(seen) >= 5
    names = [n for _, n, _ in seen]
    assert any("Tanh" in n for n in names) and any("Mm" in n or "Matmul" in n.title() for n in names)
    assert names.index(next(n for n in names if "Tanh" in n)) < names.index(next(n for n in names if "Mm" in n))
    assert a.grad is not None and w.grad is not None
    n = len(seen)
    b = Tensor.fromList([2], [1.0, 2.0], requiresGrad=True)
    (b * b).sum().backward()
    assert len(seen) == n
