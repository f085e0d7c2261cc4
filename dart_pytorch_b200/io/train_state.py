"""Training-state sidecar: everything a resume needs that the DPTC checkpoint does not carry.

The reference checkpoint holds parameters only -- no optimizer moments, step counter, scheduler state or RNG
(lib/core/nn/serialize.dart:37-227; resume there means re-creating the optimizer from scratch).  The DPTC file stays
bit-compatible and parameter-only; this sidecar (``.dpts``) sits next to it:

    "DPTS" | u32 version = 1 | u32 header_len | UTF-8 JSON header | raw little-endian tensor blobs

The JSON lists the blobs ``{name, dtype, shape, offset, nbytes}`` plus scalar state: optimizer kind, step, lr and hyper
parameters, scheduler class / step count, Python / torch CPU / CUDA RNG states (hex), and free-form ``extra``.
Adam moments and SGD momentum are stored per parameter in ``parameters()`` order, so a sidecar written with a flat
parameter arena loads into an optimizer without one and vice versa.  The fp32 master copy of bf16 parameters is
stored too, so a resumed run continues from the exact master values rather than from their bf16 rounding.
"""
from __future__ import annotations

import json
import os
import random
import struct
from typing import Dict, List, Optional

import torch

MAGIC = b"DPTS"
VERSION = 1
_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I64": torch.int64, "U8": torch.uint8}
_NAMES = {v: k for k, v in _DTYPES.items()}


def _moment_views(opt):
    """``[(name, [tensor per parameter])]`` of the optimizer's per-parameter state, in ``parameters()`` order."""
    out = []
    params = opt.parameters
    arena = getattr(opt, "arena", None)

    def per_param(flat):
        return [flat[arena.offsets[id(p)]:arena.offsets[id(p)] + p.numel()].view(p.shape) for p in params]
    if arena is not None:
        for name in ("m", "v", "buf"):
            flat = getattr(opt, name, None)
            if not isinstance(flat, torch.Tensor):
                flat = getattr(opt, "_" + name, None)        # SGD keeps its flat momentum buffer as `_buf`
            if isinstance(flat, torch.Tensor) and flat.numel() == arena.numel:
                out.append((name, per_param(flat)))
        if arena.master is not None:
            out.append(("master", per_param(arena.master)))
    else:
        # SGD without an arena keeps its momentum per parameter in `_velocity`
        for name, store in (("m", getattr(opt, "_m", None)), ("v", getattr(opt, "_v", None)),
                            ("buf", getattr(opt, "_velocity", None))):
            if isinstance(store, dict) and store:
                out.append((name, [store.get(id(p)) for p in params]))
    return out


def save_train_state(path: str, optimizer=None, scheduler=None, extra: Optional[dict] = None,
                     include_rng: bool = True) -> None:
    header: Dict[str, object] = {"version": VERSION, "tensors": [], "extra": extra or {}}
    blobs: List[bytes] = []
    offset = 0

    def add(name: str, t: torch.Tensor):
        nonlocal offset
        c = t.detach().contiguous().cpu()
        raw = c.view(torch.uint8).numpy().tobytes() if c.numel() else b""
        header["tensors"].append({"name": name, "dtype": _NAMES[c.dtype], "shape": list(c.shape), "offset": offset,
                                  "nbytes": len(raw)})
        blobs.append(raw)
        offset += len(raw)
    if optimizer is not None:
        o = {"kind": type(optimizer).__name__, "lr": float(optimizer.lr), "step": int(getattr(optimizer, "_step", getattr(optimizer, "_steps", 0))),
             "num_params": len(optimizer.parameters)}
        for k in ("beta1", "beta2", "eps", "weight_decay", "momentum"):
            if hasattr(optimizer, k):
                o[k] = float(getattr(optimizer, k))
        o["shapes"] = [list(p.shape) for p in optimizer.parameters]
        header["optimizer"] = o
        for name, views in _moment_views(optimizer):
            for i, t in enumerate(views):
                if t is not None:
                    add(f"opt.{name}.{i}", t)
    if scheduler is not None:
        header["scheduler"] = {"kind": type(scheduler).__name__, "step_count": int(scheduler.step_count),
                               "last_lr": float(getattr(scheduler, "last_lr", optimizer.lr if optimizer else 0.0))}
    if include_rng:
        rng = {"python": json.dumps(random.getstate()), "torch_cpu": torch.get_rng_state().numpy().tobytes().hex()}
        if torch.cuda.is_available():
            rng["torch_cuda"] = [s.cpu().numpy().tobytes().hex() for s in torch.cuda.get_rng_state_all()]
        try:
            from ..ops import cuda as _cu
            rng["kernel_rng"] = dict(_cu._rng_state)
        except Exception:
            pass
        header["rng"] = rng
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    parent = os.path.dirname(os.path.abspath(path))
    os.makedirs(parent, exist_ok=True)
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<II", VERSION, len(hj)) + hj)
        for b in blobs:
            f.write(b)


def load_train_state(path: str, optimizer=None, scheduler=None, restore_rng: bool = True) -> dict:
    """Validate everything first (magic, version, parameter count and shapes, blob sizes), then write in place.
    Returns the header's ``extra`` dict."""
    with open(path, "rb") as f:
        data = f.read()
    if len(data) < 12 or data[:4] != MAGIC:
        raise ValueError("train state: bad magic (not a DPTS file)")
    version, hlen = struct.unpack("<II", data[4:12])
    if version != VERSION:
        raise ValueError(f"train state: unsupported version {version}")
    if 12 + hlen > len(data):
        raise ValueError("train state: truncated header")
    header = json.loads(data[12:12 + hlen].decode("utf-8"))
    body = memoryview(data)[12 + hlen:]
    tensors = {}
    for e in header["tensors"]:
        if e["dtype"] not in _DTYPES:
            raise ValueError(f"train state: unsupported dtype {e['dtype']}")
        if e["offset"] + e["nbytes"] > len(body):
            raise ValueError(f"train state: blob {e['name']} exceeds the file")
        dt = _DTYPES[e["dtype"]]
        n = 1
        for s in e["shape"]:
            n *= s
        if n * torch.empty(0, dtype=dt).element_size() != e["nbytes"]:
            raise ValueError(f"train state: blob {e['name']} has {e['nbytes']} bytes for shape {e['shape']}")
        raw = bytes(body[e["offset"]:e["offset"] + e["nbytes"]])
        tensors[e["name"]] = torch.frombuffer(bytearray(raw), dtype=dt).reshape(e["shape"]) if n else \
            torch.empty(e["shape"], dtype=dt)
    if optimizer is not None:
        o = header.get("optimizer")
        if o is None:
            raise ValueError("train state: file holds no optimizer state")
        if o["kind"] != type(optimizer).__name__:
            raise ValueError(f"train state: saved for {o['kind']}, loading into {type(optimizer).__name__}")
        if o["num_params"] != len(optimizer.parameters) or o["shapes"] != [list(p.shape) for p in optimizer.parameters]:
            raise ValueError("train state: parameter count or shapes differ from the optimizer's")
        targets = dict(_moment_views(optimizer))
        arena = getattr(optimizer, "arena", None)
        with torch.no_grad():
            for name in ("m", "v", "buf", "master"):
                for i, p in enumerate(optimizer.parameters):
                    src = tensors.get(f"opt.{name}.{i}")
                    if src is None:
                        continue
                    if name in targets and targets[name][i] is not None:
                        targets[name][i].copy_(src.to(targets[name][i].device))
                    elif arena is None and name != "master":
                        store = getattr(optimizer, "_velocity" if name == "buf" else f"_{name}", None)
                        if isinstance(store, dict):
                            store[id(p)] = src.to(device=p.device, dtype=p.dtype if name == "buf" else torch.float32
                                                  if p.dtype == torch.float32 else p.dtype).clone()
            if arena is not None and arena.master is not None and any(k.startswith("opt.master.") for k in tensors):
                arena.sync_to_params()
        optimizer.lr = float(o["lr"])
        if hasattr(optimizer, "_steps"):
            # SGD: its first step *overwrites* the momentum buffer with the gradient, so a restored buffer must not be
            # taken for a first step
            loaded_buf = any(k.startswith("opt.buf.") for k in tensors)
            optimizer._steps = max(int(o["step"]), 1 if loaded_buf else 0)
        else:
            optimizer._step = int(o["step"])
        for k in ("beta1", "beta2", "eps", "weight_decay", "momentum"):
            if k in o and hasattr(optimizer, k):
                setattr(optimizer, k, float(o[k]))
    if scheduler is not None and "scheduler" in header:
        s = header["scheduler"]
        if s["kind"] != type(scheduler).__name__:
            raise ValueError(f"train state: saved scheduler {s['kind']}, loading into {type(scheduler).__name__}")
        scheduler.step_count = int(s["step_count"])
        if hasattr(scheduler, "last_lr"):
            try:
                scheduler.last_lr = float(s["last_lr"])
            except AttributeError:
                pass
    if restore_rng and "rng" in header:
        rng = header["rng"]
        st = json.loads(rng["python"])
        random.setstate((st[0], tuple(st[1]), st[2]))
        torch.set_rng_state(torch.frombuffer(bytearray(bytes.fromhex(rng["torch_cpu"])), dtype=torch.uint8))
        if "torch_cuda" in rng and torch.cuda.is_available() and len(rng["torch_cuda"]) == torch.cuda.device_count():
            torch.cuda.set_rng_state_all([torch.frombuffer(bytearray(bytes.fromhex(h)), dtype=torch.uint8)
                                          for h in rng["torch_cuda"]])
        if "kernel_rng" in rng:
            try:
                from ..ops import cuda as _cu
                _cu._rng_state.update({k: int(v) for k, v in rng["kernel_rng"].items()})
            except Exception:
                pass
    return header.get("extra", {})
