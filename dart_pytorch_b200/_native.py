"""ctypes binding of the in-tree native library ``_C/libdptb200.so`` (sm_100a kernels).

This plays the role of the reference's FFI layer (lib/core/tensor/cuda_engine.dart:241-457) with one
difference in kind: the native side receives raw device pointers of tensors that PyTorch already owns
plus the current CUDA stream, so there is no handle table, no per-op allocation and no implicit sync.

The library is looked up at ``DPTB200_NATIVE_LIB`` (if set) and then next to this file.  When a CUDA device is
present and the library cannot be loaded, every kernel-backed op raises: there is no silent fallback.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
_LIB_ERROR: Optional[str] = None
_HERE = Path(__file__).resolve().parent

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float


class NativeLibraryError(RuntimeError):
    pass


class KernelError(RuntimeError):
    """A launcher returned a non-zero code, or a kernel recorded a failure in the device status word."""


LIB_NAME = "libdptb200.so"


def candidate_paths() -> list:
    """Discovery order (reference: lib/core/tensor/cuda_engine.dart:428-455): explicit ``DPTB200_NATIVE_LIB``, the working
    directory, the directory of the running program, then the package's own ``_C`` directory."""
    import sys
    out = []
    env = os.environ.get("DPTB200_NATIVE_LIB")
    if env:
        out.append(Path(env))
    out.append(Path.cwd() / LIB_NAME)
    if sys.argv and sys.argv[0]:
        out.append(Path(sys.argv[0]).resolve().parent / LIB_NAME)
    out.append(_HERE / "_C" / LIB_NAME)
    return out


def looks_like_shared_object(path: Path) -> bool:
    """ELF magic check, the analogue of the reference's check on a fetched library
    (lib/core/tensor/native_lib_download.dart:143-162)."""
    try:
        with open(path, "rb") as f:
            return f.read(4) == b"\x7fELF"
    except OSError:
        return False


def build_native_library() -> Optional[Path]:
    """Where the reference can fetch a prebuilt library, this build compiles its own: with ``DPTB200_AUTO_BUILD=1`` a
    missing library is built from ``csrc/`` with ``nvcc`` (when both exist) and its path returned."""
    import shutil
    import subprocess
    import sys
    script = _HERE.parent / "csrc" / "build.py"
    if os.environ.get("DPTB200_AUTO_BUILD", "0") != "1" or not script.exists() or shutil.which("nvcc") is None:
        return None
    subprocess.run([sys.executable, str(script)], check=True)
    built = _HERE / "_C" / LIB_NAME
    return built if looks_like_shared_object(built) else None


def lib_path() -> Path:
    env = os.environ.get("DPTB200_NATIVE_LIB")
    if env:                      # an explicit override is used as given, even when it does not exist (and then fails)
        return Path(env)
    for p in candidate_paths():
        if p.exists() and looks_like_shared_object(p):
            return p
    return build_native_library() or _HERE / "_C" / LIB_NAME


def ensure_native_lib() -> str:
    """Path of the native library, building it in-tree when no candidate exists (there is nothing to download: the
    library ships as source).  An environment override that points at a missing file is an error
    (reference contract: lib/core/tensor/native_lib_download.dart:35-48)."""
    env = os.environ.get("DPTB200_NATIVE_LIB")
    if env and not Path(env).exists():
        raise NativeLibraryError(f"DPTB200_NATIVE_LIB={env} does not exist")
    path = lib_path()
    if not path.exists():
        raise NativeLibraryError(f"no native library at {path}; build it with `python csrc/build.py`")
    return str(path)


ensureNativeLib = ensure_native_lib


def load(required: bool = True) -> Optional[ctypes.CDLL]:
    global _LIB, _LIB_ERROR
    if _LIB is not None:
        return _LIB
    if _LIB_ERROR is None:
        path = lib_path()
        try:
            _LIB = ctypes.CDLL(str(path))
            _declare(_LIB)
            return _LIB
        except OSError as e:  # missing file or unresolved symbol
            _LIB_ERROR = f"cannot load {path}: {e}; build it with `python csrc/build.py`"
    if required:
        raise NativeLibraryError(_LIB_ERROR)
    return None


def available() -> bool:
    return load(required=False) is not None


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("A", c_void_p), ("B", c_void_p), ("C", c_void_p), ("bias", c_void_p), ("residual", c_void_p),
        ("aux_out", c_void_p), ("aux_in", c_void_p),
        ("lda", c_ll), ("ldb", c_ll), ("ldc", c_ll), ("ldr", c_ll), ("ld_aux_out", c_ll), ("ld_aux_in", c_ll),
        ("M", c_int), ("N", c_int), ("K", c_int),
        ("trans_a", c_int), ("trans_b", c_int), ("a_f32", c_int), ("b_f32", c_int),
        ("bias_f32", c_int), ("out_f32", c_int), ("accumulate", c_int), ("act", c_int),
        ("alpha", c_float), ("force_simt", c_int), ("bn", c_int), ("splits", c_int),
        ("ws", c_void_p), ("ws_bytes", c_ll), ("counters", c_void_p), ("num_counters", c_int),
    ]


def _declare(lib: ctypes.CDLL) -> None:
    def sig(name, *argtypes):
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.argtypes = list(argtypes)
            fn.restype = c_int

    P, I, L, F = c_void_p, c_int, c_ll, c_float
    sig("dptb_gemm", ctypes.POINTER(GemmArgs), P)
    sig("dptb_gemm_skinny", ctypes.POINTER(GemmArgs), P, P)
    sig("dptb_status_read", ctypes.POINTER(c_int * 4))
    sig("dptb_status_clear")
    sig("dptb_layernorm_fwd", P, P, P, P, P, P, L, I, F, I, P)
    sig("dptb_rmsnorm_fwd", P, P, P, P, L, I, F, I, P)
    sig("dptb_layernorm_bwd", P, P, P, P, P, P, P, P, P, P, I, I, L, I, I, P, I, P)
    sig("dptb_norm_param_grad_reduce", P, I, I, P, P, I, I, P)
    sig("dptb_rmsnorm_bwd", P, P, P, P, P, P, P, P, I, I, L, I, I, P, I, P)
    sig("dptb_ce_fwd", P, L, P, P, P, L, I, I, P)
    sig("dptb_ce_bwd", P, L, P, P, P, I, F, P, L, L, I, I, I, P)
    sig("dptb_softmax_fwd", P, P, L, I, I, P)
    sig("dptb_softmax_bwd", P, P, P, L, I, I, P)
    sig("dptb_mean_f32", P, L, P, F, P)
    sig("dptb_embedding_fwd", P, L, P, P, L, I, I, P, L, I, I, P)
    sig("dptb_embedding_bwd", P, L, P, P, P, P, L, I, I, P)
    sig("dptb_pos_embedding_bwd", P, L, I, I, L, P, I, I, P)
    sig("dptb_sqnorm_parts", L)
    sig("dptb_grad_norm", P, L, I, P, P, F, I, P)
    sig("dptb_scale_by_ctrl", P, L, I, P, P)
    sig("dptb_adam_flat", P, P, P, I, P, P, L, P, F, F, F, F, F, F, F, I, P, P)
    sig("dptb_sgd_flat", P, P, P, I, P, L, P, F, F, F, I, P)
    sig("dptb_attn_fwd", P, P)
    sig("dptb_attn_bwd", P, P)
    sig("dptb_attn_decode", P, P)
    sig("dptb_binary", P, P, P, L, L, I, I, I, P)
    sig("dptb_unary", P, P, L, I, F, I, P)
    sig("dptb_unary_bwd", P, P, P, L, I, F, I, P)
    sig("dptb_colsum", P, L, P, P, L, I, I, I, I, P)
    sig("dptb_sum_all", P, L, P, P, F, I, P)
    sig("dptb_transpose2d", P, P, L, L, I, P)
    sig("dptb_copy2d", P, L, P, L, L, L, I, P)
    sig("dptb_rope", P, P, L, I, I, I, I, I, F, I, I, L, L, P, P)
    sig("dptb_dropout", P, P, L, F, ctypes.c_ulonglong, ctypes.c_ulonglong, I, P)
    sig("dptb_swiglu_fwd", P, L, P, L, P, L, L, I, I, P)
    sig("dptb_swiglu_bwd", P, L, P, L, P, L, P, L, P, L, L, I, I, P)
    sig("dptb_argmax_rows", P, L, P, L, I, I, P)
    sig("dptb_topk_sample", P, L, P, P, L, I, I, F, I, I, P)
    sig("dptb_im2col_nhwc", P, P, I, I, I, I, I, P)
    sig("dptb_conv_lower", P, P, I, I, I, I, I, I, I, I, I, I, P)
    sig("dptb_aft_fwd", P, P, P, P, P, I, I, I, I, I, P)
    sig("dptb_aft_bwd", P, P, P, P, P, P, P, P, P, I, I, I, I, I, P)
    sig("dptb_patchify", P, P, I, I, I, I, I, I, P)


# --------------------------------------------------------------------------- helpers
def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise TypeError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc > 0:
        raise KernelError(f"{what}: CUDA error {rc}")
    names = {-1: "bad shape / stride / alignment", -2: "driver entry point for tensor maps not found",
             -3: "tensor map rejected by the driver", -4: "scratch capacity exceeded", -5: "unsupported configuration"}
    raise KernelError(f"{what}: {names.get(rc, 'library error')} ({rc})")


def read_status() -> tuple:
    """(code, block, waits_timed_out, reserved) of the device status word; synchronises the device."""
    lib = load()
    buf = (c_int * 4)()
    torch.cuda.synchronize()
    check(lib.dptb_status_read(ctypes.byref(buf)), "status_read")
    return tuple(buf)


def clear_status() -> None:
    check(load().dptb_status_clear(), "status_clear")


def raise_on_device_error() -> None:
    code, block, waits, _ = read_status()
    if code != 0:
        clear_status()
        raise KernelError(f"device status {code} (block {block}, {waits} waits ran out): a bounded wait inside a kernel "
                          f"gave up; the results of that launch are invalid")
