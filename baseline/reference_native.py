"""ctypes driver for the reference's own native CUDA library (kernel-level baseline).

The reference's device code is one translation unit, ``lib/native/src/engine.cu``, exporting a C ABI over opaque
fp32 2-D tensor handles (``create_tensor(rows, cols, host_ptr)``, ``matmul_tensors(a, b)``, ``layernorm_forward`` ...:
lib/native/src/engine.cu:94-586).  Its Dart layer cannot run without a Dart SDK, but the library itself builds with
nvcc as-is.  ``build()`` compiles the unmodified source for sm_100a into ``baseline/_ref/libdart_engine.so`` and
``RefLib`` calls it the way the Dart FFI layer does (lib/core/tensor/tensor.dart: one handle per tensor, one call per
op, every result a freshly allocated handle).  Used by ``benchmarks/reference_kernels_bench.py`` only; nothing in the
package or the training / serving path imports this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "libdart_engine.so")


def build(reference_root: str, out: str = LIB_PATH) -> str:
    """Compile ``<reference_root>/lib/native/src/engine.cu`` unmodified (the reference's own build line plus the
    sm_100a target)."""
    src = os.path.join(reference_root, "lib", "native", "src", "engine.cu")
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    os.makedirs(os.path.dirname(out), exist_ok=True)
    cmd = ["nvcc", "--shared", "-Xcompiler", "-fPIC", "-O3", "-gencode", "arch=compute_100a,code=sm_100a",
           "-o", out, src]
    subprocess.run(cmd, check=True)
    return out


class RefLib:
    """Thin handle-based wrapper; every method mirrors one exported function of the reference library."""

    def __init__(self, path: Optional[str] = None):
        path = path or LIB_PATH
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path}: build it first (python -m baseline.reference_native --build <ref root>)")
        self.lib = L = ctypes.CDLL(path)
        vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.create_tensor.restype, L.create_tensor.argtypes = vp, [ci, ci, vp]
        L.destroy_tensor.restype, L.destroy_tensor.argtypes = None, [vp]
        L.get_tensor_data.restype, L.get_tensor_data.argtypes = None, [vp, vp]
        for name, args in (("matmul_tensors", [vp, vp]), ("add_tensors", [vp, vp]), ("mul_tensors", [vp, vp]),
                           ("add_tensor_row_broadcast", [vp, vp]), ("relu_tensor", [vp]), ("tanh_tensor", [vp]),
                           ("transpose_tensor", [vp]), ("sum_tensor", [vp]),
                           ("layernorm_forward", [vp, vp, vp, cf]), ("rmsnorm_forward", [vp, vp, cf]),
                           ("layernorm_backward", [vp, vp, vp, vp, vp, cf]),
                           ("softmax_forward", [vp]), ("softmax_backward", [vp, vp]),
                           ("cross_entropy_forward", [vp, vp]), ("cross_entropy_backward", [vp, vp, vp]),
                           ("embedding_forward", [vp, vp, ci]), ("aft_full_forward", [vp, vp, vp, vp, ci])):
            fn = getattr(L, name)
            fn.restype, fn.argtypes = vp, args
        L.embedding_backward.restype, L.embedding_backward.argtypes = None, [vp, vp, vp, ci]

    def tensor(self, array: np.ndarray):
        a = np.ascontiguousarray(array, dtype=np.float32)
        if a.ndim == 1:
            a = a.reshape(-1, 1)
        h = self.lib.create_tensor(a.shape[0], a.shape[1], a.ctypes.data_as(ctypes.c_void_p))
        if not h:
            raise MemoryError("create_tensor returned null")
        return h

    def zeros(self, rows: int, cols: int):
        return self.lib.create_tensor(rows, cols, None)

    def read(self, h, rows: int, cols: int) -> np.ndarray:
        out = np.empty((rows, cols), dtype=np.float32)
        self.lib.get_tensor_data(h, out.ctypes.data_as(ctypes.c_void_p))
        return out

    def free(self, *handles) -> None:
        for h in handles:
            if h:
                self.lib.destroy_tensor(h)


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--build", metavar="REFERENCE_ROOT", required=True)
    print(build(ap.parse_args().build))
