"""GPU test of the allocation-free column sum (``dptb_colsum_static``).

Callers that cannot allocate while they run (inside a graph capture, a serving loop that must not synchronise, a host
application that owns the device memory pool) get one entry point whose scratch is a fixed array inside the library.
The test calls it through its exported C symbol, twice in a row so the second call runs over the first call's leftovers
in the shared scratch, and compares each result with the existing scratch-taking entry point ``dptb_colsum`` and with a
plain fp32 column sum; it also checks that the device's free memory does not move across calls.
This file sorts last on purpose: a run that stops at the first failure has then already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from dart_pytorch_b200 import _native
    lib = _native.load(required=True)
    fn = lib.dptb_colsum_static
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return _native, fn


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_colsum_static_matches_scratch_version_on_two_calls_in_a_row(dtype):
    from dart_pytorch_b200.ops import kernels as K
    native, fn = _lib()
    code = 0 if dtype == torch.float32 else 1
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(11)
    # two different shapes back to back: the second call reuses (and must not be confused by) the first call's partials
    for rows, cols, ld in ((4096, 3072, 3072), (1000, 777, 800)):
        x = torch.randn(rows, ld, device="cuda", generator=g).to(dtype)
        want = K.colsum(x, n_cols=cols).float()
        plain = x[:, :cols].float().sum(0)               # independent of this library's kernels
        assert float((want - plain).norm() / (plain.norm() + 1e-12)) < tol
        got = torch.full((cols,), float("nan"), dtype=dtype, device="cuda")
        rc = fn(x.data_ptr(), ld, got.data_ptr(), rows, cols, 0, code, stream)
        assert rc == 0
        torch.cuda.synchronize()
        err = float((got.float() - want).norm() / (want.norm() + 1e-12))
        assert err < tol, (rows, cols, err)
        assert float((got.float() - plain).norm() / (plain.norm() + 1e-12)) < tol
        # accumulate on top of an existing value
        base = torch.ones(cols, dtype=dtype, device="cuda")
        assert fn(x.data_ptr(), ld, base.data_ptr(), rows, cols, 1, code, stream) == 0
        torch.cuda.synchronize()
        err = float((base.float() - (want + 1.0)).norm() / ((want + 1.0).norm() + 1e-12))
        assert err < tol * 2
    native.raise_on_device_error()


def test_colsum_static_allocates_no_device_memory():
    """Once the first call on the device has resolved the scratch address, further calls leave the driver's count of
    free device memory exactly where it was (torch's caching allocator is not involved: the buffers exist before)."""
    _, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    x = torch.randn(2048, 1024, device="cuda")
    out = torch.empty(1024, device="cuda")
    assert fn(x.data_ptr(), 1024, out.data_ptr(), 2048, 1024, 0, 0, stream) == 0     # first call: set-up done here
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert fn(x.data_ptr(), 1024, out.data_ptr(), 2048, 1024, 0, 0, stream) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert float((out - x.sum(0)).abs().max()) < 1e-2


def test_colsum_static_rejects_sizes_beyond_its_fixed_scratch():
    _, fn = _lib()
    cols = 8192 + 64
    x = torch.zeros(8, cols, device="cuda")
    out = torch.full((cols,), 7.0, device="cuda")
    rc = fn(x.data_ptr(), cols, out.data_ptr(), 8, cols, 0, 0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == -4                      # refused with the capacity error ...
    assert float(out.min()) == 7.0       # ... and nothing was launched
    ok = torch.empty(8192, device="cuda")
    assert fn(x.data_ptr(), cols, ok.data_ptr(), 8, 8192, 0, 0, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert float(ok.abs().max()) == 0.0
