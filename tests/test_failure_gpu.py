"""Device-side failure reporting: a bounded wait that runs out records a status code, the kernel returns, the host
raises, and the CUDA context stays usable.  Nothing here faults, traps or hangs the GPU: the wait is on a flag that no
one sets and gives up after its time limit."""
import time

import pytest
import torch

from dart_pytorch_b200 import _native as N
from dart_pytorch_b200.ops import kernels as K

pytestmark = pytest.mark.gpu


def test_flag_wait_times_out_into_status_word():
    lib = N.load()
    import ctypes
    from dart_pytorch_b200.parallel.dp_fused import _declare
    _declare(lib)
    nb, world = 1, 2
    pad = torch.zeros(int(lib.dptb_dp_pad_words(nb)), dtype=torch.int32, device="cuda")   # done flags never raised
    epochs = torch.ones(nb, dtype=torch.int32, device="cuda")                              # ... but epoch 1 expected
    ctrl = torch.zeros(4, dtype=torch.float32, device="cuda")
    N.raise_on_device_error()
    t0 = time.time()
    N.check(lib.dptb_dp_finalize(pad.data_ptr(), epochs.data_ptr(), nb, world, ctypes.c_float(1.0), ctrl.data_ptr(),
                                 0, N.stream_ptr()), "dp_finalize")          # wait limit 0: the default (one second)
    torch.cuda.synchronize()
    took = time.time() - t0
    assert 0.5 < took < 10.0                      # the wait is bounded (about one second), not endless
    with pytest.raises(N.KernelError):
        N.raise_on_device_error()                 # reports the recorded code and clears it
    N.raise_on_device_error()                     # clean again
    assert not torch.isfinite(ctrl[0])            # the kernel marked its result unusable
    # the context is intact: an ordinary kernel still runs and is correct
    a = torch.randn(256, 128, device="cuda").bfloat16()
    b = torch.randn(192, 128, device="cuda").bfloat16()
    c = torch.empty(256, 192, device="cuda", dtype=torch.bfloat16)
    K.gemm(a, b, c, trans_b=True)
    assert torch.allclose(c.float(), a.float() @ b.float().t(), atol=0.5, rtol=2e-2)
