"""Kernels writing into canary-padded outputs on odd shapes: nothing outside the payload may change."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from dart_pytorch_b200.ops import decode as D
from dart_pytorch_b200.ops import kernels as K
from dart_pytorch_b200.utils import guard


def _mk(shape, dtype=torch.bfloat16, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(dtype)


@pytest.mark.parametrize("M,N,Kd", [(77, 40, 72), (1000, 760, 264), (128, 256, 64), (300, 8, 96), (33, 768, 4096),
                                    (512, 3072, 768)])
def test_gemm_outputs_stay_inside_their_buffers(M, N, Kd):
    a, w = _mk((M, Kd), seed=1), _mk((N, Kd), seed=2, scale=0.05)
    bias, res = _mk((N,), seed=3), _mk((M, N), seed=4)
    with guard.guarded() as pool:
        out = pool.empty((M, N), torch.bfloat16, "cuda")
        K.gemm(a, w, out, trans_b=True, bias=bias, residual=res)
        aux = pool.empty((M, N), torch.bfloat16, "cuda")
        out2 = pool.empty((M, N), torch.bfloat16, "cuda")
        K.gemm(a, w, out2, trans_b=True, bias=bias, act="gelu_tanh_d", aux_out=aux)
        out3 = pool.empty((M, N), torch.float32, "cuda")
        K.gemm(a, w, out3, trans_b=True)
        dw = pool.empty((N, Kd), torch.bfloat16, "cuda")
        dw.zero_()
        K.gemm(res, a, dw, trans_a=True, accumulate=True)          # weight-gradient form, split-K when it pays
    ref = a.float() @ w.float().t() + bias.float() + res.float()
    assert float((out.float() - ref).abs().max()) <= 0.02 * float(ref.abs().max()) + 0.05


@pytest.mark.parametrize("rows,D", [(9, 100), (17, 4096), (33, 768), (16384, 768)])
def test_norm_and_reduction_outputs_stay_inside_their_buffers(rows, D):
    x, dy = _mk((rows, D), seed=1), _mk((rows, D), seed=2)
    g = (1.0 + 0.1 * _mk((D,), torch.float32, seed=3)).bfloat16()
    b = (0.1 * _mk((D,), torch.float32, seed=4)).bfloat16()
    y, mean, rstd = K.layernorm_fwd(x, g, b, 1e-5)
    with guard.guarded() as pool:
        dg = pool.empty((D,), torch.bfloat16, "cuda")
        db = pool.empty((D,), torch.bfloat16, "cuda")
        dg.zero_()
        db.zero_()
        K.layernorm_bwd(x, dy, g, mean, rstd, dgamma=dg, dbeta=db, accumulate=True)
        cs = pool.empty((D,), torch.bfloat16, "cuda")
        K.colsum(dy, out=cs)
        yo = pool.empty((rows, D), torch.bfloat16, "cuda")
        K.rmsnorm_fwd(x, g, 1e-6, out=yo)
    assert float((cs.float() - dy.float().sum(0)).abs().max()) <= 0.02 * float(dy.float().sum(0).abs().max()) + 0.1


@pytest.mark.parametrize("B,Sk,Hq,Hkv,hd", [(3, 333, 4, 1, 128), (2, 700, 8, 2, 64), (5, 2304, 4, 4, 128)])
def test_decode_attention_output_stays_inside_its_buffer(B, Sk, Hq, Hkv, hd):
    q = _mk((B, Hq * hd), seed=1)
    kc, vc = _mk((B, Sk, Hkv * hd), seed=2), _mk((B, Sk, Hkv * hd), seed=3)
    with guard.guarded() as pool:
        out = pool.empty((B, Hq * hd), torch.bfloat16, "cuda")
        D.attn_decode(q, kc, vc, B, 1, Sk, Hq, Hkv, hd, Sk - 1, out=out)
    ref = D.attn_decode_reference(q, kc, vc, B, 1, Sk, Hq, Hkv, hd, Sk - 1, None)
    assert float((out.float() - ref.float()).abs().max()) < 3e-2
