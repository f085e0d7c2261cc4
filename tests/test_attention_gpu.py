"""GPU numerics of the tcgen05 attention kernels against the fp32 reference formula."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from dart_pytorch_b200.ops import flash as A
from dart_pytorch_b200.ops import reference as R


def _rel(a, b):
    a, b = a.float(), b.float()
    return float(((a - b).norm() / (b.norm() + 1e-12)).detach())


def _qkv(B, S, H, Hkv, hd, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(B * S, (H + 2 * Hkv) * hd, device="cuda", generator=g).to(torch.bfloat16)


def _split(qkv, B, S, H, Hkv, hd):
    x = qkv.float().reshape(B, S, -1)
    dq, dkv = H * hd, Hkv * hd
    q = x[..., :dq].reshape(B, S, H, hd).transpose(1, 2)
    k = x[..., dq:dq + dkv].reshape(B, S, Hkv, hd).transpose(1, 2)
    v = x[..., dq + dkv:].reshape(B, S, Hkv, hd).transpose(1, 2)
    return q, k, v


FWD_CASES = [
    # B, S, H, Hkv, hd, causal
    (1, 128, 1, 1, 64, False), (1, 128, 1, 1, 64, True), (2, 256, 2, 2, 64, True), (2, 384, 3, 3, 64, True),
    (2, 1024, 4, 4, 64, True), (3, 197, 2, 2, 64, False), (1, 300, 2, 1, 64, True), (2, 512, 4, 2, 64, False),
    (1, 128, 1, 1, 128, True), (2, 256, 4, 1, 128, True), (1, 1000, 2, 2, 128, False),
]
# head sizes the kernels take zero-padded to 64 / 128 (through the public wrapper, which does the padding)
PADDED_FWD_CASES = [(2, 200, 4, 4, 32, True), (1, 96, 2, 1, 16, True), (2, 64, 2, 2, 8, False), (1, 256, 2, 2, 96, True)]


@pytest.mark.parametrize("B,S,H,Hkv,hd,causal", FWD_CASES)
def test_attention_forward(B, S, H, Hkv, hd, causal):
    qkv = _qkv(B, S, H, Hkv, hd)
    dq, dkv = H * hd, Hkv * hd
    o, lse = A.attn_fwd(qkv[:, :dq], qkv[:, dq:dq + dkv], qkv[:, dq + dkv:], B, S, S, H, Hkv, hd, causal)
    q, k, v = _split(qkv, B, S, H, Hkv, hd)
    ref = R.attention(q, k, v, causal=causal).transpose(1, 2).reshape(B * S, dq)
    assert torch.isfinite(o.float()).all()
    assert _rel(o, ref) < 2e-2
    g = H // Hkv
    s = (q @ k.repeat_interleave(g, 1).transpose(-1, -2)) / math.sqrt(hd)
    if causal:
        s = s + torch.triu(torch.full((S, S), float("-inf"), device="cuda"), 1)
    assert _rel(lse, torch.logsumexp(s, -1)) < 1e-3


@pytest.mark.parametrize("B,S,H,Hkv,hd,causal", PADDED_FWD_CASES)
def test_attention_forward_padded_head_sizes(B, S, H, Hkv, hd, causal):
    qkv = _qkv(B, S, H, Hkv, hd)
    before = _launches()
    o = A.attention_packed(qkv, B, S, H, Hkv, hd, causal)
    assert _launches() - before == 1            # one flash kernel, not a GEMM + softmax per (batch, head)
    q, k, v = _split(qkv, B, S, H, Hkv, hd)
    ref = R.attention(q, k, v, causal=causal).transpose(1, 2).reshape(B * S, H * hd)
    assert o.shape == ref.shape and torch.isfinite(o.float()).all()
    assert _rel(o, ref) < 2e-2


def test_attention_forward_q_offset():
    B, Sq, Sk, H, hd = 2, 128, 384, 2, 64
    g = torch.Generator(device="cuda").manual_seed(1)
    q2 = torch.randn(B * Sq, H * hd, device="cuda", generator=g).bfloat16()
    k2 = torch.randn(B * Sk, H * hd, device="cuda", generator=g).bfloat16()
    v2 = torch.randn(B * Sk, H * hd, device="cuda", generator=g).bfloat16()
    o, _ = A.attn_fwd(q2, k2, v2, B, Sq, Sk, H, H, hd, True, q_offset=Sk - Sq)
    q = q2.float().reshape(B, Sq, H, hd).transpose(1, 2)
    k = k2.float().reshape(B, Sk, H, hd).transpose(1, 2)
    v = v2.float().reshape(B, Sk, H, hd).transpose(1, 2)
    ref = R.attention(q, k, v, causal=True, q_offset=Sk - Sq).transpose(1, 2).reshape(B * Sq, H * hd)
    assert _rel(o, ref) < 2e-2


BWD_CASES = [(1, 128, 1, 1, 64, False), (1, 128, 1, 1, 64, True), (2, 256, 2, 2, 64, True), (2, 640, 3, 3, 64, True),
             (3, 197, 2, 2, 64, False), (1, 300, 4, 2, 64, True), (2, 1024, 2, 2, 64, True),
             # padded head sizes (kernel at 64), and 128, which has no backward kernel and takes the composed path
             (2, 200, 4, 4, 32, True), (1, 96, 4, 2, 16, True), (2, 40, 2, 2, 8, False), (1, 128, 4, 1, 128, True)]


@pytest.mark.parametrize("B,S,H,Hkv,hd,causal", BWD_CASES)
def test_attention_backward(B, S, H, Hkv, hd, causal):
    qkv = _qkv(B, S, H, Hkv, hd).requires_grad_(True)
    o = A.attention_packed(qkv, B, S, H, Hkv, hd, causal)
    g = torch.Generator(device="cuda").manual_seed(5)
    do = torch.randn(o.shape, device="cuda", generator=g).bfloat16()
    o.backward(do)
    x = qkv.detach().float().requires_grad_(True)
    q, k, v = _split(x, B, S, H, Hkv, hd)
    ref = R.attention(q, k, v, causal=causal).transpose(1, 2).reshape(B * S, H * hd)
    ref.backward(do.float())
    dq_, dkv_ = H * hd, Hkv * hd
    for name, sl in (("dq", slice(0, dq_)), ("dk", slice(dq_, dq_ + dkv_)), ("dv", slice(dq_ + dkv_, None))):
        assert torch.isfinite(qkv.grad[:, sl].float()).all(), name
        assert _rel(qkv.grad[:, sl], x.grad[:, sl]) < 3e-2, name


def _launches():
    import ctypes
    from dart_pytorch_b200 import _native
    lib = _native.load(required=True)
    lib.dptb_launch_count.restype = ctypes.c_longlong
    return lib.dptb_launch_count()


@pytest.mark.parametrize("hd,heads,kv_heads", [(32, 4, 4), (128, 2, 1), (64, 2, 2), (16, 4, 2)])
def test_self_attention_module_gradients(hd, heads, kv_heads):
    """bf16 ``MultiHeadAttention`` on the GPU against the same module in fp32 on the CPU, output and every gradient,
    for head sizes with a backward kernel (64, and 16 / 32 padded) and without one (128)."""
    from dart_pytorch_b200.nn.attention import MultiHeadAttention
    D = hd * heads
    torch.manual_seed(0)
    ref = MultiHeadAttention(D, heads, num_kv_heads=kv_heads, bias=True, seed=3)
    dev = MultiHeadAttention(D, heads, num_kv_heads=kv_heads, bias=True, seed=3).to("cuda", torch.bfloat16)
    x = torch.randn(2, 48, D)
    xr = x.clone().requires_grad_(True)
    xd = x.to("cuda", torch.bfloat16).requires_grad_(True)
    yr = ref(xr, causal=True)
    yd = dev(xd, causal=True)
    assert _rel(yd.cpu(), yr) < 3e-2
    g = torch.randn_like(yr)
    yr.backward(g)
    yd.backward(g.to("cuda", torch.bfloat16))
    assert _rel(xd.grad.cpu(), xr.grad) < 5e-2
    for pd, pr in zip(dev.parameters(), ref.parameters()):
        assert pd.grad is not None and _rel(pd.grad.cpu(), pr.grad) < 5e-2


def test_deterministic_option_gives_bit_identical_attention_gradients(monkeypatch):
    """``DPTB200_DETERMINISTIC=1`` takes attention that needs gradients off the flash backward kernel (whose dQ tiles
    meet in fp32 atomics): two runs are then bit-identical, and still match the fp32 module."""
    from dart_pytorch_b200.nn.attention import MultiHeadAttention
    monkeypatch.setenv("DPTB200_DETERMINISTIC", "1")
    assert A.kernel_head_dim(64, backward=True) is None and A.kernel_head_dim(64) == 64
    D, heads = 256, 4
    ref = MultiHeadAttention(D, heads, bias=True, seed=3)
    dev = MultiHeadAttention(D, heads, bias=True, seed=3).to("cuda", torch.bfloat16)
    torch.manual_seed(1)
    x = torch.randn(2, 384, D)
    g = torch.randn(2, 384, D)
    runs = []
    for _ in range(2):
        xd = x.to("cuda", torch.bfloat16).requires_grad_(True)
        for p in dev.parameters():
            p.grad = None
        before = _launches()
        dev(xd, causal=True).backward(g.to("cuda", torch.bfloat16))
        runs.append([xd.grad.clone()] + [p.grad.clone() for p in dev.parameters()])
        assert _launches() > before
    for a, b in zip(*runs):
        assert torch.equal(a, b)
    xr = x.clone().requires_grad_(True)
    ref(xr, causal=True).backward(g)
    assert _rel(runs[0][0].cpu(), xr.grad) < 5e-2


@pytest.mark.parametrize("hd", [32, 128, 64])
def test_cross_attention_module_gradients(hd):
    from dart_pytorch_b200.nn.attention import MultiHeadCrossAttention
    heads = 2
    D = hd * heads
    ref = MultiHeadCrossAttention(D, 48, heads, bias=True, seed=5)
    dev = MultiHeadCrossAttention(D, 48, heads, bias=True, seed=5).to("cuda", torch.bfloat16)
    torch.manual_seed(1)
    xq, xkv = torch.randn(2, 40, D), torch.randn(2, 24, 48)
    xqr, xkvr = xq.clone().requires_grad_(True), xkv.clone().requires_grad_(True)
    xqd = xq.to("cuda", torch.bfloat16).requires_grad_(True)
    xkvd = xkv.to("cuda", torch.bfloat16).requires_grad_(True)
    yr, yd = ref(xqr, xkvr), dev(xqd, xkvd)
    assert _rel(yd.cpu(), yr) < 3e-2
    g = torch.randn_like(yr)
    yr.backward(g)
    yd.backward(g.to("cuda", torch.bfloat16))
    assert _rel(xqd.grad.cpu(), xqr.grad) < 5e-2
    assert _rel(xkvd.grad.cpu(), xkvr.grad) < 5e-2


def test_small_heads_run_the_flash_kernels():
    """A head size of 32 must reach ``attn_fwd_kernel`` / ``attn_bwd_kernel`` (padded), not the composed path: the
    composed path launches a GEMM and a softmax per (batch, head), the kernels a handful in total."""
    B, S, H, hd = 2, 128, 8, 32
    qkv = _qkv(B, S, H, H, hd).requires_grad_(True)
    before = _launches()
    o = A.attention_packed(qkv, B, S, H, H, hd, True)
    o.backward(torch.ones_like(o))
    assert _launches() - before <= 6
