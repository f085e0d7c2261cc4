"""GPU numerics: every native kernel against a plain PyTorch fp32 computation of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from dart_pytorch_b200.ops import kernels as K
from dart_pytorch_b200.ops import reference as R


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return float(((a - b).norm() / (b.norm() + 1e-12)).detach())


def _mk(shape, dtype=torch.bfloat16, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(dtype)


GEMM_SHAPES = [(128, 128, 64), (256, 256, 128), (384, 512, 192), (128, 256, 768), (1000, 760, 264), (77, 40, 72),
               (2048, 2304, 768), (130, 50257 // 64, 64)]


@pytest.mark.parametrize("M,N,Kd", GEMM_SHAPES)
@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_tc_layouts(M, N, Kd, trans_a, trans_b, bn):
    if trans_a and M % 8:
        pytest.skip("MN-major A needs M % 8 == 0 for the row stride")
    if not trans_b and N % 8:
        pytest.skip("MN-major B needs N % 8 == 0 for the row stride")
    a = _mk((Kd, M) if trans_a else (M, Kd), seed=1)
    b = _mk((N, Kd) if trans_b else (Kd, N), seed=2)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    K.gemm(a, b, out, trans_a=trans_a, trans_b=trans_b, bn=bn)
    af = a.float().t() if trans_a else a.float()
    bf = b.float().t() if trans_b else b.float()
    ref = af @ bf
    assert torch.isfinite(out.float()).all()
    assert _rel_err(out, ref) < 1e-2


@pytest.mark.parametrize("act", [None, "relu", "gelu_tanh", "quick_gelu", "silu"])
def test_gemm_epilogue_forward(act):
    M, N, Kd = 512, 384, 256
    a, w = _mk((M, Kd), seed=3), _mk((N, Kd), scale=0.05, seed=4)
    bias = _mk((N,), dtype=torch.float32, seed=5)
    res = _mk((M, N), seed=6)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    pre = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    K.gemm(a, w, out, trans_b=True, bias=bias, residual=res, aux_out=pre, act=act)
    pre_ref = a.float() @ w.float().t() + bias
    ref = R.ACTIVATIONS[act](pre_ref) + res.float()
    assert _rel_err(pre, pre_ref) < 1e-2
    assert _rel_err(out, ref) < 1e-2


@pytest.mark.parametrize("act", [None, "gelu_tanh", "silu"])
@pytest.mark.parametrize("M,N,Kd,bn", [(512, 384, 256, 128), (1000, 760, 264, 256), (300, 2304, 768, 256)])
def test_gemm_epilogue_forward_bf16_bias(act, M, N, Kd, bn):
    """bf16 bias: the row-per-thread epilogue with TMA tile stores (ragged M is clipped by the store, the ragged last
    column block takes the staged path)."""
    a, w = _mk((M, Kd), seed=3), _mk((N, Kd), scale=0.05, seed=4)
    bias = _mk((N,), seed=5)
    res = _mk((M, N), seed=6)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    pre = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    K.gemm(a, w, out, trans_b=True, bias=bias, residual=res, aux_out=pre, act=act, bn=bn)
    pre_ref = a.float() @ w.float().t() + bias.float()
    ref = R.ACTIVATIONS[act](pre_ref) + res.float()
    assert torch.isfinite(out.float()).all() and torch.isfinite(pre.float()).all()
    assert _rel_err(pre, pre_ref) < 1e-2
    assert _rel_err(out, ref) < 1e-2


def test_gemm_epilogue_in_place_residual_accumulate_and_padding():
    M, N, Kd = 640, 200, 192
    a, w = _mk((M, Kd), seed=21), _mk((N, Kd), scale=0.05, seed=22)
    # residual aliases the output (x += a @ w^T), output rows padded to 256 columns that must stay untouched
    buf = torch.zeros(M, 256, dtype=torch.bfloat16, device="cuda")
    base = _mk((M, N), seed=23)
    buf[:, :N] = base
    buf[:, N:] = 7.0
    K.gemm(a, w, buf, trans_b=True, residual=buf, n_cols=N)
    ref = base.float() + a.float() @ w.float().t()
    assert _rel_err(buf[:, :N], ref) < 1e-2
    assert bool((buf[:, N:] == 7.0).all())
    # accumulate into a bf16 output
    out = base.clone()
    K.gemm(a, w, out, trans_b=True, accumulate=True)
    assert _rel_err(out, ref) < 1e-2


@pytest.mark.parametrize("M", [1, 7, 32, 33, 64])
@pytest.mark.parametrize("N,Kd", [(768, 4096), (200, 264), (4096, 512), (16032, 1024)])
@pytest.mark.parametrize("extras", [False, True])
def test_gemm_skinny_rows(M, N, Kd, extras):
    """Decode-sized rows take the weight-streaming kernel (operands swapped on the tensor core, K split over the SMs)."""
    x, w = _mk((M, Kd), seed=31), _mk((N, Kd), scale=0.05, seed=32)
    bias = _mk((N,), seed=33) if extras else None
    res = _mk((M, N), seed=34) if extras else None
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    K.gemm(x, w, out, trans_b=True, bias=bias, residual=res)
    ref = x.float() @ w.float().t()
    if extras:
        ref = ref + bias.float() + res.float()
    assert torch.isfinite(out.float()).all()
    assert _rel_err(out, ref) < 1e-2
    again = torch.empty_like(out)
    K.gemm(x, w, again, trans_b=True, bias=bias, residual=res)
    assert torch.equal(out, again)          # split-K partials are summed in a fixed order


@pytest.mark.parametrize("act", ["relu", "gelu_tanh", "quick_gelu", "silu"])
def test_gemm_epilogue_act_backward(act):
    M, N, Kd = 256, 256, 128
    dy, w = _mk((M, Kd), seed=7), _mk((Kd, N), scale=0.05, seed=8)
    pre = _mk((M, N), seed=9)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    K.gemm(dy, w, out, aux_in=pre, act_bwd=act)
    x = pre.float().requires_grad_(True)
    R.ACTIVATIONS[act](x).backward(dy.float() @ w.float())
    assert _rel_err(out, x.grad) < 2e-2


@pytest.mark.parametrize("M,N,Kd", [(256, 256, 128), (512, 3072, 768), (100, 200, 72)])
def test_gemm_gelu_with_saved_derivative(M, N, Kd):
    """Forward GELU that saves the derivative instead of the pre-activation, and the one-multiply backward epilogue."""
    x, w, b = _mk((M, Kd), seed=41), _mk((N, Kd), scale=0.05, seed=42), _mk((N,), seed=43)
    y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    d = torch.empty_like(y)
    K.gemm(x, w, y, trans_b=True, bias=b, act="gelu_tanh_d", aux_out=d)
    pre = (x.float() @ w.float().t() + b.float()).requires_grad_(True)
    ref = R.ACTIVATIONS["gelu_tanh"](pre)
    ref.sum().backward()
    assert _rel_err(y, ref) < 1e-2
    assert _rel_err(d, pre.grad) < 1e-2
    dy, w2 = _mk((M, Kd), seed=44), _mk((Kd, N), scale=0.05, seed=45)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    K.gemm(dy, w2, out, aux_in=d, act_bwd="mul")
    assert _rel_err(out, (dy.float() @ w2.float()) * d.float()) < 1e-2


def test_gemm_accumulate_fp32_out_and_padded_ld():
    M, N, Kd = 256, 200, 128
    a, w = _mk((M, Kd), seed=10), _mk((N, Kd), seed=11)
    buf = torch.zeros(M, 256, dtype=torch.float32, device="cuda")
    base = torch.randn(M, N, device="cuda")
    buf[:, :N] = base
    K.gemm(a, w, buf, trans_b=True, accumulate=True, n_cols=N)
    ref = base + a.float() @ w.float().t()
    assert _rel_err(buf[:, :N], ref) < 1e-2
    assert float(buf[:, N:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_simt(dtype):
    M, N, Kd = 67, 45, 33
    a, b = _mk((M, Kd), dtype=dtype, seed=12), _mk((Kd, N), dtype=dtype, seed=13)
    out = torch.empty(M, N, dtype=dtype, device="cuda")
    K.gemm(a, b, out, force_simt=True)
    assert _rel_err(out, a.float() @ b.float()) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,D", [(64, 768), (33, 1024), (17, 4096), (9, 100), (5, 64), (1000, 256)])
def test_layernorm(dtype, rows, D):
    x = _mk((rows, D), dtype=dtype, seed=1)
    g = (1.0 + 0.1 * _mk((D,), dtype=torch.float32, seed=2)).to(dtype)
    b = (0.1 * _mk((D,), dtype=torch.float32, seed=3)).to(dtype)
    dy = _mk((rows, D), dtype=dtype, seed=4)
    dres = _mk((rows, D), dtype=dtype, seed=5)
    y, mean, rstd = K.layernorm_fwd(x, g, b, 1e-5)
    xf = x.float().requires_grad_(True)
    gf, bf_ = g.float().requires_grad_(True), b.float().requires_grad_(True)
    yr = R.layer_norm(xf, gf, bf_, 1e-5)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert _rel_err(y, yr) < tol
    yr.backward(dy.float())
    dx, dg, db = K.layernorm_bwd(x, dy, g, mean, rstd, dres=dres)
    assert _rel_err(dx, xf.grad + dres.float()) < tol * 2
    assert _rel_err(dg, gf.grad) < tol * 2
    assert _rel_err(db, bf_.grad) < tol * 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,D", [(64, 1024), (17, 4096), (9, 100)])
def test_rmsnorm(dtype, rows, D):
    x = _mk((rows, D), dtype=dtype, seed=1)
    g = (1.0 + 0.1 * _mk((D,), dtype=torch.float32, seed=2)).to(dtype)
    dy = _mk((rows, D), dtype=dtype, seed=4)
    y, rstd = K.rmsnorm_fwd(x, g, 1e-6)
    xf, gf = x.float().requires_grad_(True), g.float().requires_grad_(True)
    yr = R.rms_norm(xf, gf, 1e-6)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert _rel_err(y, yr) < tol
    yr.backward(dy.float())
    dx, dg = K.rmsnorm_bwd(x, dy, g, rstd)
    assert _rel_err(dx, xf.grad) < tol * 2
    assert _rel_err(dg, gf.grad) < tol * 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,V,ld", [(64, 50257, 50304), (33, 1000, 1000), (7, 65, 65), (16, 32000, 32000)])
def test_cross_entropy(dtype, rows, V, ld):
    buf = torch.zeros(rows, ld, dtype=dtype, device="cuda")
    buf[:, :V] = _mk((rows, V), dtype=dtype, scale=2.0, seed=1)
    tgt = torch.randint(0, V, (rows,), device="cuda")
    loss, lse = K.ce_fwd(buf, tgt, V)
    xf = buf[:, :V].float().requires_grad_(True)
    ref = R.cross_entropy(xf, tgt)
    assert _rel_err(loss, ref.squeeze(1)) < 1e-4
    g = torch.rand(rows, device="cuda") + 0.5
    ref.backward(g.unsqueeze(1))
    d = torch.empty_like(buf)
    K.ce_bwd(buf, tgt, lse, g, 1.0, V, out=d, pad_to=ld if ld % 8 == 0 else V)
    assert _rel_err(d[:, :V], xf.grad) < (1e-4 if dtype == torch.float32 else 1e-2)
    if ld > V and ld % 8 == 0:
        assert float(d[:, V:].float().abs().max()) == 0.0


def test_lm_head_loss_applies_the_upstream_scalar():
    """The fused loss writes its gradient before backward knows the upstream scalar; a scaled loss must still give
    scaled gradients."""
    from dart_pytorch_b200.ops.cuda import LMHeadLossFn
    torch.manual_seed(0)
    h = (torch.randn(256, 64, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(500, 64, device="cuda") * 0.1).bfloat16().requires_grad_(True)
    tgt = torch.randint(0, 500, (256,), device="cuda")
    (LMHeadLossFn.apply(h, w, tgt) * 3.0).backward()
    hr, wr = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    (torch.nn.functional.cross_entropy(hr @ wr.t(), tgt) * 3.0).backward()
    assert _rel_err(h.grad, hr.grad) < 3e-2 and _rel_err(w.grad, wr.grad) < 3e-2


def test_softmax_rows():
    x = _mk((37, 513), dtype=torch.float32, seed=1)
    y = K.softmax_fwd(x)
    assert _rel_err(y, R.softmax(x)) < 1e-5
    dy = _mk((37, 513), dtype=torch.float32, seed=2)
    xr = x.clone().requires_grad_(True)
    R.softmax(xr).backward(dy)
    assert _rel_err(K.softmax_bwd(y, dy), xr.grad) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_backward(dtype):
    V, D, B, S = 1000, 96, 4, 32
    table, pos = _mk((V, D), dtype=dtype, seed=1), _mk((64, D), dtype=dtype, seed=2)
    idx = torch.randint(0, V, (B, S), device="cuda")
    idx[0, 0] = V + 5  # out of range -> zero row
    out = K.embedding_fwd(table, idx, pos_table=pos, pos_start=3, seq_len=S)
    ref = R.embedding(table.float(), idx) + pos.float()[3:3 + S].unsqueeze(0)
    assert _rel_err(out, ref) < (1e-6 if dtype == torch.float32 else 1e-2)
    dout = _mk((B, S, D), dtype=dtype, seed=3)
    for det in (True, False):
        dt = torch.zeros(V, D, dtype=dtype, device="cuda")
        K.embedding_bwd(dt, idx, dout, deterministic=det)
        refd = R.scatter_rows_add(dout.float().reshape(-1, D), idx.reshape(-1), V)
        assert _rel_err(dt, refd) < (1e-5 if dtype == torch.float32 else 2e-2)
    dp = torch.zeros(64, D, dtype=dtype, device="cuda")
    K.pos_embedding_bwd(dp, dout, 3, S, B)
    assert _rel_err(dp[3:3 + S], dout.float().sum(0)) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
def test_grad_norm_and_adam(gdtype):
    n = 1_000_003
    p = torch.randn(n, device="cuda")
    g = (torch.randn(n, device="cuda") * 0.1).to(gdtype)
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    shadow = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    ctrl = torch.zeros(4, device="cuda")
    K.grad_norm(g, ctrl, 1.0)
    total = float(g.float().norm())
    assert abs(float(ctrl[0]) - total) / total < 1e-4
    assert abs(float(ctrl[1]) - min(1.0, 1.0 / total)) < 1e-5
    p0 = p.clone()
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.999, 1e-8, 0.1
    K.adam_flat(p, shadow, g, m, v, ctrl, lr, b1, b2, eps, wd, 1 - b1, 1 - b2)
    gs = g.float() * float(ctrl[1])
    mr, vr = (1 - b1) * gs, (1 - b2) * gs * gs
    pr = p0 - (lr * (mr / (1 - b1)) / ((vr / (1 - b2)).sqrt() + eps) + lr * wd * p0)
    assert _rel_err(p, pr) < 1e-4
    assert _rel_err(shadow, pr) < 1e-2
    assert _rel_err(m, mr) < 1e-4 and _rel_err(v, vr) < 1e-4


@pytest.mark.parametrize("M,N,Kd,trans_a,trans_b", [(768, 768, 4096, True, False), (384, 520, 2048, True, False),
                                                    (256, 256, 1024, False, True), (130, 200, 1536, False, False)])
@pytest.mark.parametrize("splits,bn", [(2, 256), (4, 128), (3, 256), (0, 0)])
def test_gemm_split_k_matches_and_is_deterministic(M, N, Kd, trans_a, trans_b, splits, bn):
    a = _mk((Kd, M) if trans_a else (M, Kd), seed=21)
    b = _mk((N, Kd) if trans_b else (Kd, N), seed=22)
    bias = _mk((N,), dtype=torch.float32, seed=23)
    outs = []
    for _ in range(2):
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        K.gemm(a, b, out, trans_a=trans_a, trans_b=trans_b, bias=bias, splits=splits, bn=bn)
        outs.append(out)
    af = a.float().t() if trans_a else a.float()
    bf = b.float().t() if trans_b else b.float()
    assert _rel_err(outs[0], af @ bf + bias) < 1e-2
    assert torch.equal(outs[0], outs[1])
    acc = torch.ones(M, N, dtype=torch.float32, device="cuda")
    K.gemm(a, b, acc, trans_a=trans_a, trans_b=trans_b, accumulate=True, splits=splits, bn=bn)
    assert _rel_err(acc, af @ bf + 1.0) < 1e-2


@pytest.mark.parametrize("gate,groups,top_groups,k", [("softmax", 1, 1, 2), ("sigmoid", 1, 1, 2), ("sigmoid", 4, 2, 3),
                                                      ("softmax", 4, 2, 2)])
def test_moe_route_gate_bias_and_grouped_topk(gate, groups, top_groups, k):
    """The expert-parallel router against the routing rule of the single-device layer: gate function, choice on
    score + bias, grouped top-k, weights from the unbiased scores, renormalisation."""
    from dart_pytorch_b200.parallel import ep
    T, E = 257, 16
    g = torch.Generator(device="cuda").manual_seed(3)
    logits = torch.randn(T, E, device="cuda", generator=g)
    bias = torch.randn(E, device="cuda", generator=g) * 0.3
    probs, idx, w = ep.route(logits, k, renorm=True, route_scale=1.5, gate=gate, bias=bias, groups=groups,
                             top_groups=top_groups)
    scores = torch.softmax(logits, -1) if gate == "softmax" else torch.sigmoid(logits)
    assert _rel_err(probs, scores) < 1e-5
    biased = scores + bias
    if groups > 1:
        per = E // groups
        grp = biased.view(T, groups, per)
        gscore = grp.topk(2, -1).values.sum(-1) if gate == "sigmoid" else grp.max(-1).values
        keep = torch.zeros(T, groups, dtype=torch.bool, device="cuda")
        keep.scatter_(1, gscore.topk(top_groups, -1).indices, True)
        biased = torch.where(keep.unsqueeze(-1).expand(T, groups, per).reshape(T, E), biased,
                             torch.full_like(biased, float("-inf")))
    want_idx = biased.topk(k, -1).indices
    assert torch.equal(idx.long().sort(-1).values, want_idx.sort(-1).values)
    sel = torch.gather(scores, 1, idx.long())
    assert _rel_err(w, sel / (sel.sum(-1, keepdim=True) + 1e-9) * 1.5) < 1e-5
