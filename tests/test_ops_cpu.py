"""CPU oracle ops: closed forms, reference quirks and finite-difference gradient checks
(modelled on the reference's test/autograd_test.dart and test/softmax_ce_embedding_test.dart)."""
import math

import pytest
import torch

from dart_pytorch_b200 import ops as F
from dart_pytorch_b200.ops import reference as R


def _fd(fn, x, eps=1e-3):
    g = torch.zeros_like(x)
    flat = x.reshape(-1)
    for i in range(flat.numel()):
        old = float(flat[i])
        flat[i] = old + eps
        up = float(fn(x))
        flat[i] = old - eps
        dn = float(fn(x))
        flat[i] = old
        g.reshape(-1)[i] = (up - dn) / (2 * eps)
    return g


def test_matmul_shapes_and_errors():
    a, b = torch.randn(2, 3, 4), torch.randn(4, 5)
    assert F.matmul(a, b).shape == (2, 3, 5)
    with pytest.raises(ValueError):
        F.matmul(torch.randn(3, 4), torch.randn(5, 2))
    with pytest.raises(ValueError):
        F.matmul(torch.randn(3, 4), torch.randn(2, 4, 2))


def test_linear_activation_residual():
    x, w, b, r = torch.randn(5, 4), torch.randn(3, 4), torch.randn(3), torch.randn(5, 3)
    for act in (None, "relu", "gelu_tanh", "quick_gelu", "silu"):
        y = F.linear(x, w, b, act, r)
        ref = R.ACTIVATIONS[act](x @ w.t() + b) + r
        assert torch.allclose(y, ref, atol=1e-6)


def test_gelu_tanh_matches_formula():
    x = torch.linspace(-3, 3, 13)
    expect = 0.5 * x * (1 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
    assert torch.allclose(F.gelu_tanh(x), expect, atol=1e-6)
    assert torch.allclose(F.quick_gelu(x), x * torch.sigmoid(1.702 * x), atol=1e-6)


def test_layer_norm_and_rms_norm_gradients_fd():
    torch.manual_seed(0)
    x = torch.randn(3, 6, dtype=torch.float64)
    g = torch.rand(6, dtype=torch.float64) + 0.5
    b = torch.randn(6, dtype=torch.float64)
    w = torch.randn(3, 6, dtype=torch.float64)
    xr = x.clone().requires_grad_(True)
    (F.layer_norm(xr, g, b, 1e-5) * w).sum().backward()
    fd = _fd(lambda t: (R.layer_norm(t, g, b, 1e-5) * w).sum(), x.clone(), 1e-5)
    assert torch.allclose(xr.grad, fd, atol=1e-6)
    xr = x.clone().requires_grad_(True)
    (F.rms_norm(xr, g, 1e-6) * w).sum().backward()
    fd = _fd(lambda t: (R.rms_norm(t, g, 1e-6) * w).sum(), x.clone(), 1e-5)
    assert torch.allclose(xr.grad, fd, atol=1e-6)
    y = F.layer_norm(x, torch.ones(6, dtype=torch.float64), torch.zeros(6, dtype=torch.float64))
    assert torch.allclose(y.mean(-1), torch.zeros(3, dtype=torch.float64), atol=1e-9)


def test_softmax_rows_sum_to_one_and_cross_entropy_contract():
    x = torch.randn(4, 7)
    assert torch.allclose(F.softmax(x).sum(-1), torch.ones(4), atol=1e-6)
    t = torch.tensor([0.0, 6.0, 3.2, 2.6])  # float targets round half up: 3.2 -> 3, 2.6 -> 3
    loss = F.cross_entropy(x, t)
    assert loss.shape == (4, 1)
    idx = torch.tensor([0, 6, 3, 3])
    ref = torch.logsumexp(x, -1) - x[torch.arange(4), idx]
    assert torch.allclose(loss.squeeze(1), ref, atol=1e-6)
    l3 = F.cross_entropy(torch.randn(2, 3, 5), torch.zeros(2, 3))
    assert l3.shape == (6, 1)
    with pytest.raises(ValueError):
        F.cross_entropy(x, torch.zeros(3))
    xr = x.clone().requires_grad_(True)
    F.cross_entropy(xr, idx).mean().backward()
    p = torch.softmax(x, -1)
    p[torch.arange(4), idx] -= 1
    assert torch.allclose(xr.grad, p / 4, atol=1e-6)


def test_embedding_out_of_range_and_scatter_adjoint():
    table = torch.randn(5, 3)
    idx = torch.tensor([[0.0, 4.0], [7.0, -1.0]])
    out = F.embedding(table, idx)
    assert out.shape == (2, 2, 3)
    assert torch.equal(out[0, 0], table[0]) and torch.equal(out[0, 1], table[4])
    assert float(out[1].abs().sum()) == 0.0
    rows = torch.randn(4, 3)
    sc = F.scatter_rows_add(rows, torch.tensor([1, 1, 4, 9]), 5)
    assert torch.allclose(sc[1], rows[0] + rows[1]) and torch.allclose(sc[4], rows[2])
    assert float(sc[0].abs().sum() + sc[2].abs().sum() + sc[3].abs().sum()) == 0.0
    # <embedding(T, i), R> == <T, scatter(R, i)>
    t2, i2, r2 = torch.randn(6, 3), torch.tensor([5, 0, 0, 2]), torch.randn(4, 3)
    assert abs(float((F.embedding(t2, i2) * r2).sum() - (t2 * F.scatter_rows_add(r2, i2, 6)).sum())) < 1e-5


def test_attention_gqa_matches_per_head_sdpa_and_causal_mask():
    torch.manual_seed(1)
    q, k, v = torch.randn(2, 4, 5, 8), torch.randn(2, 2, 5, 8), torch.randn(2, 2, 5, 8)
    o = F.attention(q, k, v, causal=True)
    mask = F.causal_mask(5)
    for b in range(2):
        for h in range(4):
            ref = R.sdpa(q[b, h], k[b, h // 2], v[b, h // 2], mask)
            assert torch.allclose(o[b, h], ref, atol=1e-5)
    assert float(mask[0, 1]) == -1e9 and float(mask[1, 0]) == 0.0
    with pytest.raises(ValueError):
        F.attention(q, torch.randn(2, 3, 5, 8), torch.randn(2, 3, 5, 8))


def test_rope_closed_form_partial_and_start_pos():
    hd = 8
    x = torch.randn(6, hd)
    y = F.rope(x, start_pos=3, base=10000.0)
    for n in range(6):
        for i in range(hd // 2):
            ang = (3 + n) * 10000.0 ** (-2.0 * i / hd)
            a, b = float(x[n, i]), float(x[n, i + hd // 2])
            assert abs(float(y[n, i]) - (a * math.cos(ang) - b * math.sin(ang))) < 1e-5
            assert abs(float(y[n, i + hd // 2]) - (b * math.cos(ang) + a * math.sin(ang))) < 1e-5
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    z = F.rope(x, rotary_dim=4)
    assert torch.equal(z[:, 4:], x[:, 4:])
    # several heads side by side == each head on its own
    xh = torch.randn(5, 3 * hd)
    yh = F.rope(xh, start_pos=2, heads=3)
    for h in range(3):
        assert torch.allclose(yh[:, h * hd:(h + 1) * hd], F.rope(xh[:, h * hd:(h + 1) * hd], start_pos=2), atol=1e-6)


def test_elementwise_reference_quirks():
    a = torch.tensor([1.0, -2.0, 3.0])
    assert torch.allclose(R.safe_div(a, torch.tensor([0.0, 0.0, 2.0])), torch.tensor([1e20, -2e20, 1.5]))
    assert torch.allclose(R.safe_pow(torch.tensor([-2.0, 0.0, 2.0]), 2.0), torch.tensor([4.0, 0.0, 4.0]))
    assert torch.allclose(R.safe_pow(torch.tensor([-2.0, 0.0, 2.0]), -1.0), torch.tensor([-0.5, 0.0, 0.5]))
    assert torch.allclose(R.safe_pow(torch.tensor([-4.0, 4.0]), 0.5), torch.tensor([0.0, 2.0]))
    assert F.sum(torch.ones(2, 3)).shape == (1, 1) and float(F.mean(torch.arange(4.0))) == 1.5
    m = torch.randn(3, 4)
    assert torch.allclose(F.add(m, torch.arange(4.0)), m + torch.arange(4.0))
    assert torch.allclose(F.mul(m, 2.0), m * 2)
    with pytest.raises(ValueError):
        F.add(m, torch.randn(5))
    with pytest.raises(ValueError):
        F.transpose(torch.randn(2, 3, 4))


def test_dropout_contract():
    x = torch.ones(1000)
    assert F.dropout(x, 0.5, training=False) is x
    assert F.dropout(x, 0.0, training=True) is x
    y = F.dropout(x, 0.5, training=True, generator=torch.Generator().manual_seed(0))
    vals = set(y.unique().tolist())
    assert vals <= {0.0, 2.0} and 300 < int((y == 0).sum()) < 700
    with pytest.raises(ValueError):
        F.dropout(x, 1.0, True)


def test_concat_split_slice():
    a, b = torch.randn(2, 3), torch.randn(4, 3)
    assert F.concat([a, b], 0).shape == (6, 3)
    with pytest.raises(ValueError):
        F.concat([a, b], 2)
    parts = F.split_rows(torch.randn(6, 2), 3)
    assert len(parts) == 2 and parts[0].shape == (3, 2)
    with pytest.raises(ValueError):
        F.split_rows(torch.randn(5, 2), 3)
    assert F.slice_top_left(torch.randn(4, 5), 2, 3).shape == (2, 3)


def test_aft_full_matches_loop_and_im2col_shape():
    torch.manual_seed(2)
    t, d = 5, 3
    q, k, v, w = torch.randn(t, d), torch.randn(t, d), torch.randn(t, d), torch.randn(t, t)
    out = F.aft_full(q, k, v, w, causal=True)
    for i in range(t):
        for c in range(d):
            logits = torch.tensor([float(k[j, c] + w[i, j]) for j in range(i + 1)])
            e = torch.exp(logits - logits.max())
            num = float((e * v[:i + 1, c]).sum())
            den = float(e.sum()) + 1e-6
            assert abs(float(out[i, c]) - float(torch.sigmoid(q[i, c])) * num / den) < 1e-5
    x = torch.randn(2 * 64, 4)
    cols = F.im2col_nhwc(x, 2, 4, 3)
    assert cols.shape == (128, 36)
    # centre tap of cell (3,3) of image 0, channel 1 is the cell itself; column order is (ky, kx) stacked last
    assert torch.allclose(cols[3 * 8 + 3].reshape(4, 9)[1, 4], x[3 * 8 + 3, 1])


def test_sampler_greedy_topk_and_seeded():
    import random
    logits = torch.tensor([0.1, 2.0, -1.0, 1.9])
    assert F.sample_from_logits(logits, 0.0, None, random.Random(0)) == 1
    assert F.sample_from_logits(logits, 1.0, 1, random.Random(0)) == 1
    draws = {F.sample_from_logits(logits, 1.0, 2, random.Random(s)) for s in range(50)}
    assert draws == {1, 3}
    a = [F.sample_from_logits(logits, 0.7, None, random.Random(5)) for _ in range(3)]
    b = [F.sample_from_logits(logits, 0.7, None, random.Random(5)) for _ in range(3)]
    assert a == b


def test_native_library_discovery_order(tmp_path, monkeypatch):
    """Env override wins and is taken as given; otherwise cwd, program directory, package directory; non-ELF files
    are skipped (reference behaviour: native_lib_download_test.dart)."""
    from dart_pytorch_b200 import _native as N
    monkeypatch.delenv("DPTB200_NATIVE_LIB", raising=False)
    monkeypatch.delenv("DPTB200_AUTO_BUILD", raising=False)
    monkeypatch.chdir(tmp_path)
    assert N.candidate_paths()[0] == tmp_path / N.LIB_NAME and N.candidate_paths()[-1].parent.name == "_C"
    (tmp_path / N.LIB_NAME).write_bytes(b"not an elf")
    assert N.lib_path() != tmp_path / N.LIB_NAME
    (tmp_path / N.LIB_NAME).write_bytes(b"\x7fELF" + bytes(16))
    assert N.lib_path() == tmp_path / N.LIB_NAME and N.looks_like_shared_object(tmp_path / N.LIB_NAME)
    monkeypatch.setenv("DPTB200_NATIVE_LIB", str(tmp_path / "custom.so"))
    assert N.lib_path() == tmp_path / "custom.so" and N.candidate_paths()[0] == tmp_path / "custom.so"
    assert N.build_native_library() is None          # opt-in only


def test_fused_cpu_ops_match_the_reference_formulas_in_value_and_gradient():
    """``ops/cpu_fast.py`` (single ATen calls, the CPU execution path) against ``ops/reference.py`` (the oracle)."""
    from dart_pytorch_b200.ops import cpu_fast as C
    g = torch.Generator().manual_seed(0)

    def rnd(*shape):
        return torch.randn(*shape, generator=g, dtype=torch.float64).requires_grad_()

    def same(fast_fn, ref_fn, *inputs, tol=1e-9):
        a = fast_fn(*inputs)
        grads_a = torch.autograd.grad(a.sum() + (a * a).sum(), inputs, allow_unused=True)
        b = ref_fn(*inputs)
        grads_b = torch.autograd.grad(b.sum() + (b * b).sum(), inputs, allow_unused=True)
        assert a.shape == b.shape and torch.allclose(a, b.to(a.dtype), atol=tol, rtol=tol)
        for ga, gb in zip(grads_a, grads_b):
            assert (ga is None) == (gb is None)
            if ga is not None:
                assert torch.allclose(ga, gb, atol=10 * tol, rtol=10 * tol)
    x, w, b, r = rnd(5, 7), rnd(3, 7), rnd(1, 3), rnd(5, 3)
    for act in (None, "relu", "gelu_tanh", "silu", "sigmoid", "tanh", "quick_gelu"):
        same(lambda x, w, b, r: C.linear(x, w, b, act, r), lambda x, w, b, r: R.linear(x, w, b, act, r), x, w, b, r)
    same(C.gelu_tanh, R.gelu_tanh, rnd(4, 9))
    gam, bet = rnd(1, 7), rnd(7)
    same(lambda x, g_, b_: C.layer_norm(x, g_, b_, 1e-5), lambda x, g_, b_: R.layer_norm(x, g_, b_, 1e-5), x, gam, bet)
    same(lambda x, g_: C.layer_norm(x, g_, None, 1e-5), lambda x, g_: R.layer_norm(x, g_, None, 1e-5), x, gam)
    same(C.softmax, R.softmax, rnd(2, 3, 6))
    q, k, v = (t.detach().float().requires_grad_() for t in (rnd(2, 4, 5, 8), rnd(2, 2, 9, 8), rnd(2, 2, 9, 8)))
    same(lambda q, k, v: C.attention(q, k, v, causal=True, q_offset=4),
         lambda q, k, v: R.attention(q, k, v, causal=True, q_offset=4), q, k, v, tol=1e-5)   # the oracle works in fp32
    mask = torch.randn(5, 9, generator=g)
    same(lambda q, k, v: C.attention(q, k, v, mask=mask), lambda q, k, v: R.attention(q, k, v, mask=mask), q, k, v, tol=1e-5)
    logits, tgt = rnd(6, 11).detach().float().requires_grad_(), torch.tensor([0, 10, 3, 3, 7, 1])
    same(lambda l: C.cross_entropy(l, tgt), lambda l: R.cross_entropy(l, tgt), logits, tol=1e-5)
    table = rnd(10, 4)
    same(lambda t: C.embedding(t, torch.tensor([[1, 9], [0, 3]])), lambda t: R.embedding(t, torch.tensor([[1, 9], [0, 3]])), table)
    oob = torch.tensor([1.0, 12.0, -3.0])
    assert torch.equal(C.embedding(table, oob), R.embedding(table, oob)) and float(C.embedding(table, oob)[1].detach().abs().sum()) == 0
    # other dtypes and seeded dropout keep the reference path; unseeded dropout keeps the {0, 1/(1-p)} contract
    xb, wb = torch.randn(2, 7).bfloat16(), w.detach().bfloat16()
    assert torch.equal(C.linear(xb, wb, None, "gelu_tanh"), R.linear(xb, wb, None, "gelu_tanh"))
    y = C.dropout(torch.ones(2000), 0.25, True)
    kept = y[y != 0]
    assert torch.allclose(kept, torch.full_like(kept, 1.0 / 0.75)) and 300 < int((y == 0).sum()) < 700
    y1 = C.dropout(torch.ones(50), 0.5, True, torch.Generator().manual_seed(3))
    y2 = R.dropout(torch.ones(50), 0.5, True, torch.Generator().manual_seed(3))
    assert torch.equal(y1, y2)
