"""LC0 reader / input / network against a plain conv2d + batch-norm oracle, Conv2d against torch, Hungarian matching
against brute force."""
import gzip
import itertools
import struct

import numpy as np
import pytest
import torch

from dart_pytorch_b200.models.lc0 import START_FEN, Lc0Input, Lc0Net, Lc0Reader
from dart_pytorch_b200.nn.conv import Conv2d, im2col
from dart_pytorch_b200.utils.hungarian import HungarianAlgorithm


# ---- a minimal protobuf writer for the LC0 Net message ------------------------------------------------------
def _varint(v: int) -> bytes:
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _ld(num: int, payload: bytes) -> bytes:
    return _varint((num << 3) | 2) + _varint(len(payload)) + payload


def _layer(t: torch.Tensor, enc: int) -> bytes:
    a = t.detach().reshape(-1).numpy().astype(np.float32)
    if enc == 1:
        lo, hi = float(a.min()), float(a.max())
        if hi == lo:
            hi = lo + 1.0
        q = np.round((a - lo) / (hi - lo) * 65535.0).astype("<u2")
        body = q.tobytes()
    elif enc == 2:
        lo = hi = 0.0
        body = a.astype("<f2").tobytes()
    else:
        lo = hi = 0.0
        body = (a.view(np.uint32) >> 16).astype("<u2").tobytes()
    return (_varint((1 << 3) | 5) + struct.pack("<f", lo) + _varint((2 << 3) | 5) + struct.pack("<f", hi)
            + _ld(3, body) + _varint((4 << 3) | 0) + _varint(enc))


def _conv_block(w, b, mean, var, gamma, beta, enc) -> bytes:
    return b"".join(_ld(i + 1, _layer(t, enc)) for i, t in enumerate((w, b, mean, var, gamma, beta)))


def _rand_block(cout, cin, k, g):
    return (torch.randn(cout, cin, k, k, generator=g) * 0.1, torch.randn(cout, generator=g) * 0.1,
            torch.randn(cout, generator=g) * 0.1, torch.rand(cout, generator=g) + 0.5,
            torch.rand(cout, generator=g) + 0.5, torch.randn(cout, generator=g) * 0.1)


def _build_net(enc: int, filters=8, blocks=2, planes=5, vf=4, fc=16, wdl=3, se_hidden=4, seed=0):
    g = torch.Generator().manual_seed(seed)
    t = dict(input=_rand_block(filters, 112, 3, g), res=[], policy1=_rand_block(filters, filters, 3, g),
             policy=_rand_block(planes, filters, 3, g), value=_rand_block(vf, filters, 1, g),
             ip1w=torch.randn(fc, vf * 64, generator=g) * 0.1, ip1b=torch.randn(fc, generator=g) * 0.1,
             ip2w=torch.randn(wdl, fc, generator=g) * 0.1, ip2b=torch.randn(wdl, generator=g) * 0.1)
    body = _ld(1, _conv_block(*t["input"], enc))
    for i in range(blocks):
        c1, c2 = _rand_block(filters, filters, 3, g), _rand_block(filters, filters, 3, g)
        se = None
        blob = _ld(1, _conv_block(*c1, enc)) + _ld(2, _conv_block(*c2, enc))
        if i % 2 == 0:
            se = (torch.randn(filters, se_hidden, generator=g) * 0.3, torch.randn(se_hidden, generator=g) * 0.1,
                  torch.randn(se_hidden, 2 * filters, generator=g) * 0.3, torch.randn(2 * filters, generator=g) * 0.1)
            blob += _ld(3, b"".join(_ld(j + 1, _layer(x, enc)) for j, x in enumerate(se)))
        t["res"].append((c1, c2, se))
        body += _ld(2, blob)
    body += _ld(3, _conv_block(*t["policy"], enc)) + _ld(6, _conv_block(*t["value"], enc))
    body += _ld(7, _layer(t["ip1w"], enc)) + _ld(8, _layer(t["ip1b"], enc))
    body += _ld(9, _layer(t["ip2w"], enc)) + _ld(10, _layer(t["ip2b"], enc))
    body += _ld(11, _conv_block(*t["policy1"], enc))
    net = _varint((1 << 3) | 5) + struct.pack("<I", 0x1C0) + _ld(10, body)
    return net, t


def _oracle(w, planes):
    """The classical net with explicit batch norm on NCHW tensors, from the *dequantised* weights."""
    def cbr(x, cb, k, relu=True):
        y = torch.nn.functional.conv2d(x, cb.weights, cb.biases, padding=k // 2)
        y = (y - cb.bn_means.view(1, -1, 1, 1)) / torch.sqrt(cb.bn_stddivs.view(1, -1, 1, 1) + 1e-5)
        y = y * cb.bn_gammas.view(1, -1, 1, 1) + cb.bn_betas.view(1, -1, 1, 1)
        return torch.relu(y) if relu else y
    h = cbr(planes, w.input, 3)
    for r in w.residual:
        a = cbr(h, r.conv1, 3)
        b = cbr(a, r.conv2, 3, relu=False)
        if r.se is not None:
            c = w.filters
            pool = b.mean((2, 3))
            fc1 = torch.relu(pool @ r.se.w1 + r.se.b1)
            z = fc1 @ r.se.w2 + r.se.b2
            gamma, beta = torch.sigmoid(z[:, :c]), z[:, c:]
            b = b * gamma.view(-1, c, 1, 1) + beta.view(-1, c, 1, 1)
        h = torch.relu(b + h)
    pol = cbr(cbr(h, w.policy1, 3), w.policy_out, 3, relu=False)
    v = cbr(h, w.value_conv, 1).reshape(planes.shape[0], -1)
    v = torch.relu(v @ w.ip1_val_w.t() + w.ip1_val_b)
    v = v @ w.ip2_val_w.t() + w.ip2_val_b
    return pol, torch.softmax(v, -1) if w.wdl == 3 else v


@pytest.mark.parametrize("enc", [1, 2, 3])
def test_lc0_reader_and_net_match_oracle(tmp_path, enc):
    raw, t = _build_net(enc)
    path = tmp_path / "net.pb.gz"
    path.write_bytes(gzip.compress(raw))
    w = Lc0Reader.read_file(str(path))
    assert (w.filters, w.num_blocks, w.policy_output_planes, w.value_filters, w.value_fc_units, w.wdl) == \
        (8, 2, 5, 4, 16, 3)
    assert w.residual[0].se is not None and w.residual[1].se is None and w.moves_left_conv is None
    tol = {1: 2e-4, 2: 2e-3, 3: 2e-2}[enc]
    assert torch.allclose(w.input.weights, t["input"][0], atol=tol)
    assert torch.allclose(w.ip2_val_b, t["ip2b"], atol=tol)
    net = Lc0Net(w, device="cpu")
    planes = torch.cat([Lc0Input.from_fen(START_FEN),
                        Lc0Input.from_fen("r3k2r/8/8/8/8/8/8/R3K2R b Kq - 12 40")], 0)
    pol, val = net.forward_planes(planes)
    opol, oval = _oracle(w, planes)
    assert torch.allclose(pol, opol, atol=2e-4) and torch.allclose(val, oval, atol=2e-5)
    outs = net.call_batch([planes[:1], planes[1:]])
    assert outs[0].policy_logits.shape == (1, 5, 8, 8) and outs[1].value.shape == (1, 3)
    assert abs(outs[0].scalar_value - float(oval[0, 0] - oval[0, 2])) < 1e-4
    single = net(planes[:1])
    assert torch.allclose(single.policy_logits, outs[0].policy_logits, atol=1e-5)
    with pytest.raises(ValueError):
        net(torch.zeros(1, 3, 8, 8))


def test_lc0_reader_rejects_truncated_weights():
    raw, _ = _build_net(2)
    with pytest.raises(ValueError):
        Lc0Reader.read_bytes(_varint((1 << 3) | 5) + struct.pack("<I", 1))      # no field 10


def test_lc0_input_planes():
    p = Lc0Input.from_fen(START_FEN)[0]
    assert p.shape == (112, 8, 8)
    assert p[0].sum() == 8 and torch.all(p[0, 1] == 1)           # own pawns on rank 2
    assert p[6].sum() == 8 and torch.all(p[6, 6] == 1)           # their pawns on rank 7
    assert p[5, 0, 4] == 1 and p[11, 7, 4] == 1                  # kings on e1 / e8
    assert all(torch.all(p[i] == 1) for i in (104, 105, 106, 107, 111))
    assert torch.all(p[108] == 0) and torch.all(p[110] == 0)
    assert torch.all(p[12:104] == 0)                             # no history planes
    b = Lc0Input.from_fen("r3k2r/8/8/8/8/8/8/R3K2R b Kq - 12 40")[0]
    assert torch.all(b[108] == 1) and torch.all(b[109] == 12)
    assert b[5, 0, 4] == 1 and b[11, 7, 4] == 1                  # black king now "ours", on the flipped first rank
    assert torch.all(b[104] == 1) and torch.all(b[105] == 0)     # black may castle queen-side only
    assert torch.all(b[106] == 0) and torch.all(b[107] == 1)     # white may castle king-side only
    for bad in ("", "8/8/8 w - - 0 1", "rnbqkbnr/pppppppp/8/8/8/8/PPPPPPPP/RNBQKBNX w - - 0 1",
                "8/8/8/8/8/8/8/8 x - - 0 1"):
        with pytest.raises(ValueError):
            Lc0Input.from_fen(bad)


@pytest.mark.parametrize("k,stride,pad", [(3, 1, 1), (3, 2, 0), (1, 1, 0), (5, 2, 2)])
def test_conv2d_matches_torch_and_is_differentiable(k, stride, pad):
    torch.manual_seed(0)
    conv = Conv2d(3, 6, kernel=k, stride=stride, padding=pad, seed=3)
    x = torch.randn(2, 3, 9, 10, requires_grad=True)
    y = conv(x)
    want = torch.nn.functional.conv2d(x, conv.weight, conv.bias, stride=stride, padding=pad)
    assert y.shape == want.shape and torch.allclose(y, want, atol=1e-5)
    gy = torch.randn_like(y)
    gx, gw, gb = torch.autograd.grad(y, [x, conv.weight, conv.bias], gy)
    wx, ww, wb = torch.autograd.grad(want, [x, conv.weight, conv.bias], gy)
    assert torch.allclose(gx, wx, atol=1e-4) and torch.allclose(gw, ww, atol=1e-4) and torch.allclose(gb, wb, atol=1e-4)
    assert conv(x[0]).shape == want.shape[1:]
    assert [tuple(p.shape) for p in conv.reference_parameters()] == [(6, 3, k, k), (6,)]
    with pytest.raises(ValueError):
        conv(torch.randn(2, 4, 9, 10))


def test_im2col_column_order():
    x = torch.arange(2 * 2 * 3 * 3, dtype=torch.float32).reshape(2, 2, 3, 3)
    cols = im2col(x, 2, 2, 1, 0)
    assert cols.shape == (2 * 2 * 2, 2 * 2 * 2)
    # first row = top-left window of image 0: channel 0 (0,1,3,4) then channel 1 (9,10,12,13)
    assert cols[0].tolist() == [0, 1, 3, 4, 9, 10, 12, 13]


def test_hungarian_matches_brute_force():
    g = torch.Generator().manual_seed(1)
    for n in (1, 2, 3, 5, 6):
        cost = torch.randint(0, 30, (n, n), generator=g).tolist()
        h = HungarianAlgorithm(cost)
        a = h.get_assignment()
        assert sorted(a) == list(range(n))
        best = min(sum(cost[i][p[i]] for i in range(n)) for p in itertools.permutations(range(n)))
        assert h.total_cost() == best
    assert HungarianAlgorithm([[4, 1, 3], [2, 0, 5], [3, 2, 2]]).get_assignment() == [1, 0, 2]
    # padded rectangular problem: the sentinel column absorbs the unmatched row
    big = 10 ** 6
    a = HungarianAlgorithm([[1, 9, big], [9, 1, big], [5, 5, big]]).get_assignment()
    assert a[0] == 0 and a[1] == 1 and a[2] == 2
    with pytest.raises(ValueError):
        HungarianAlgorithm([[1, 2], [3]])
