"""CPU tests of cross attention, the decoder stack, the encoder-decoder transformer, AFT, the SwiGLU feed-forward and
``TransformerLM``, case by case after the reference's test/encoder_decoder_test.dart, test/aft_test.dart,
test/swiglu_test.dart and test/transformer_lm_test.dart."""
import math

import pytest
import torch

from dart_pytorch_b200 import Adam, SGD
from dart_pytorch_b200 import ops as F
from dart_pytorch_b200.models import AFTLanguageModel, EncoderDecoderTransformer, TransformerLM
from dart_pytorch_b200.models.seq_models import AFTAttention, AFTBlock
from dart_pytorch_b200.nn.attention import MultiHeadCrossAttention
from dart_pytorch_b200.nn.layers import SwiGluFfn
from dart_pytorch_b200.nn.transformer import TransformerDecoder, TransformerDecoderBlock, TransformerEncoder


def _x(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


def _fit(model, params, loss_fn, steps, lr=0.01):
    opt = Adam(params, lr=lr)
    first = last = None
    for _ in range(steps):
        opt.zero_grad()
        loss = loss_fn()
        loss.backward()
        opt.step()
        last = float(loss.detach())
        first = last if first is None else first
    return first, last


# ------------------------------------------------------------------------------------------ encoder-decoder ---
def test_cross_attention_shapes_batching_and_rejections():
    ca = MultiHeadCrossAttention(16, 24, 4, seed=1)
    q, kv = _x(5, 16), _x(7, 24, seed=1)
    assert ca(q, kv).shape == (5, 16)
    qb, kvb = _x(3, 5, 16), _x(3, 7, 24, seed=1)
    assert torch.allclose(ca(qb, kvb), torch.stack([ca(a, b) for a, b in zip(qb, kvb)]), atol=1e-5)
    for bad_q, bad_kv in ((qb, kv), (_x(5, 15), kv), (q, _x(7, 23)), (qb, _x(2, 7, 24))):
        with pytest.raises(ValueError):
            ca(bad_q, bad_kv)
    with pytest.raises(ValueError):
        MultiHeadCrossAttention(16, 24, 3)


def test_decoder_block_trains_and_stack_matches_manual_composition():
    blk = TransformerDecoderBlock(16, 4, seed=2)
    x, mem = _x(6, 16), _x(9, 16, seed=3)
    assert blk(x, mem).shape == (6, 16) and blk(_x(2, 6, 16), _x(2, 9, 16)).shape == (2, 6, 16)
    target = _x(6, 16, seed=4)
    first, last = _fit(blk, blk.parameters(), lambda: ((blk(x, mem) - target) ** 2).mean(), 40)
    assert last < 0.6 * first
    dec = TransformerDecoder(2, 16, 4, seed=5).eval()
    h = x
    for b in dec.blocks:
        h = b(h, mem)
    assert torch.allclose(dec(x, mem), dec.final_norm(h), atol=1e-6)


def test_encoder_decoder_transformer_shapes_training_and_decoding():
    model = EncoderDecoderTransformer(12, 14, 16, 4, 1, 1, 10, 32, seed=1)
    src, tgt = torch.tensor([3, 4, 5, 6, 7]), torch.tensor([1, 3, 4, 5])
    assert model(src, tgt).shape == (4, 14)
    assert model(torch.stack([src, src]), torch.stack([tgt, tgt])).shape == (2, 4, 14)
    with pytest.raises(ValueError):
        model(torch.stack([src, src]), tgt)                                   # rank mismatch between src and tgt
    tgt_in, tgt_out = torch.tensor([1, 3, 4, 5, 6, 7]), torch.tensor([3, 4, 5, 6, 7, 2])
    first, last = _fit(model, model.parameters(), lambda: model.loss(src, tgt_in, tgt_out), 150)
    assert last < 0.1 * first
    assert model.greedy_decode(src, bos=1, eos=2, max_new_tokens=8) == [1, 3, 4, 5, 6, 7, 2]   # starts at BOS, stops at EOS


# ------------------------------------------------------------------------------------------------------ AFT ---
def _aft_loops(q, k, v, w, causal):
    T, D = q.shape
    out = torch.zeros(T, D, dtype=torch.float64)
    for t in range(T):
        lim = t + 1 if causal else T
        for d in range(D):
            logits = [float(k[s, d]) + float(w[t, s]) for s in range(lim)]
            m = max(logits)
            e = [math.exp(l - m) for l in logits]
            num = sum(ei * float(v[s, d]) for s, ei in zip(range(lim), e))
            out[t, d] = 1.0 / (1.0 + math.exp(-float(q[t, d]))) * num / sum(e)
    return out


@pytest.mark.parametrize("causal", [False, True])
def test_aft_full_matches_double_precision_loops_and_finite_differences(causal):
    q, k, v, w = _x(5, 3), _x(5, 3, seed=1), _x(5, 3, seed=2), 0.3 * _x(5, 5, seed=3)
    got = F.aft_full(q, k, v, w, causal=causal)
    assert torch.allclose(got.double(), _aft_loops(q, k, v, w, causal), atol=1e-5)
    ins = [t.double().requires_grad_() for t in (q, k, v, w)]
    assert torch.autograd.gradcheck(lambda a, b, c, d: F.aft_full(a, b, c, d, causal=causal), ins, atol=1e-5)
    if causal:
        F.aft_full(*ins, causal=True).sum().backward()
        assert float(torch.triu(ins[3].grad, diagonal=1).abs().sum()) == 0.0  # no gradient above the diagonal
    with pytest.raises((ValueError, RuntimeError)):
        F.aft_full(q, k[:4], v, w, causal=causal)


def test_aft_modules_shapes_limits_and_training():
    attn = AFTAttention(8, 10, masked=True, seed=1)
    assert attn(_x(6, 8)).shape == (6, 8) and attn.pos_bias.shape == (10, 10)
    assert float(attn.pos_bias.detach().abs().max()) <= 0.02
    blk = AFTBlock(8, 10, masked=True, seed=2)
    x, target = _x(6, 8), _x(6, 8, seed=5)
    opt = SGD(blk.parameters(), lr=0.05)
    losses = []
    for _ in range(40):
        opt.zero_grad()
        loss = ((blk(x) - target) ** 2).mean()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0]
    lm = AFTLanguageModel(11, 16, 1, 8, seed=3)
    toks = torch.tensor([1, 2, 3, 4, 5, 6, 7])
    assert lm(toks[:-1]).shape == (6, 11)
    with pytest.raises(ValueError):
        lm(torch.zeros(2, 3, dtype=torch.long))
    with pytest.raises(ValueError):
        lm(torch.zeros(9, dtype=torch.long))
    first, last = _fit(lm, lm.parameters(), lambda: lm.loss(toks[:-1], toks[1:]), 200, lr=0.02)
    assert last < 0.05


# --------------------------------------------------------------------------------------------------- SwiGLU ---
def test_swiglu_ffn_shape_parameters_and_manual_reference():
    ffn = SwiGluFfn(4, 6, seed=1)
    x = _x(2, 4)
    assert ffn(x).shape == (2, 4) and ffn(_x(3, 2, 4)).shape == (3, 2, 4)
    ref_params = ffn.reference_parameters()
    assert [tuple(p.shape) for p in ref_params] == [(6, 4), (6, 4), (4, 6)]          # gate, up, down; no biases
    gate, up, down = ref_params
    want = (torch.nn.functional.silu(x @ gate.t()) * (x @ up.t())) @ down.t()
    assert torch.allclose(ffn(x), want, atol=1e-6)
    ffn(x).sum().backward()
    assert ffn.w_gate_up.grad is not None and ffn.down.weight.grad is not None


# ------------------------------------------------------------------------------------------- TransformerLM ---
def test_causal_mask_structure():
    m = F.causal_mask(4)
    assert m.shape == (4, 4) and float(m[2, 1]) == 0.0 and float(m[1, 2]) == -1e9
    assert torch.equal(m == 0, torch.tril(torch.ones(4, 4)).bool())
    assert float(F.causal_mask(3, block_value=-5.0)[0, 2]) == -5.0


def test_transformer_encoder_structure_modes_and_gradients():
    enc = TransformerEncoder(3, 16, 4, dropout_p=0.1, seed=1)
    one = TransformerEncoder(1, 16, 4, seed=1)
    no_norm = TransformerEncoder(1, 16, 4, final_norm=False, seed=1)
    n = lambda m: sum(p.numel() for p in m.parameters())                           # noqa: E731
    per_block = n(one) - 32
    assert n(enc) == 3 * per_block + 32 and n(no_norm) == per_block
    x = _x(5, 16)
    assert enc.eval()(x).shape == (5, 16)
    enc.train()
    assert all(b.dropout.training for b in enc.blocks)
    enc.eval()
    assert not any(b.dropout.training for b in enc.blocks)
    enc(x, mask=F.causal_mask(5)).sum().backward()
    assert all(p.grad is not None for p in enc.parameters())


def test_transformer_lm_limits_overfit_and_greedy_generation():
    lm = TransformerLM(9, 16, 1, 4, 8, seed=2)
    toks = torch.tensor([1, 4, 2, 7, 3, 8, 5])
    assert lm(toks[:-1]).shape == (6, 9)
    assert sum(p.numel() for p in lm.parameters()) == 9 * 16 + sum(p.numel() for p in lm.encoder.parameters()) + 16 * 9 + 9
    with pytest.raises(ValueError):
        lm(torch.zeros(2, 2, 2, dtype=torch.long))
    with pytest.raises(ValueError):
        lm(torch.zeros(9, dtype=torch.long))
    first, last = _fit(lm, lm.parameters(), lambda: lm.loss(toks[:-1], toks[1:]), 200, lr=0.02)
    assert last < 0.05
    lm.eval()
    seq = [1]
    for _ in range(6):
        seq.append(int(lm(torch.tensor(seq))[-1].argmax()))
    assert seq == toks.tolist()
