"""CPU tests of the KV cache, grouped-query attention and the batched ``[B, S, D]`` paths, case by case after the
reference's test/kv_cache_test.dart, test/gqa_test.dart and test/batched_test.dart."""
import pytest
import torch

from dart_pytorch_b200 import GPT, GPTConfig, Adam
from dart_pytorch_b200 import ops as F
from dart_pytorch_b200.nn import (Dropout, Embedding, LayerNorm, LearnedPositionalEmbedding, Linear,
                                  SinusoidalPositionalEncoding)
from dart_pytorch_b200.nn.attention import EncoderCache, MHACache, MultiHeadAttention
from dart_pytorch_b200.nn.transformer import TransformerBlock, TransformerEncoder


def _x(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


# ------------------------------------------------------------------------------------------------- KV cache ---
def test_empty_cache_and_append_growth():
    c = MHACache(num_kv_heads=2)
    assert c.seqLen == 0 and c.k == [None, None] and c.v == [None, None]
    k1, v1 = _x(1, 3, 8, seed=1), _x(1, 3, 8, seed=2)
    c.append(k1, v1)
    k2, v2 = _x(1, 2, 8, seed=3), _x(1, 2, 8, seed=4)
    ka, va = c.append(k2, v2)
    assert c.seqLen == 5 and ka.shape == (1, 5, 8)
    assert torch.equal(ka, torch.cat([k1, k2], 1)) and torch.equal(va, torch.cat([v1, v2], 1))
    assert c.k[1].shape == (5, 4) and torch.equal(c.k[1], torch.cat([k1, k2], 1)[0, :, 4:])   # per-head view
    c.reset()
    assert c.seqLen == 0
    enc = EncoderCache.empty(num_layers=3, num_kv_heads=2)
    assert len(enc.layers) == 3 and all(l.num_kv_heads == 2 for l in enc.layers) and enc.seq_len == 0


def test_cache_prefill_with_mask_matches_uncached_and_mask_rule():
    mha = MultiHeadAttention(16, 4, seed=3)
    x = _x(6, 16)
    mask = F.causal_mask(6)
    cache = MHACache(4)
    assert torch.allclose(mha(x, mask=mask, cache=cache), mha(x, mask=mask), atol=1e-6)
    assert cache.seqLen == 6
    with pytest.raises(ValueError):
        mha(_x(1, 16), mask=F.causal_mask(1), cache=cache)         # mask + non-empty cache


def test_cached_step_equals_last_row_of_uncached_forward():
    cfg = GPTConfig(vocab_size=30, max_ctx=16, embed_dim=16, num_layers=2, num_heads=4, seed=5)
    gpt = GPT(cfg).eval()
    toks = torch.tensor([3, 7, 1, 9, 4, 2])
    full = gpt(toks)
    cache = EncoderCache.empty(2, 4)
    gpt(toks[:5], start_pos=0, cache=cache)
    step = gpt(toks[5:], start_pos=5, cache=cache)
    assert cache.seq_len == 6 and torch.allclose(step[-1], full[-1], atol=1e-5)
    a = gpt.generate([3, 7, 1], 6, temperature=0.0, use_cache=True)
    b = gpt.generate([3, 7, 1], 6, temperature=0.0, use_cache=False)
    assert a == b and len(a) == 9


# ------------------------------------------------------------------------------------------------------ GQA ---
def test_gqa_construction_rules_and_parameter_shapes():
    assert MultiHeadAttention(16, 4).num_kv_heads == 4                        # default: plain MHA
    g = MultiHeadAttention(16, 4, num_kv_heads=2)
    assert g.num_head_groups == 2 and g.w_qkv.shape == (16 + 2 * 8, 16)
    m = MultiHeadAttention(16, 4, num_kv_heads=1)
    assert m.num_head_groups == 4 and m.w_qkv.shape == (16 + 2 * 4, 16)
    assert len(g.own_reference_parameters()) == 4 + 2 + 2                      # wq x4, wk x2, wv x2
    with pytest.raises(ValueError):
        MultiHeadAttention(16, 4, num_kv_heads=3)


def test_full_kv_heads_equal_plain_mha_and_gqa_shapes():
    x = _x(5, 16)
    a, b = MultiHeadAttention(16, 4, seed=9), MultiHeadAttention(16, 4, num_kv_heads=4, seed=9)
    assert torch.equal(a(x, causal=True), b(x, causal=True))
    for kv in (2, 1):
        assert MultiHeadAttention(16, 4, num_kv_heads=kv, seed=1)(x, causal=True).shape == (5, 16)
        assert MultiHeadAttention(16, 4, num_kv_heads=kv, seed=1)(_x(2, 5, 16)).shape == (2, 5, 16)


def test_mqa_query_heads_share_the_single_kv_head():
    mha = MultiHeadAttention(16, 4, num_kv_heads=1, seed=2)
    x = _x(5, 16)
    hd = 4
    k = x @ mha.wk_weight(0).t()
    v = x @ mha.wv_weight(0).t()
    heads = [F.sdpa(x @ mha.wq_weight(h).t(), k, v) for h in range(4)]
    want = mha.wo(torch.cat(heads, 1))
    assert torch.allclose(mha(x), want, atol=1e-5) and k.shape == (5, hd)


def test_gqa_cache_holds_kv_heads_and_token_by_token_matches_prefill():
    mha = MultiHeadAttention(16, 4, num_kv_heads=2, seed=4)
    x = _x(6, 16)
    full = mha(x, causal=True)
    cache = MHACache(2)
    rows = [mha(x[t:t + 1], cache=cache, start_pos=t, causal=True) for t in range(6)]
    assert len(cache.k) == 2 and cache.k[0].shape == (6, 4) and cache.k_buf.shape[2] == 2 * 4
    assert torch.allclose(torch.cat(rows, 0), full, atol=1e-5)


# -------------------------------------------------------------------------------------------------- batched ---
def test_reshape_roundtrip_and_gradient():
    x = _x(2, 3, 4).requires_grad_()
    flat = x.reshape(6, 4)
    assert torch.equal(flat.reshape(2, 3, 4), x) and flat.data_ptr() == x.data_ptr()
    with pytest.raises(RuntimeError):
        x.reshape(5, 5)
    (flat * torch.arange(24.0).reshape(6, 4)).sum().backward()
    assert torch.equal(x.grad, torch.arange(24.0).reshape(2, 3, 4))


def test_rowwise_ops_on_3d_equal_per_sample():
    x = _x(3, 5, 8)
    assert torch.allclose(F.softmax(x), torch.stack([F.softmax(s) for s in x]), atol=1e-7)
    g, b = _x(8, seed=1), _x(8, seed=2)
    assert torch.allclose(F.layer_norm(x, g, b), torch.stack([F.layer_norm(s, g, b) for s in x]), atol=1e-6)
    logits, tgt = _x(3, 5, 11), torch.randint(0, 11, (3, 5), generator=torch.Generator().manual_seed(0))
    assert torch.allclose(F.cross_entropy(logits, tgt), F.cross_entropy(logits.reshape(15, 11), tgt.reshape(15)))
    w = _x(8, 6, seed=3)
    assert torch.allclose(F.matmul(x, w), torch.stack([s @ w for s in x]), atol=1e-6)


def test_batched_cross_entropy_gradients_equal_summed_per_sample():
    logits = _x(2, 4, 7).requires_grad_()
    tgt = torch.tensor([[1, 2, 3, 0], [6, 5, 4, 3]])
    F.cross_entropy(logits, tgt).sum().backward()
    per = logits.detach().clone().requires_grad_()
    sum(F.cross_entropy(per[i], tgt[i]).sum() for i in range(2)).backward()
    assert torch.allclose(logits.grad, per.grad, atol=1e-6)


def test_modules_on_3d_equal_per_sample():
    emb = Embedding(20, 8, seed=1)
    idx = torch.randint(0, 20, (3, 5), generator=torch.Generator().manual_seed(1))
    assert emb(idx).shape == (3, 5, 8) and torch.equal(emb(idx), torch.stack([emb(i) for i in idx]))
    lin = Linear(8, 6, seed=2)
    x = _x(3, 5, 8).requires_grad_()
    y = lin(x)
    assert y.shape == (3, 5, 6) and torch.allclose(y, torch.stack([lin(s) for s in x]), atol=1e-6)
    y.sum().backward()
    assert torch.allclose(lin.weight.grad, torch.ones(15, 6).t() @ x.detach().reshape(15, 8), atol=1e-5)
    ln = LayerNorm(8)
    assert torch.allclose(ln(x), torch.stack([ln(s) for s in x]), atol=1e-6)
    drop = Dropout(0.4)
    drop.eval()
    assert drop(x) is x
    drop.train()
    z = drop(torch.ones(4, 50, 8))
    assert z.shape == (4, 50, 8) and 0.3 < float((z == 0).float().mean()) < 0.5


def test_positional_modules_on_3d_and_limits():
    x = _x(2, 5, 8)
    sin = SinusoidalPositionalEncoding(8)
    assert torch.allclose(sin(x), torch.stack([sin(s) for s in x]), atol=1e-6)
    pos = LearnedPositionalEmbedding(6, 8, seed=3)
    assert torch.allclose(pos(x), torch.stack([pos(s) for s in x]), atol=1e-6)
    assert torch.allclose(pos(x[:, :2], start_pos=4), torch.stack([pos(s[:2], start_pos=4) for s in x]))
    with pytest.raises(ValueError):
        pos(x, start_pos=2)                                       # 2 + 5 > 6


def test_concat_and_split_roundtrip_with_gradient_routing():
    a, b = _x(2, 4).requires_grad_(), _x(3, 4, seed=1).requires_grad_()
    c = F.concat([a, b], axis=0)
    assert c.shape == (5, 4)
    (c * torch.arange(20.0).reshape(5, 4)).sum().backward()
    assert torch.equal(a.grad, torch.arange(8.0).reshape(2, 4)) and torch.equal(b.grad, torch.arange(8.0, 20.0).reshape(3, 4))
    parts = F.split_rows(_x(6, 4), 2)
    assert len(parts) == 3 and torch.equal(F.concat(parts, axis=0), _x(6, 4))
    with pytest.raises(ValueError):
        F.split_rows(_x(5, 4), 2)


def test_attention_block_and_encoder_on_3d_equal_per_sample():
    x = _x(3, 5, 16)
    mha = MultiHeadAttention(16, 4, seed=6)
    assert torch.allclose(mha(x), torch.stack([mha(s) for s in x]), atol=1e-5)
    mask = F.causal_mask(5)
    assert torch.allclose(mha(x, mask=mask), torch.stack([mha(s, mask=mask) for s in x]), atol=1e-5)
    assert torch.allclose(mha(x, causal=True), mha(x, mask=mask), atol=1e-5)        # fused flag == shared mask
    blk = TransformerBlock(16, 4, seed=7).eval()
    assert torch.allclose(blk(x, causal=True), torch.stack([blk(s, causal=True) for s in x]), atol=1e-5)
    enc = TransformerEncoder(2, 16, 4, seed=8).eval()
    assert torch.allclose(enc(x), torch.stack([enc(s) for s in x]), atol=1e-5)


def test_gpt_batched_forward_and_training_step():
    gpt = GPT(GPTConfig(vocab_size=20, max_ctx=8, embed_dim=16, num_layers=1, num_heads=4, seed=2))
    toks = torch.randint(0, 20, (4, 9), generator=torch.Generator().manual_seed(4))
    x, y = toks[:, :-1], toks[:, 1:]
    gpt.eval()
    logits = gpt(x)
    assert logits.shape == (4, 8, 20) and torch.allclose(logits, torch.stack([gpt(r) for r in x]), atol=1e-5)
    gpt.train()
    opt = Adam(gpt.parameters(), lr=0.01)
    first = last = None
    for _ in range(30):
        opt.zero_grad()
        loss = gpt.loss(x, y)
        loss.backward()
        opt.step()
        last = float(loss.detach())
        first = last if first is None else first
    assert last < 0.7 * first


def test_per_head_cache_appends_with_the_reference_signature():
    c = MHACache(2)
    k0 = c.appendK(0, torch.ones(3, 4))
    c.appendK(1, 2 * torch.ones(3, 4))
    c.appendV(0, 5 * torch.ones(3, 4))
    c.appendV(1, 6 * torch.ones(3, 4))
    assert k0.shape == (3, 4) and c.seqLen == 3 and c.v[1][:, 0].tolist() == [6.0, 6.0, 6.0]
    k1 = c.appendK(0, 3 * torch.ones(1, 4))
    assert k1.shape == (4, 4) and k1[:, 0].tolist() == [1.0, 1.0, 1.0, 3.0] and c.seqLen == 4
    assert c.k[1][:3, 0].tolist() == [2.0, 2.0, 2.0]
    with pytest.raises(IndexError):
        c.appendK(2, torch.ones(1, 4))
    c.reset()
    assert c.seqLen == 0 and c.appendV(1, torch.ones(2, 4)).shape == (2, 4) and c.seqLen == 2
