"""CPU module / model behaviour: shapes, argument rejection, cache == no-cache, batched == per-sample, convergence,
optimizers, schedules, DPTC golden bytes (modelled on the reference's test/gpt_test.dart, kv_cache_test.dart,
batched_test.dart, optim_test.dart, lr_scheduler_test.dart, serialize_test.dart)."""
import json
import math
import random
import struct

import pytest
import torch

import dart_pytorch_b200 as dp
from dart_pytorch_b200 import nn
from dart_pytorch_b200.nn.transformer import Activation


def tiny_gpt(seed=0, **kw):
    base = dict(vocab_size=65, max_ctx=32, embed_dim=64, num_layers=2, num_heads=4, init_std=0.02, seed=seed)
    base.update(kw)
    return dp.GPT(dp.GPTConfig(**base))


def test_linear_layout_and_checks():
    lin = nn.Linear(4, 3, seed=1)
    assert lin.weight.shape == (3, 4) and lin.bias.shape == (3,)
    assert [tuple(p.shape) for p in lin.reference_parameters()] == [(3, 4), (1, 3)]
    assert float(lin.weight.abs().max()) <= 0.5 + 1e-6
    assert lin(torch.randn(2, 5, 4)).shape == (2, 5, 3)
    with pytest.raises(ValueError):
        lin(torch.randn(4))
    with pytest.raises(ValueError):
        lin(torch.randn(2, 5))
    assert torch.equal(nn.Linear(4, 3, seed=1).weight, lin.weight)
    assert not torch.equal(nn.Linear(4, 3, seed=2).weight, lin.weight)


def test_module_train_eval_recursion_and_param_order():
    blk = nn.TransformerBlock(16, 2, dropout_p=0.1, attn_bias=True)
    blk.eval()
    assert not blk.training and not blk.mha.training and not blk.dropout.training
    blk.train()
    assert blk.mha.wo.training
    shapes = [tuple(p.shape) for p in blk.reference_parameters()]
    # ln1 g,b, ln2 g,b, (wq w,b)x2, (wk w,b)x2, (wv w,b)x2, wo w,b, ffn1 w,b, ffn2 w,b
    assert shapes[:4] == [(16,)] * 4
    assert shapes[4:16] == [(8, 16), (1, 8)] * 6
    assert shapes[16:] == [(16, 16), (1, 16), (64, 16), (1, 64), (16, 64), (1, 16)]


def test_mha_gqa_grouping_cache_and_mask_rules():
    torch.manual_seed(0)
    mha = nn.MultiHeadAttention(16, 4, num_kv_heads=2, rope=nn.RopeCache(32, 4))
    x = torch.randn(6, 16)
    full = mha(x, causal=True)
    cache = nn.MHACache(2)
    a = mha(x[:4], cache=cache, causal=True, start_pos=0)
    b = mha(x[4:5], cache=cache, start_pos=4)
    c = mha(x[5:6], cache=cache, start_pos=5)
    assert cache.seq_len == 6 and cache.k[0].shape == (6, 4)
    assert torch.allclose(torch.cat([a, b, c]), full, atol=1e-5)
    with pytest.raises(ValueError):
        mha(x[:1], mask=torch.zeros(1, 7), cache=cache)
    with pytest.raises(ValueError):
        nn.MultiHeadAttention(16, 4, num_kv_heads=3)
    with pytest.raises(ValueError):
        nn.MultiHeadAttention(15, 4)
    # explicit additive causal mask == causal flag
    m2 = nn.MultiHeadAttention(16, 4)
    assert torch.allclose(m2(x, mask=nn.causal_mask(6)), m2(x, causal=True), atol=1e-5)
    # batched == per-sample
    xb = torch.randn(3, 6, 16)
    yb = m2(xb, causal=True)
    for i in range(3):
        assert torch.allclose(yb[i], m2(xb[i], causal=True), atol=1e-5)


def test_cross_attention_and_decoder_shapes():
    ca = nn.MultiHeadCrossAttention(16, 12, 4)
    assert ca(torch.randn(5, 16), torch.randn(7, 12)).shape == (5, 16)
    assert ca(torch.randn(2, 5, 16), torch.randn(2, 7, 12)).shape == (2, 5, 16)
    dec = nn.TransformerDecoder(2, 16, 4, memory_dim=12)
    assert dec(torch.randn(5, 16), torch.randn(7, 12)).shape == (5, 16)


def test_positional_encodings():
    pe = nn.SinusoidalPositionalEncoding(8)
    y = pe(torch.zeros(4, 8), start_pos=2)
    assert abs(float(y[0, 0]) - math.sin(2.0)) < 1e-6 and abs(float(y[0, 1]) - math.cos(2.0)) < 1e-6
    assert abs(float(y[1, 2]) - math.sin(3.0 * 10000 ** (-2 / 8))) < 1e-6
    lp = nn.LearnedPositionalEmbedding(10, 8)
    assert torch.allclose(lp(torch.zeros(3, 8), start_pos=4), lp.table.weight[4:7])
    with pytest.raises(ValueError):
        lp(torch.zeros(8, 8), start_pos=4)


def test_gpt_shapes_tied_params_and_limits():
    m = tiny_gpt()
    assert m(torch.randint(0, 65, (7,))).shape == (7, 65)
    assert m(torch.randint(0, 65, (3, 7))).shape == (3, 7, 65)
    assert len(m.reference_parameters()) == 46
    untied = tiny_gpt(tie_weights=False)
    assert len(untied.reference_parameters()) == 47
    with pytest.raises(ValueError):
        m(torch.zeros(33, dtype=torch.long))
    with pytest.raises(ValueError):
        dp.GPTConfig(vocab_size=10, max_ctx=8, embed_dim=10, num_layers=1, num_heads=3)
    x = torch.randint(0, 65, (2, 9))
    per = torch.stack([m(x[0]), m(x[1])])
    assert torch.allclose(m(x), per, atol=1e-5)


def test_gpt_cache_equals_no_cache_and_seeded_sampling():
    m = tiny_gpt(seed=3)
    prompt = [1.0, 5.0, 9.0, 2.0]
    a = m.generate(prompt, 12, temperature=0.0, use_cache=True)
    b = m.generate(prompt, 12, temperature=0.0, use_cache=False)
    assert a == b and len(a) == 16 and a[:4] == prompt
    s1 = m.generate(prompt, 10, temperature=0.9, top_k=5, rng=random.Random(3))
    s2 = m.generate(prompt, 10, temperature=0.9, top_k=5, rng=random.Random(3), use_cache=False)
    assert s1 == s2
    assert m.training  # restored
    with pytest.raises(ValueError):
        m.generate([], 3)
    with pytest.raises(ValueError):
        m.generate([1.0] * 40, 3)
    long = m.generate([1.0] * 30, 8, temperature=0.0)  # cache fills at maxCtx: stops early
    assert len(long) == 33
    assert len(m.generate([1.0] * 40, 3, temperature=0.0, use_cache=False)) == 43


def test_tiny_char_gpt_config_trains_saves_loads_generates():
    """The CPU baseline config: 200 Adam steps with warmup + cosine and clip 1.0, DPTC round trip, greedy generate."""
    torch.manual_seed(0)
    m = tiny_gpt(dropout_p=0.1)
    opt = dp.Adam(m.parameters(), lr=3e-3)
    sched = dp.LinearWarmupCosineDecay(opt, warmup_steps=20, total_steps=200, max_lr=3e-3)
    g = torch.Generator().manual_seed(0)
    x = torch.randint(0, 65, (8, 32), generator=g)
    y = torch.roll(x, -1, 1)
    first = last = None
    for step in range(200):
        opt.zero_grad()
        loss = m.loss(x, y)
        loss.backward()
        dp.clip_grad_norm(m.parameters(), 1.0)
        opt.step()
        sched.step()
        first = float(loss) if first is None else first
        last = float(loss)
    assert first > 3.5 and last < 0.5
    blob = dp.Checkpoint.save_bytes(m)
    other = tiny_gpt(seed=99, dropout_p=0.1)
    dp.Checkpoint.load_into_bytes(other, blob)
    assert m.generate([3.0, 4.0], 32, temperature=0.0) == other.generate([3.0, 4.0], 32, temperature=0.0)


def test_adam_single_step_formula_and_weight_decay():
    p = torch.tensor([1.0, -2.0], requires_grad=True)
    opt = dp.Adam([p], lr=0.1, weight_decay=0.5)
    p.grad = torch.tensor([0.5, -0.25])
    opt.step()
    # t=1: m/bc1 = g, sqrt(v/bc2) = |g| -> update = lr*sign(g) (+eps) + lr*wd*p
    expect = torch.tensor([1.0 - (0.1 * 0.5 / (0.5 + 1e-8) + 0.1 * 0.5 * 1.0), -2.0 - (-0.1 + 0.1 * 0.5 * -2.0)])
    assert torch.allclose(p.detach(), expect, atol=1e-6)
    q = torch.tensor([1.0], requires_grad=True)
    dp.Adam([q], lr=0.1).step()  # no grad -> skipped
    assert float(q) == 1.0


def test_sgd_momentum_and_quadratic_bowl():
    p = torch.tensor([1.0], requires_grad=True)
    opt = dp.SGD([p], lr=0.1, momentum=0.9, weight_decay=0.1)
    p.grad = torch.tensor([1.0])
    opt.step()  # g = 1 + 0.1*1 = 1.1; v = g; p = 1 - 0.11
    assert abs(float(p) - 0.89) < 1e-6
    p.grad = torch.tensor([1.0])
    opt.step()  # g = 1.089; v = 0.9*1.1 + 1.089 = 2.079; p = 0.89 - 0.2079
    assert abs(float(p) - 0.6821) < 1e-6
    w = torch.tensor([3.0, -4.0], requires_grad=True)
    o = dp.SGD([w], lr=0.1)
    for _ in range(200):
        o.zero_grad()
        (w * w).sum().backward()
        o.step()
    assert float(w.abs().max()) < 1e-6


def test_clip_grad_norm_rules():
    a = torch.zeros(2, requires_grad=True)
    b = torch.zeros(1, requires_grad=True)
    a.grad, b.grad = torch.tensor([3.0, 0.0]), torch.tensor([4.0])
    n = dp.clip_grad_norm([a, b], 1.0)
    assert abs(n - 5.0) < 1e-9 and torch.allclose(a.grad, torch.tensor([0.6, 0.0])) and abs(float(b.grad) - 0.8) < 1e-6
    n2 = dp.clip_grad_norm([a, b], 10.0)
    assert abs(n2 - 1.0) < 1e-6 and abs(float(b.grad) - 0.8) < 1e-6
    a.grad = torch.tensor([float("nan"), 1.0])
    n3 = dp.clip_grad_norm([a, b], 0.1)
    assert math.isnan(n3) and abs(float(b.grad) - 0.8) < 1e-6  # not scaled when the norm is not finite
    with pytest.raises(ValueError):
        dp.clip_grad_norm([a], 0.0)


def test_schedulers_boundaries():
    p = torch.zeros(1, requires_grad=True)
    opt = dp.SGD([p], lr=1.0)
    s = dp.LinearWarmupCosineDecay(opt, warmup_steps=10, total_steps=100, max_lr=2.0, min_lr=0.2)
    assert abs(opt.lr - 0.2) < 1e-12
    assert abs(s.lr_at(10) - 2.0) < 1e-12 and abs(s.lr_at(100) - 0.2) < 1e-12 and abs(s.lr_at(500) - 0.2) < 1e-12
    assert abs(s.lr_at(55) - (0.2 + 0.5 * 1.8 * (1 + math.cos(math.pi * 0.5)))) < 1e-12
    for _ in range(10):
        s.step()
    assert s.step_count == 10 and abs(opt.lr - 2.0) < 1e-12
    st = dp.StepLR(opt, step_size=3, gamma=0.5, initial_lr=1.0)
    assert opt.lr == 1.0
    for _ in range(3):
        st.step()
    assert abs(opt.lr - 0.5) < 1e-12
    with pytest.raises(ValueError):
        dp.StepLR(opt, step_size=0)
    with pytest.raises(ValueError):
        dp.LinearWarmupCosineDecay(opt, warmup_steps=5, total_steps=3, max_lr=1.0)


def test_dptc_golden_bytes_and_rejections():
    lin = nn.Linear(2, 3, seed=0)
    with torch.no_grad():
        lin.weight.copy_(torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]]))
        lin.bias.copy_(torch.tensor([0.5, -0.5, 0.25]))
    blob = dp.Checkpoint.save_bytes(lin)
    header = b'{"version":1,"params":[{"shape":[3,2]},{"shape":[1,3]}],"totalScalars":9}'
    expect = b"DPTC" + struct.pack("<II", 1, len(header)) + header + \
        struct.pack("<9f", 1, 2, 3, 4, 5, 6, 0.5, -0.5, 0.25)
    assert blob == expect
    half = dp.Checkpoint.save_bytes(lin, fp16=True)
    hh = json.loads(half[12:12 + struct.unpack("<I", half[8:12])[0]])
    assert hh["params"][0] == {"shape": [3, 2], "dtype": "F16"}
    assert len(half) - 12 - struct.unpack("<I", half[8:12])[0] == 18
    other = nn.Linear(2, 3, seed=5)
    dp.Checkpoint.load_into_bytes(other, half)
    assert torch.allclose(other.weight, lin.weight) and torch.allclose(other.bias, lin.bias)
    before = other.weight.clone()
    for bad in (b"DPT", b"XXXX" + blob[4:], blob[:4] + struct.pack("<I", 2) + blob[8:], blob[:20], blob[:-4],
                blob + b"\0\0\0\0"):
        with pytest.raises(ValueError):
            dp.Checkpoint.load_into_bytes(other, bad)
    wrong = nn.Linear(3, 3)
    with pytest.raises(ValueError):
        dp.Checkpoint.load_into_bytes(wrong, blob)
    with pytest.raises(ValueError):
        dp.Checkpoint.load_into_bytes(nn.LayerNorm(3), blob)
    bad_dtype = blob.replace(b'{"shape":[3,2]}', b'{"shape":[3,2],"dtype":"I8"}')
    bad_dtype = bad_dtype[:8] + struct.pack("<I", len(header) + 13) + bad_dtype[12:]
    with pytest.raises(ValueError):
        dp.Checkpoint.load_into_bytes(other, bad_dtype)
    assert torch.equal(other.weight, before)  # nothing was written by the failed loads


def test_tensor_facade_contract():
    T = dp.Tensor
    a = T.fromList([2, 2], [1, 2, 3, 4], requiresGrad=True)
    b = T.fromList([2, 2], [1, 0, 0, 1])
    loss = (a.matmul(b) * 2.0).sum()
    assert loss.shape == [1, 1]
    loss.backward()
    assert a.grad.toList() == [2.0, 2.0, 2.0, 2.0]
    with pytest.raises(ValueError):
        T.fromList([2, 2], [1, 2, 3])
    with pytest.raises(RuntimeError):
        T.fromList([1], [1.0]).backward()
    c = T.fill([3], 2.0)
    c.assign(T.fromList([3], [1, 2, 3]))
    assert c.toList() == [1.0, 2.0, 3.0]
    h = T.fromList([2], [1.0, 65520.0]).toFp16()
    assert h.dtype == dp.DType.fp16 and h.toList()[0] == 1.0 and math.isinf(h.toList()[1])
    with pytest.raises(RuntimeError):
        h.assign(c)
    out = T.noGrad(lambda: a * 3.0)
    assert not out.requiresGrad
    logits = T.fromList([2, 3], [0.0, 1.0, 2.0, 2.0, 1.0, 0.0], requiresGrad=True)
    ce = logits.crossEntropy(T.fromList([2], [2.0, 0.0]))
    assert ce.shape == [2, 1]
    lin = nn.Linear(3, 2)
    assert isinstance(lin(logits), T)


def test_train_state_sidecar_resumes_exactly(tmp_path):
    """Parameters (DPTC) + sidecar (optimizer moments, step, scheduler, RNG) reproduce an uninterrupted run."""
    import random
    from dart_pytorch_b200.io.dptc import Checkpoint
    from dart_pytorch_b200.io.train_state import load_train_state, save_train_state
    from dart_pytorch_b200.models import GPT, GPTConfig
    import dart_pytorch_b200 as dp

    def make():
        m = GPT(GPTConfig(vocab_size=31, max_ctx=12, embed_dim=16, num_layers=1, num_heads=2, seed=4))
        o = dp.Adam(m.parameters(), lr=1e-2, weight_decay=0.05)
        s = dp.LinearWarmupCosineDecay(o, warmup_steps=3, total_steps=20, max_lr=1e-2, min_lr=1e-3)
        return m, o, s

    def run(m, o, s, steps, g):
        for _ in range(steps):
            x = torch.randint(0, 31, (2, 12), generator=g)
            o.zero_grad()
            m.loss(x[:, :-1], x[:, 1:]).backward()
            o.step()
            s.step()
    g = torch.Generator().manual_seed(0)
    m1, o1, s1 = make()
    run(m1, o1, s1, 4, g)
    Checkpoint.save_file(m1, str(tmp_path / "m.dptc"))
    save_train_state(str(tmp_path / "m.dpts"), o1, s1, extra={"tokens_seen": 96})
    gstate = g.get_state()
    random.seed(123)
    torch.manual_seed(77)
    save_train_state(str(tmp_path / "rng.dpts"))
    want_py, want_t = random.random(), torch.rand(3)
    run(m1, o1, s1, 3, g)
    m2, o2, s2 = make()
    Checkpoint.load_into_file(m2, str(tmp_path / "m.dptc"))
    extra = load_train_state(str(tmp_path / "m.dpts"), o2, s2, restore_rng=False)
    assert extra == {"tokens_seen": 96} and o2._step == 4 and s2.step_count == 4 and abs(o2.lr - o1.lr) > 0
    g2 = torch.Generator()
    g2.set_state(gstate)
    run(m2, o2, s2, 3, g2)
    for a, b in zip(m1.parameters(), m2.parameters()):
        assert torch.allclose(a, b, atol=1e-6)
    assert abs(o1.lr - o2.lr) < 1e-12
    load_train_state(str(tmp_path / "rng.dpts"))
    assert random.random() == want_py and torch.equal(torch.rand(3), want_t)
    blob = (tmp_path / "m.dpts").read_bytes()
    (tmp_path / "bad.dpts").write_bytes(b"XXXX" + blob[4:])
    with pytest.raises(ValueError):
        load_train_state(str(tmp_path / "bad.dpts"), o2, s2)
    (tmp_path / "short.dpts").write_bytes(blob[:len(blob) - 10])
    with pytest.raises(ValueError):
        load_train_state(str(tmp_path / "short.dpts"), o2, s2)
    sgd = dp.SGD(m2.parameters(), lr=0.1)
    with pytest.raises(ValueError):
        load_train_state(str(tmp_path / "m.dpts"), sgd)
