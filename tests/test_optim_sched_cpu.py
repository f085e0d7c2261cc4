"""CPU tests of the optimizers, learning-rate schedules, dropout and gradient clipping, case by case after the
reference's test/optim_test.dart, test/lr_scheduler_test.dart and test/dropout_regularization_test.dart."""
import math

import pytest
import torch

from dart_pytorch_b200 import SGD, Adam, clip_grad_norm
from dart_pytorch_b200 import ops as F
from dart_pytorch_b200.nn import Dropout, Embedding, LayerNorm, Linear
from dart_pytorch_b200.nn.module import Module
from dart_pytorch_b200.optim.lr_scheduler import LinearWarmupCosineDecay, StepLR
from dart_pytorch_b200.tensor import Tensor


def _param(values):
    return torch.tensor(values, dtype=torch.float32, requires_grad=True)


# ------------------------------------------------------------------------------------------------------- SGD ---
def test_sgd_single_step_is_p_minus_lr_grad():
    p = _param([1.0, -2.0, 3.0])
    (p * torch.tensor([0.5, 1.0, -2.0])).sum().backward()
    SGD([p], lr=0.1).step()
    assert torch.allclose(p.detach(), torch.tensor([0.95, -2.1, 3.2]))


def test_grad_is_retained_across_step_and_zero_grad_clears():
    p = _param([1.0, 2.0])
    opt = SGD([p], lr=0.1)
    (p * p).sum().backward()
    g = p.grad.clone()
    opt.step()
    assert torch.equal(p.grad, g)
    opt.zero_grad()
    assert p.grad is None or float(p.grad.abs().sum()) == 0.0


def test_sgd_quadratic_bowl_converges():
    p = _param([3.0, -4.0])
    opt = SGD([p], lr=0.1)
    for _ in range(200):
        opt.zero_grad()
        (p * p).sum().backward()
        opt.step()
    assert float(p.detach().abs().max()) < 1e-6


def test_sgd_momentum_velocity_two_steps():
    p = _param([1.0])
    opt = SGD([p], lr=0.1, momentum=0.9)
    for expected in (0.9, 0.71):          # v1 = g = 1 -> 0.9 ; v2 = 0.9*1 + 1 = 1.9 -> 0.9 - 0.19
        opt.zero_grad()
        p.sum().backward()
        opt.step()
        assert float(p.detach()) == pytest.approx(expected, abs=1e-6)


def test_sgd_weight_decay_adds_wd_times_p_to_the_gradient():
    p = _param([2.0])
    opt = SGD([p], lr=0.5, weight_decay=0.1)
    p.sum().backward()
    opt.step()
    assert float(p.detach()) == pytest.approx(2.0 - 0.5 * (1.0 + 0.1 * 2.0))


# ------------------------------------------------------------------------------------------------------ Adam ---
def _ref_adam(p, g, m, v, t, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.0):
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    update = lr * (m / (1 - b1 ** t)) / (math.sqrt(v / (1 - b2 ** t)) + eps) + lr * wd * p
    return p - update, m, v


def test_adam_steps_match_the_reference_formula():
    p = _param([0.5, -1.5])
    opt = Adam([p], lr=0.01, weight_decay=0.1)
    want = [(0.5, 0.0, 0.0), (-1.5, 0.0, 0.0)]
    for t in (1, 2, 3):
        opt.zero_grad()
        (p * p * p).sum().backward()
        grads = p.grad.tolist()
        opt.step()
        want = [_ref_adam(pv, g, m, v, t, lr=0.01, wd=0.1) for (pv, m, v), g in zip(want, grads)]
        assert p.detach().tolist() == pytest.approx([w[0] for w in want], rel=1e-5)


def test_adam_bias_correction_at_t1_gives_a_step_of_lr():
    for g in (1e-4, 1.0, 1e4):            # |update| = lr whatever the gradient scale: no v_hat blow-up
        p = _param([0.0])
        (p * g).sum().backward()
        Adam([p], lr=0.01).step()
        assert float(p.detach()) == pytest.approx(-0.01, rel=1e-3)


def test_adam_quadratic_bowl_converges_faster_than_sgd():
    def run(make):
        p = _param([3.0, -4.0])
        opt = make(p)
        for _ in range(60):
            opt.zero_grad()
            (p * p).sum().backward()
            opt.step()
        return float(p.detach().abs().max())
    adam, sgd = run(lambda p: Adam([p], lr=0.3)), run(lambda p: SGD([p], lr=0.01))
    assert adam < 0.5 and adam < sgd


def test_adam_skips_parameters_without_gradients_and_keeps_state_tensors():
    a, b = _param([1.0]), _param([2.0])
    opt = Adam([a, b], lr=0.1)
    a.sum().backward()
    opt.step()
    m_before = opt._m[id(a)]
    assert float(b.detach()) == 2.0 and id(b) not in opt._m
    opt.zero_grad()
    (a.sum() + b.sum()).backward()
    opt.step()
    # the step counter is global: b's first update already uses the bias corrections of t = 2
    want = 2.0 - 0.1 * (0.1 / (1 - 0.9 ** 2)) / math.sqrt(0.001 / (1 - 0.999 ** 2))
    assert opt._m[id(a)] is m_before and float(b.detach()) == pytest.approx(want, rel=1e-5)


def test_sgd_trains_layernorm_gamma_beta_on_a_synthetic_target():
    torch.manual_seed(0)
    ln = LayerNorm(4)
    x = torch.randn(16, 4)
    target = F.layer_norm(x, torch.tensor([2.0, 0.5, -1.0, 1.5]), torch.tensor([0.1, -0.2, 0.3, 0.0]))
    opt = SGD(ln.parameters(), lr=0.2)
    for _ in range(300):
        opt.zero_grad()
        ((ln(x) - target) ** 2).mean().backward()
        opt.step()
    assert torch.allclose(ln.gamma.detach(), torch.tensor([2.0, 0.5, -1.0, 1.5]), atol=1e-2)
    assert torch.allclose(ln.beta.detach(), torch.tensor([0.1, -0.2, 0.3, 0.0]), atol=1e-2)


def test_adam_trains_embedding_on_a_lookup_regression():
    emb = Embedding(5, 3, seed=1)
    target = torch.arange(15, dtype=torch.float32).reshape(5, 3) / 10
    idx = torch.tensor([0, 1, 2, 3, 4, 4, 2])
    opt = Adam(emb.parameters(), lr=0.05)
    for _ in range(400):
        opt.zero_grad()
        ((emb(idx) - target[idx]) ** 2).mean().backward()
        opt.step()
    assert torch.allclose(emb.weight.detach(), target, atol=2e-2)


def test_assign_overwrites_in_place_and_rejects_mismatches():
    p = Tensor.fromList([3], [1.0, 2.0, 3.0], requiresGrad=True)
    storage = p.t
    p.assign(Tensor.fromList([3], [10.0, 20.0, 30.0]))
    assert p.t is storage and p.toList() == [10.0, 20.0, 30.0] and p.requiresGrad
    with pytest.raises(ValueError):
        p.assign(Tensor.fromList([4], [1, 2, 3, 4]))
    with pytest.raises(ValueError):
        p.assign(torch.zeros(3, device="meta"))


# ------------------------------------------------------------------------------------------------- schedules ---
def test_step_lr():
    opt = SGD([_param([0.0])], lr=123.0)
    with pytest.raises(ValueError):
        StepLR(opt, step_size=0)
    sched = StepLR(opt, step_size=3, gamma=0.5, initial_lr=0.8)
    assert opt.lr == 0.8                                   # set on construction
    seen = []
    for _ in range(7):
        sched.step()
        seen.append(opt.lr)
        assert sched.last_lr == opt.lr
    assert seen == pytest.approx([0.8, 0.8, 0.4, 0.4, 0.4, 0.2, 0.2])


def test_linear_warmup_cosine_decay_boundaries():
    opt = Adam([_param([0.0])], lr=1.0)
    for bad in (dict(warmup_steps=-1, total_steps=10), dict(warmup_steps=5, total_steps=0),
                dict(warmup_steps=11, total_steps=10), dict(warmup_steps=1, total_steps=10, max_lr=0.1, min_lr=0.2)):
        with pytest.raises(ValueError):
            LinearWarmupCosineDecay(opt, **bad)
    s = LinearWarmupCosineDecay(opt, warmup_steps=10, total_steps=110, max_lr=1.0, min_lr=0.1)
    assert opt.lr == pytest.approx(0.1)                     # lr_at(1) on construction
    assert s.lr_at(10) == pytest.approx(1.0)                # reaches max exactly at the end of warm-up
    assert s.lr_at(110) == pytest.approx(0.1) and s.lr_at(500) == pytest.approx(0.1)
    assert s.lr_at(60) == pytest.approx(0.55)               # midpoint of the cosine phase
    warm = [s.lr_at(t) for t in range(1, 11)]
    decay = [s.lr_at(t) for t in range(10, 111)]
    assert all(b > a for a, b in zip(warm, warm[1:])) and all(b <= a for a, b in zip(decay, decay[1:]))


@pytest.mark.parametrize("make", [lambda p: SGD([p], lr=0.5), lambda p: Adam([p], lr=0.5)])
def test_scheduler_drives_any_optimizer(make):
    p = _param([1.0])
    opt = make(p)
    sched = LinearWarmupCosineDecay(opt, warmup_steps=2, total_steps=4, max_lr=0.5)
    lrs = []
    for _ in range(5):
        opt.zero_grad()
        (p * p).sum().backward()
        opt.step()
        sched.step()
        lrs.append(opt.lr)
    assert lrs == pytest.approx([0.25, 0.5, 0.25, 0.0, 0.0]) and sched.stepCount == 5


# --------------------------------------------------------------------------------------- dropout / clipping ---
def test_dropout_function_contract():
    x = torch.ones(4000, requires_grad=True)
    assert F.dropout(x, 0.3, training=False) is x and F.dropout(x, 0.0, training=True) is x
    y = F.dropout(x, 0.3, training=True)
    kept = y.detach() != 0
    assert torch.allclose(y.detach()[kept], torch.full((int(kept.sum()),), 1 / 0.7))
    assert 0.62 < float(kept.float().mean()) < 0.78 and float(y.detach().mean()) == pytest.approx(1.0, abs=0.06)
    y.sum().backward()
    assert torch.allclose(x.grad[kept], torch.full((int(kept.sum()),), 1 / 0.7)) and float(x.grad[~kept].abs().sum()) == 0
    for bad in (-0.1, 1.0, 1.5):
        with pytest.raises(ValueError):
            F.dropout(x, bad, True)


def test_dropout_module_follows_train_eval_of_its_parent():
    class Net(Module):
        def __init__(self):
            super().__init__()
            self.lin, self.drop = Linear(4, 4, seed=0), Dropout(0.5)

        def submodules(self):
            return [self.lin, self.drop]

        def forward(self, x):
            return self.drop(self.lin(x))
    net = Net()
    x = torch.ones(64, 4)
    net.eval()
    assert not net.drop.training and torch.equal(net(x), net(x))
    net.train()
    assert net.drop.training and net.lin.training
    assert int((net(x) == 0).sum()) > 0
    with pytest.raises(ValueError):
        Dropout(1.0)


def test_clip_grad_norm_cases():
    a, b, c = _param([3.0, 0.0]), _param([0.0, 4.0]), _param([1.0])
    (a * torch.tensor([3.0, 0.0])).sum().backward()
    (b * torch.tensor([0.0, 4.0])).sum().backward()
    assert float(clip_grad_norm([a, b, c], 10.0)) == pytest.approx(5.0)        # no-op below the limit, c skipped
    assert a.grad.tolist() == [3.0, 0.0] and b.grad.tolist() == [0.0, 4.0] and c.grad is None
    assert float(clip_grad_norm([a, b, c], 1.0)) == pytest.approx(5.0)         # returns the norm before scaling
    total = math.sqrt(float((a.grad ** 2).sum() + (b.grad ** 2).sum()))
    assert total == pytest.approx(1.0, rel=1e-6) and a.grad.tolist() == pytest.approx([0.6, 0.0])
    with pytest.raises(ValueError):
        clip_grad_norm([a], 0.0)
    assert float(clip_grad_norm([c], 1.0)) == 0.0


def test_sgd_momentum_survives_a_save_and_resume(tmp_path):
    """SGD keeps its momentum per parameter; the sidecar must carry it (and the step count, because the first SGD
    step overwrites the momentum with the gradient), so that a resumed run equals the uninterrupted one."""
    import dart_pytorch_b200 as dp
    from dart_pytorch_b200.io.dptc import Checkpoint
    from dart_pytorch_b200.io.train_state import load_train_state, save_train_state
    from dart_pytorch_b200.models import GPT, GPTConfig

    def make():
        m = GPT(GPTConfig(vocab_size=29, max_ctx=10, embed_dim=16, num_layers=1, num_heads=2, seed=9))
        return m, dp.SGD(m.parameters(), lr=5e-2, momentum=0.9, weight_decay=0.01)

    def run(m, o, steps, g):
        for _ in range(steps):
            x = torch.randint(0, 29, (2, 10), generator=g)
            o.zero_grad()
            m.loss(x[:, :-1], x[:, 1:]).backward()
            o.step()

    g = torch.Generator().manual_seed(1)
    m1, o1 = make()
    run(m1, o1, 3, g)
    Checkpoint.save_file(m1, str(tmp_path / "s.dptc"))
    save_train_state(str(tmp_path / "s.dpts"), o1)
    gstate = g.get_state()
    run(m1, o1, 3, g)
    m2, o2 = make()
    Checkpoint.load_into_file(m2, str(tmp_path / "s.dptc"))
    load_train_state(str(tmp_path / "s.dpts"), o2, restore_rng=False)
    assert o2._steps == 3 and len(o2._velocity) == len(o2.parameters)
    g2 = torch.Generator()
    g2.set_state(gstate)
    run(m2, o2, 3, g2)
    for a, b in zip(m1.parameters(), m2.parameters()):
        assert torch.allclose(a, b, atol=1e-6)
