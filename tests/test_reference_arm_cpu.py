"""The reference arm of the benchmark restates the reference's Dart tensor / autograd / nn layers over the C ABI of its
native library.  Here the same graph runs on the NumPy stand-in of that ABI and is checked against torch autograd:
loss, every gradient, and the parameters after clip + AdamW steps, with the batch in one pass and split in two."""
import math

import numpy as np
import pytest
import torch

from baseline import reference_arm as ra

CFG = dict(vocab_size=37, max_ctx=8, embed_dim=16, num_layers=2, num_heads=2)


def torch_params(state):
    return [torch.tensor(p.to_host().reshape(p.shape), dtype=torch.float64, requires_grad=True) for p in state.params]


def torch_loss(ps, x, y, cfg):
    """The same model in torch, reading parameters in the arm's order (wte, wpe, per block: ln1, ln2, per-head q/k/v
    Linear pairs, wo, ffn1, ffn2; final norm)."""
    it = iter(ps)
    wte, wpe = next(it), next(it)
    D, H = cfg["embed_dim"], cfg["num_heads"]
    hd = D // H
    B, S = x.shape
    h = wte[x] + wpe[torch.arange(S)]
    mask = torch.triu(torch.full((S, S), -1e9, dtype=torch.float64), diagonal=1)
    for _ in range(cfg["num_layers"]):
        g1, b1, g2, b2 = next(it), next(it), next(it), next(it)
        proj = [[(next(it), next(it)) for _ in range(H)] for _ in range(3)]
        wo, bo, w1, bb1, w2, bb2 = (next(it) for _ in range(6))
        a = torch.nn.functional.layer_norm(h, (D,), g1, b1, 1e-5)
        heads = []
        for i in range(H):
            q = a @ proj[0][i][0].T + proj[0][i][1]
            k = a @ proj[1][i][0].T + proj[1][i][1]
            v = a @ proj[2][i][0].T + proj[2][i][1]
            sc = q @ k.transpose(1, 2) / math.sqrt(hd) + mask
            heads.append(torch.softmax(sc, -1) @ v)
        h = h + torch.cat(heads, -1) @ wo.T + bo
        f = torch.nn.functional.layer_norm(h, (D,), g2, b2, 1e-5) @ w1.T + bb1
        f = 0.5 * f * (1 + torch.tanh(0.7978845608028654 * (f + 0.044715 * f ** 3)))
        h = h + f @ w2.T + bb2
    gf, bf = next(it), next(it)
    logits = torch.nn.functional.layer_norm(h, (D,), gf, bf, 1e-5) @ wte.T
    return torch.nn.functional.cross_entropy(logits.reshape(B * S, -1), y.reshape(-1))


@pytest.mark.parametrize("micro", [4, 2])
def test_composed_step_matches_torch(micro):
    rt = ra.Runtime(ra.NumpyEngine())
    st = ra.TrainState(rt, CFG, lr=1e-2, weight_decay=0.1, warmup=2, total=10)
    ps = torch_params(st)
    opt = torch.optim.AdamW(ps, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    rng = np.random.default_rng(0)
    for step in range(3):
        x = rng.integers(0, CFG["vocab_size"], (4, 8))
        y = rng.integers(0, CFG["vocab_size"], (4, 8))
        for g in opt.param_groups:
            g["lr"] = ra.lr_at(step + 1, 2, 10, 1e-2, 1e-3)
        opt.zero_grad()
        ref = torch_loss(ps, torch.tensor(x), torch.tensor(y), CFG)
        ref.backward()
        torch.nn.utils.clip_grad_norm_(ps, 1.0)
        opt.step()
        loss = st.step(x, y, micro)
        assert abs(loss - float(ref.detach())) < 1e-4
        for p, q in zip(st.params, ps):
            np.testing.assert_allclose(p.to_host().reshape(p.shape), q.detach().numpy().reshape(p.shape),
                                       rtol=2e-3, atol=2e-5)
    # every intermediate was released: only parameters, their gradients and the Adam moments stay allocated
    n_param = sum(p.length for p in st.params)
    assert rt.live == 8 * 4 * n_param
    assert len(rt.e.t) == 4 * len(st.params)


def test_planner_predicts_the_peak():
    """The affine extrapolation over layers and micro-batch reproduces a direct dry run."""
    cfg = dict(CFG, num_layers=3)
    micro, predicted = ra.plan_micro_batch(cfg, 4, 8, 1e18)
    assert micro == 4
    rt = ra.Runtime(ra.ShapeEngine())
    st = ra.TrainState(rt, cfg)
    tok = np.zeros((4, 8), dtype=np.int64)
    st.step(tok, tok, 4)
    assert abs(predicted[4] - rt.peak) <= 0.02 * rt.peak
    small, _ = ra.plan_micro_batch(cfg, 4, 8, predicted[2] * 1.01)
    assert small == 2


def test_unavailable_for_several_gpus(capsys):
    class A:
        gpus, steps, warmup, batch = 2, 1, 1, 16
    ra.run(A, "m", CFG, 8)
    assert "no multi-GPU path" in capsys.readouterr().out
