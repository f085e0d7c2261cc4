"""Tracing ranges and guarded (canary-padded) buffers on CPU."""
import torch

from dart_pytorch_b200.utils import guard, trace


def test_phase_timer_collects_nested_ranges_and_restores_itself():
    assert trace._timer is None
    with trace.PhaseTimer() as t:
        with trace.range("outer"):
            with trace.range("inner"):
                torch.randn(64, 64) @ torch.randn(64, 64)
        with trace.range("outer"):
            pass
    assert trace._timer is None
    s = t.summary()
    assert s["outer"][0] == 2 and s["inner"][0] == 1
    assert s["outer"][1] >= s["inner"][1] >= 0.0
    with trace.range("free"):          # no timer installed, NVTX off (or no CUDA): nothing happens
        pass


def test_trainer_step_emits_the_phase_ranges():
    import dart_pytorch_b200 as dp
    from dart_pytorch_b200.utils.trainer import Trainer
    model = dp.GPT(dp.GPTConfig(vocab_size=31, max_ctx=16, embed_dim=16, num_layers=1, num_heads=2, seed=1))
    opt = dp.Adam(model.parameters(), lr=1e-3)
    tr = Trainer(model, opt, None, clip_norm=1.0, use_graph=False)
    x = torch.randint(0, 31, (2, 16))
    with trace.PhaseTimer() as t:
        tr.step(x, torch.roll(x, -1, 1))
    names = set(t.summary())
    assert {"step/forward", "step/backward", "step/clip", "step/optimizer"} <= names


def test_guarded_buffer_detects_writes_outside_the_payload():
    g = guard.GuardedBuffer((5, 7), torch.float32, "cpu", pad_elems=16)
    assert g.tensor.shape == (5, 7) and g.tensor.is_contiguous()
    g.tensor.fill_(3.0)
    g.check()                                  # payload writes leave the canaries alone
    flat = g.storage
    flat[g.pad_elems - 1] = 0.0                # one element before the payload
    try:
        g.check("under-run")
    except guard.GuardError as e:
        assert "before" in str(e) and "under-run" in str(e)
    else:
        raise AssertionError("under-run not detected")
    g.rearm()
    flat[g.pad_elems + 35] = 1.0               # one element after the payload
    try:
        g.check()
    except guard.GuardError as e:
        assert "after" in str(e)
    else:
        raise AssertionError("over-run not detected")


def test_guarded_context_checks_every_buffer_on_exit():
    with guard.guarded() as pool:
        a = pool.empty((4, 4), torch.float32, "cpu")
        b = pool.empty((3,), torch.int32, "cpu")
        a.zero_()
        b.fill_(7)
    assert pool.checked == 2
