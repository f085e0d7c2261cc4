"""Worker of the multi-GPU data-parallel tests (launched by torch.distributed.run, one rank per GPU).

Checks the fused all-reduce kernel (peer loads / stores, and multimem when the fabric offers it) against a plain
fp32 average of the same gradients and against the norm of that average; then trains a small GPT for a few steps
under the Trainer on every rank and checks that replicas stay identical."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dart_pytorch_b200 as dp  # noqa: E402
from dart_pytorch_b200 import _native  # noqa: E402
from dart_pytorch_b200.nn.transformer import Activation  # noqa: E402
from dart_pytorch_b200.parallel.dp import GradReducer  # noqa: E402
from dart_pytorch_b200.utils.trainer import Trainer  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    mode = sys.argv[1] if len(sys.argv) > 1 else "auto"
    if mode == "p2p":
        os.environ["DPTB200_DP_NVLS"] = "0"
    cfg = dp.GPTConfig(vocab_size=512, max_ctx=128, embed_dim=128, num_layers=2, num_heads=2, attn_bias=True,
                       activation=Activation.geluTanh, init_std=0.02, seed=5)
    model = dp.GPT(cfg).to("cuda", torch.bfloat16)
    opt = dp.Adam(model.parameters(), lr=1e-3, weight_decay=0.1)
    red = GradReducer(opt.arena, world, mode="fused", bucket_mb=0.25, overlap=(mode == "overlap"))
    assert red.mode == "fused"
    arena = opt.arena
    # 1. raw reduction against an fp32 reference
    for trial in range(3):
        g = torch.Generator(device="cuda").manual_seed(100 * trial + rank)
        local_grad = (torch.randn(arena.numel, device="cuda", generator=g) * 0.01).bfloat16()
        arena.grad.copy_(local_grad)
        ref = local_grad.float()
        dist.all_reduce(ref)
        ref = (ref / world)
        ctrl = torch.zeros(4, device="cuda")
        torch.cuda.synchronize()
        dist.barrier()
        handled = red.reduce(ctrl, 1.0)
        torch.cuda.synchronize()
        _native.raise_on_device_error()
        assert handled
        got = arena.grad.float()
        err = float((got - ref).norm() / ref.norm())
        assert err < 5e-3, err
        want_norm = float(got.norm())
        assert abs(float(ctrl[0]) - want_norm) / want_norm < 1e-3, (float(ctrl[0]), want_norm)
        assert abs(float(ctrl[1]) - min(1.0, 1.0 / want_norm)) < 1e-3
        # every rank holds the same bits
        mine = arena.grad.clone()
        other = mine.clone()
        dist.broadcast(other, 0)
        assert torch.equal(mine.view(torch.int16), other.view(torch.int16))
    # 1b. one rank reaches the reduction late (its host was busy for longer than a pipeline wait lasts): the others
    #     wait for it inside the kernel, up to the reducer's skew limit, and the result is still the exact average
    if mode == "late":
        import time
        g = torch.Generator(device="cuda").manual_seed(900 + rank)
        local_grad = (torch.randn(arena.numel, device="cuda", generator=g) * 0.01).bfloat16()
        arena.grad.copy_(local_grad)
        ref = local_grad.float()
        dist.all_reduce(ref)
        ref = ref / world
        torch.cuda.synchronize()
        dist.barrier()
        if rank == world - 1:
            time.sleep(1.6)
        ctrl = torch.zeros(4, device="cuda")
        red.reduce(ctrl, 1.0)
        torch.cuda.synchronize()
        _native.raise_on_device_error()
        assert float(ctrl[2]) == 1.0
        assert float((arena.grad.float() - ref).norm() / ref.norm()) < 5e-3
    # 2. a few training steps: replicas must stay bit-identical
    trainer = Trainer(model, opt, None, clip_norm=1.0, reducer=red, use_graph=(mode != "nograph"))
    gen = torch.Generator().manual_seed(7 + rank)
    losses = []
    x = torch.randint(0, 512, (4, 128), generator=gen).cuda()   # one fixed batch per rank (ranks differ)
    y = torch.roll(x, -1, 1)
    for step in range(8):
        losses.append(float(trainer.step(x, y)))
    torch.cuda.synchronize()
    _native.raise_on_device_error()
    w = arena.flat.clone()
    w0 = w.clone()
    dist.broadcast(w0, 0)
    assert torch.equal(w.view(torch.int16), w0.view(torch.int16)), "replicas diverged"
    assert losses[-1] < losses[0]
    if rank == 0:
        print(f"dp_worker ok mode={mode} nvls={red.impl.use_nvls} losses={losses[0]:.3f}->{losses[-1]:.3f}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
