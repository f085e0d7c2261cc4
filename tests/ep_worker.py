"""Worker of the expert-parallel MoE test (launched by torch.distributed.run, one rank per GPU): the sharded layer's
output, input gradient, router gradient and expert weight gradients are compared with a plain fp32 restatement that
holds every expert and applies the same routing and per-source capacity rule."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dart_pytorch_b200 import _native  # noqa: E402
from dart_pytorch_b200.parallel.ep import ExpertParallelMoE, capacity  # noqa: E402


def reference(x, gate, wgu, wd, k, C, coef):
    """fp32: x [T, D]; gate [E, D]; wgu[e] [2H, D]; wd[e] [D, H]."""
    T, E = x.shape[0], gate.shape[0]
    # The layer's router GEMM writes bf16 logits; the choice of experts is made on those.  The reference rounds its fp32
    # logits the same way (straight-through for the gradient), so that a near-tie between two experts cannot route a
    # token differently on the two sides (with 16 experts such near-ties do occur among a few thousand tokens).
    logits = x @ gate.t()
    logits = logits + (logits.bfloat16().float() - logits).detach()
    probs = torch.softmax(logits, -1)
    w, idx = torch.topk(probs, k, dim=-1)                 # ties: lowest index first (as the kernel)
    y = torch.zeros_like(x)
    seen = [0] * E
    keep = torch.zeros(T, k, dtype=torch.bool)
    idx_l = idx.tolist()
    for t in range(T):
        for j in range(k):
            e = idx_l[t][j]
            if seen[e] < C:
                keep[t, j] = True
            seen[e] += 1
    for e in range(E):
        sel = (idx == e) & keep.to(idx.device)
        rows = sel.any(1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        xe = x[rows]
        gu = xe @ wgu[e].t()
        H = wgu[e].shape[0] // 2
        h = torch.nn.functional.silu(gu[:, :H]) * gu[:, H:]
        oe = h @ wd[e].t()
        we = (w * sel.float())[rows].sum(1, keepdim=True)
        y = y.index_add(0, rows, we * oe)
    f = torch.bincount(idx.reshape(-1), minlength=E).float() / float(T * k)
    aux = coef * E * (f * probs.mean(0)).sum()
    return y, aux


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    D, H, E, k, T = 64, 128, int(os.environ.get("DPTB200_EP_TEST_EXPERTS", 2 * world)), 2, 96
    cf = float(sys.argv[1]) if len(sys.argv) > 1 else 1.25
    moe = ExpertParallelMoE(D, H, E, top_k=k, capacity_factor=cf, aux_loss_coef=0.01, device="cuda", seed=5,
                            dtype=torch.bfloat16)
    C = capacity(T, k, E, cf)
    # every rank gathers all expert weights for the reference
    def gather(params):
        out = []
        for p in params:
            parts = [torch.empty_like(p.data) for _ in range(world)]
            dist.all_gather(parts, p.data.contiguous())
            out.append(parts)
        return out
    gu_all = gather(moe.w_gate_up)      # [le][rank]
    d_all = gather(moe.w_down)
    wgu = [gu_all[e % moe.El][e // moe.El].float() for e in range(E)]
    wd = [d_all[e % moe.El][e // moe.El].float() for e in range(E)]
    for trial in range(2):
        g = torch.Generator(device="cuda").manual_seed(100 * trial + rank)
        x = (torch.randn(T, D, device="cuda", generator=g)).bfloat16().requires_grad_(True)
        dy = torch.randn(T, D, device="cuda", generator=g).bfloat16()
        for p in moe.parameters():
            p.grad = None
        y = moe(x)
        (y.float() * dy.float()).sum().backward(retain_graph=False) if False else None
        loss = (y.float() * dy.float()).sum() + moe.aux_loss
        loss.backward()
        # reference on this rank's tokens with all experts (fp32, leaf copies)
        xr = x.detach().float().requires_grad_(True)
        gate_r = moe.gate.detach().float().requires_grad_(True)
        wgu_r = [t.clone().requires_grad_(True) for t in wgu]
        wd_r = [t.clone().requires_grad_(True) for t in wd]
        yr, aux_r = reference(xr, gate_r, wgu_r, wd_r, k, C, 0.01)
        ((yr * dy.float()).sum() + aux_r).backward()
        def close(a, b, tag, tol=0.05):
            err = (a.float() - b.float()).abs().max().item()
            scale = b.float().abs().max().item()
            assert err <= tol * scale + 2e-3, f"rank {rank} trial {trial} {tag}: err {err} scale {scale}"
        close(y, yr, "y")
        close(x.grad, xr.grad, "dx")
        close(moe.gate.grad, gate_r.grad, "dgate", tol=0.08)
        # expert weight gradients: contributions of ALL ranks' tokens reach the owner; sum the references
        totals = {}
        for name, ref_list in (("gu", wgu_r), ("d", wd_r)):
            for e2 in range(E):
                gsum = ref_list[e2].grad.clone() if ref_list[e2].grad is not None else torch.zeros_like(ref_list[e2])
                dist.all_reduce(gsum, op=dist.ReduceOp.SUM)
                totals[(name, e2)] = gsum
        for le in range(moe.El):
            ge = rank * moe.El + le
            close(moe.w_gate_up[le].grad, totals[("gu", ge)], f"dWgu expert {ge}", tol=0.08)
            close(moe.w_down[le].grad, totals[("d", ge)], f"dWd expert {ge}", tol=0.08)
        assert abs(float(moe.aux_loss) - float(aux_r)) < 1e-3
    torch.cuda.synchronize()
    _native.raise_on_device_error()
    dist.barrier()
    if rank == 0:
        print(f"ep_worker ok (cf={cf}, dropped={moe.last_dropped})")
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except Exception as e:  # one line the launcher's summary cannot bury
        print(f"EP_WORKER_FAIL rank {os.environ.get('RANK')}: {e!r}", flush=True)
        raise
