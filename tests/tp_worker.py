"""Worker of the multi-GPU tensor-parallel tests (launched by torch.distributed.run, one rank per GPU).

Checks the fused GEMM + all-reduce kernel against an fp32 reference of the un-sharded product for decode-sized and
prefill-sized row counts, with bias and residual, over repeated launches (epochs), on peer loads and -- when the fabric
offers a multicast mapping -- on multimem."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dart_pytorch_b200 import _native  # noqa: E402
from dart_pytorch_b200.parallel.tp import TpComm, reference_row_parallel, shard_range  # noqa: E402


def check_comm(comm, rank, world, tag):
    K, Nn = 1024, comm.width
    lo, hi = shard_range(K, rank, world)
    for trial, M in enumerate((32, 1, 128, 300, 1024)):
        g = torch.Generator(device="cuda").manual_seed(7 + trial)        # same tensors on every rank
        x_full = (torch.randn(M, K, device="cuda", generator=g) * 0.5).bfloat16()
        w_full = (torch.randn(Nn, K, device="cuda", generator=g) * 0.05).bfloat16()
        res = (torch.randn(M, Nn, device="cuda", generator=g)).bfloat16()
        bias = (torch.randn(Nn, device="cuda", generator=g)).bfloat16() if trial % 2 else None
        x, w = x_full[:, lo:hi].contiguous(), w_full[:, lo:hi].contiguous()
        resbuf = comm.buffer(1, M)
        resbuf.copy_(res)
        for rep in range(3):                     # repeated launches exercise the epoch protocol
            out = comm.gemm_allreduce(x, w, 0, residual=resbuf, bias=bias)
        torch.cuda.synchronize()
        _native.raise_on_device_error()
        want = reference_row_parallel(x_full, w_full, residual=res, bias=bias)
        err = (out.float() - want).abs().max().item()
        scale = want.abs().max().item()
        assert err <= 0.02 * scale + 0.05, f"{tag} M={M}: max err {err} (scale {scale})"
        # every rank holds the same bits
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out.contiguous())
        for r in range(world):
            assert torch.equal(gathered[r].view(torch.int16), gathered[0].view(torch.int16)), f"{tag}: rank {r} differs"
    if rank == 0:
        print(f"tp_worker {tag}: fused GEMM + all-reduce matches (nvls={comm.use_nvls})")


def check_sequence_parallel(comm, rank, world, tag):
    """Row-parallel GEMM + reduce-scatter, then (after publishing the shard) all-gather + column-parallel GEMM: the
    pair must equal the un-sharded  (x @ w1^T + res) @ w2^T  with the intermediate rounded to bf16."""
    K1, D, N2 = 1024, comm.width, 768
    lo, hi = shard_range(K1, rank, world)
    n_lo, n_hi = shard_range(N2, rank, world)
    for trial, rows_per_rank in enumerate((128, 256, 512)):
        M = rows_per_rank * world
        g = torch.Generator(device="cuda").manual_seed(100 + trial)
        x_full = (torch.randn(M, K1, device="cuda", generator=g) * 0.5).bfloat16()
        w1 = (torch.randn(D, K1, device="cuda", generator=g) * 0.05).bfloat16()
        res = torch.randn(M, D, device="cuda", generator=g).bfloat16()
        w2 = (torch.randn(N2, D, device="cuda", generator=g) * 0.05).bfloat16()
        bias2 = torch.randn(N2, device="cuda", generator=g).bfloat16()
        x, w1s = x_full[:, lo:hi].contiguous(), w1[:, lo:hi].contiguous()
        w2s, b2s = w2[n_lo:n_hi].contiguous(), bias2[n_lo:n_hi].contiguous()
        res_shard = res[rank * rows_per_rank:(rank + 1) * rows_per_rank].contiguous()
        # both forms of the all-gather GEMM, alternating: peers' shards staged in local memory by copies on a side
        # stream, and read in place by the GEMM kernel's own tile loads
        outs = {True: torch.empty(M, n_hi - n_lo, dtype=torch.bfloat16, device="cuda"),
                False: torch.empty(M, n_hi - n_lo, dtype=torch.bfloat16, device="cuda")}
        for rep in range(4):
            shard = comm.gemm_reduce_scatter(x, w1s, 0, residual=res_shard)
            comm.publish_shard()
            comm.allgather_gemm(0, rows_per_rank, w2s, outs[rep % 2 == 0], bias=b2s, staged=(rep % 2 == 0))
            # the next reduce-scatter overwrites buffer 0: its end barrier orders it after every rank's all-gather
        torch.cuda.synchronize()
        _native.raise_on_device_error()
        mid = reference_row_parallel(x_full, w1, residual=res)
        err = (shard.float() - mid[rank * rows_per_rank:(rank + 1) * rows_per_rank]).abs().max().item()
        assert err <= 0.02 * mid.abs().max().item() + 0.05, f"{tag} reduce-scatter rows/rank={rows_per_rank}: err {err}"
        want = (mid.bfloat16().float() @ w2.float().t() + bias2.float())[:, n_lo:n_hi]
        for staged, out in outs.items():
            err = (out.float() - want).abs().max().item()
            assert err <= 0.03 * want.abs().max().item() + 0.05, \
                f"{tag} all-gather GEMM (staged={staged}) rows/rank={rows_per_rank}: err {err}"
    if rank == 0:
        print(f"tp_worker {tag}: reduce-scatter GEMM and all-gather GEMM match")


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    mode = sys.argv[1] if len(sys.argv) > 1 else "auto"
    comm = TpComm(max_rows=1024, width=512, use_nvls=False if mode == "p2p" else None)
    if mode == "p2p":
        assert not comm.use_nvls
    check_comm(comm, rank, world, mode)
    big = TpComm(max_rows=512 * world, width=512, use_nvls=False if mode == "p2p" else None)
    check_sequence_parallel(big, rank, world, mode)
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print("tp_worker ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
