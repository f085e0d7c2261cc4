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


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    mode = sys.argv[1] if len(sys.argv) > 1 else "auto"
    comm = TpComm(max_rows=1024, width=512, use_nvls=False if mode == "p2p" else None)
    if mode == "p2p":
        assert not comm.use_nvls
    check_comm(comm, rank, world, mode)
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print("tp_worker ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
