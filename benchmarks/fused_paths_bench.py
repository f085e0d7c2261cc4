"""Roofline report of the fused compute + collective paths, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29610 \\
        benchmarks/fused_paths_bench.py [--json out.json]

Every path is one kernel of this package that does its arithmetic and moves its data over NVLink peer memory itself:

  P1   data-parallel gradient all-reduce (+ sum of squares for the clip), per bucket     csrc/dp_allreduce.cu
  P2a  row-parallel GEMM + all-reduce / + reduce-scatter (prefill and decode rows)        csrc/gemm.cu, gemm_skinny.cu
  P2b  all-gather + column-parallel GEMM (shards staged by copies / read in place)        parallel/tp.py, csrc/gemm.cu
  P3   expert-parallel MoE layer forward: route, dispatch, expert SwiGLU GEMMs, combine   csrc/moe_ep.cu

Each is timed with CUDA events on the launching stream after warm-up, a barrier and a synchronise on both sides, and
the maximum over the ranks is reported.  The roofline of a path is the slower of its FLOPs at the measured sustained
bf16 GEMM rate and the bytes that must cross this GPU's NVLink port (the busier direction) at the link bandwidth; the
link bandwidth is measured first with this package's own copy kernel reading a peer's buffer.  Fractions are
roofline time / achieved time.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks():
    """(sustained bf16 FLOP/s, nominal-measured NVLink bytes/s per direction) with the documented fallbacks."""
    tf, link = 1393e12, 770e9
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            tf = float(json.load(f).get("bf16_tflops_sustained", 1393.0)) * 1e12
    except (OSError, ValueError):
        pass
    return tf, link


def timed(fn, group, iters=10, warmup=3):
    """Median device time of ``fn`` in ms, max over ranks."""
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        dist.barrier(group=group)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default="")
    ap.add_argument("--only", default="", help="comma-separated: link,p1,p2a,p2b,p3")
    args = ap.parse_args()
    rank, local = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    group = dist.group.WORLD
    world = dist.get_world_size()
    want = [w for w in args.only.split(",") if w]
    on = lambda name: not want or name in want  # noqa: E731
    import torch.distributed._symmetric_memory as symm_mem
    from dart_pytorch_b200 import _native
    from dart_pytorch_b200.ops import kernels as K
    from dart_pytorch_b200.parallel.tp import TpComm, shard_range
    tf_peak, link_nominal = peaks()
    rows = []
    bf = dict(device="cuda", dtype=torch.bfloat16)

    def add(path, case, ms, flops, link_bytes, link_bw, note=""):
        t_c, t_l = flops / tf_peak * 1e3, link_bytes / link_bw * 1e3
        roof = max(t_c, t_l)
        rows.append({"path": path, "case": case, "n_gpus": world, "ms": ms, "roofline_ms": roof,
                     "fraction": roof / ms if ms > 0 else None, "bound": "compute" if t_c >= t_l else "nvlink",
                     "tflops": flops / ms / 1e9 if ms > 0 else 0.0, "link_gbs": link_bytes / ms / 1e6 if ms > 0 else 0.0,
                     "note": note})

    # ---- NVLink bandwidth seen by this package's own copy kernel (peer loads, one direction) ------------------------
    link_bw = link_nominal
    if world > 1 and on("link"):
        n = 256 * 1024 * 1024 // 2
        src = symm_mem.empty(n, **bf)
        src.normal_()
        h = symm_mem.rendezvous(src, group=group.group_name)
        peer = h.get_buffer((rank + 1) % world, (n,), torch.bfloat16)
        dst = torch.empty(n, **bf)
        ms = timed(lambda: K.copy_flat(peer, dst), group)
        link_bw = 2 * n / (ms / 1e3)
        rows.append({"path": "link", "case": "copy kernel reading 256 MiB from the next rank", "n_gpus": world, "ms": ms,
                     "link_gbs": link_bw / 1e9, "note": "denominator of the NVLink-bound rows below"})
        del src, dst, peer, h

    # ---- P1: gradient all-reduce per bucket --------------------------------------------------------------------------
    if world > 1 and on("p1"):
        from dart_pytorch_b200.parallel.dp_fused import FusedGradReducer

        class Flat:        # what the reducer needs of a parameter arena: one flat bf16 gradient buffer
            def __init__(self, numel):
                self.numel, self.device, self.params, self.offsets = numel, torch.device("cuda", local), [], {}
                self.grad = torch.zeros(numel, **bf)
        for mb in (32, 77):
            n = mb * 1024 * 1024 // 2
            arena = Flat(n)
            red = FusedGradReducer(arena, world, [(0, n)], group)
            arena.grad.normal_()
            ctrl = torch.zeros(4, device="cuda")

            def run():
                red.reduce_bucket(0, exposed=True)
                red.finalize(ctrl, 1.0)
            ms = timed(run, group)
            B = 2 * n
            # multimem: the switch reads every member's copy of a slice, the requester's own included, so a port sends
            # the whole bucket out while its reduced slice (1/N) comes in, and the broadcast is the mirror image:
            # (1 + 1/N) buckets per direction (the N / (N + 1) bus-bandwidth factor of in-switch all-reduce);
            # peer loads / stores: 2 (N-1)/N buckets per direction
            link_bytes = B * (1.0 + 1.0 / world) if red.use_nvls else 2.0 * B * (world - 1) / world
            add("P1", f"dp_allreduce bucket {mb} MiB ({'multimem' if red.use_nvls else 'peer ld/st'})", ms, 0.0,
                link_bytes, link_bw)
            del red, arena
        _native.raise_on_device_error()

    # ---- P2a / P2b: tensor-parallel GEMMs at the Llama-3-8B shapes ------------------------------------------------------
    if world > 1 and (on("p2a") or on("p2b")):
        D, FF = 4096, 14336
        M = 8192
        comm = TpComm(max_rows=M, width=D, group=group, num_bufs=3)
        g = torch.Generator(device="cuda").manual_seed(5)
        for name, Kfull in (("wo", D), ("down", FF)):
            if Kfull % world:
                continue
            Kr = Kfull // world
            x = (torch.randn(M, Kr, device="cuda", generator=g) * 0.5).bfloat16()
            w = (torch.randn(D, Kr, device="cuda", generator=g) * 0.02).bfloat16()
            res = comm.buffer(1, M)
            res.normal_()
            out_bytes = 2.0 * M * D
            flops = 2.0 * M * D * Kr
            if on("p2a"):
                # through the switch (multimem) a port carries (1 + 1/N) outputs per direction for the all-reduce and one
                # output for the reduce-scatter (every member's partial is read, the owner's included); over peer
                # pointers (N-1)/N of an output per phase
                nv = bool(comm.use_nvls)
                ar_bytes = out_bytes * (1.0 + 1.0 / world) if nv else 2.0 * out_bytes * (world - 1) / world
                rs_bytes = out_bytes if nv else out_bytes * (world - 1) / world
                ms = timed(lambda: comm.gemm_allreduce(x, w, 0, residual=res), group)
                add("P2a", f"GEMM + all-reduce, prefill {name}: [{M},{Kr}] x [{D},{Kr}]^T", ms, flops, ar_bytes, link_bw,
                    "owner reduces the partial tile through the switch, broadcasts the sum")
                if M % (world * 128) == 0:
                    rs_res = comm.buffer(2, M // world)
                    rs_res.normal_()
                    ms = timed(lambda: comm.gemm_reduce_scatter(x, w, 0, residual=rs_res), group)
                    add("P2a", f"GEMM + reduce-scatter, prefill {name}: [{M},{Kr}] x [{D},{Kr}]^T", ms, flops,
                        rs_bytes, link_bw)
                xs, ress = x[:32].contiguous(), comm.buffer(1, 32)
                ms = timed(lambda: comm.gemm_allreduce(xs, w, 0, residual=ress), group, iters=20)
                # decode rows: the floor is streaming this rank's weight slice from HBM, not NVLink
                hbm = 6551e9
                rows.append({"path": "P2a", "case": f"GEMM + all-reduce, decode {name}: [32,{Kr}] x [{D},{Kr}]^T",
                             "n_gpus": world, "ms": ms, "roofline_ms": 2.0 * D * Kr / hbm * 1e3,
                             "fraction": (2.0 * D * Kr / hbm * 1e3) / ms, "bound": "hbm (weight streaming)",
                             "tflops": 2.0 * 32 * D * Kr / ms / 1e9, "link_gbs": 2.0 * 32 * D * 4 / ms / 1e6,
                             "note": "latency chain: launch, first tile copy, split fold, one NVLink hop"})
        if on("p2b") and M % (world * 128) == 0:
            rows_per = M // world
            for name, Nfull in (("qkv", 6144), ("gate_up", 2 * FF)):
                if Nfull % world:
                    continue
                Nn = Nfull // world
                w = (torch.randn(Nn, D, device="cuda", generator=g) * 0.02).bfloat16()
                out = torch.empty(M, Nn, **bf)
                comm.buffer(1, rows_per).normal_()

                for staged in (True, False):
                    def run():
                        comm.publish_shard()
                        comm.allgather_gemm(1, rows_per, w, out, staged=staged)
                    ms = timed(run, group)
                    how = ("peer shards copied once into local memory on a side stream, GEMM per shard" if staged else
                           "one kernel: peers' row shards read in place by the GEMM's tile loads")
                    add("P2b", f"all-gather + GEMM {name} ({'staged' if staged else 'in place'}): [{M},{D}] (sharded by "
                        f"rows) x [{Nn},{D}]^T", ms, 2.0 * M * D * Nn, 2.0 * M * D * (world - 1) / world, link_bw, how)
        _native.raise_on_device_error()
        del comm

    # ---- P3: expert-parallel MoE layer (forward) ---------------------------------------------------------------------
    if world > 1 and on("p3") and 8 % world == 0:
        from dart_pytorch_b200.parallel.ep import ExpertParallelMoE
        T, d, ffn, E, k = 16384, 1024, 4096, 8, 2
        moe = ExpertParallelMoE(d, ffn, E, top_k=k, capacity_factor=1.25, group=group, device="cuda",
                                dtype=torch.bfloat16, init_std=0.02)
        x = torch.randn(T, d, **bf)

        def run():
            with torch.no_grad():
                moe(x)
        ms = timed(run, group, iters=5)
        flops = 2.0 * T * k * (3 * d * ffn)                 # routed pairs, gate + up + down projections
        link_bytes = 2.0 * (2.0 * T * k * d) * (world - 1) / world   # dispatch and return, bf16 rows
        add("P3", f"MoE layer forward: {T} tokens/GPU, d {d}, {E} experts (ffn {ffn}), top-{k}, capacity 1.25", ms,
            flops, link_bytes, link_bw, "route + slots + peer-store dispatch + expert GEMMs + return + combine")
        _native.raise_on_device_error()

    if rank == 0:
        print("| path | case | GPUs | ms | roofline ms | fraction | bound | TFLOP/s | link GB/s |")
        print("|---|---|---|---|---|---|---|---|---|")
        for r in rows:
            print(f"| {r['path']} | {r['case']} | {r['n_gpus']} | {r['ms']:.3f} | {r.get('roofline_ms', 0):.3f} | "
                  f"{(r.get('fraction') or 0):.2f} | {r.get('bound', '')} | {r.get('tflops', 0):.0f} | "
                  f"{r.get('link_gbs', 0):.0f} |")
        if args.json:
            with open(args.json, "w") as f:
                json.dump(rows, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
