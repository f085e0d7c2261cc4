"""Headline benchmark: GPT-2 124M training throughput (tokens/s) on N GPUs of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Config (the one the baseline names): 12 layers, d 768, 12 heads, ctx 1024, vocab 50257, weight-tied, learned positions,
micro-batch 16 x 1024 per GPU, bf16 compute with fp32 master weights, AdamW lr 6e-4 wd 0.1, warmup + cosine, clip 1.0,
synthetic uniform tokens, N(0, 0.02) weights.  Weak scaling: per-GPU work is fixed.

Two numbers come out of one run:
  value      device-timed: CUDA events around K steps whose inputs already sit on the device
  e2e.value  the same K steps through ``Trainer.step`` fed from pinned host memory, reading the loss back every step
Both are the max over ranks.  Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "gpt2_124m_train_tokens_per_s"
MODEL = dict(vocab_size=50257, max_ctx=1024, embed_dim=768, num_layers=12, num_heads=12)
MICRO_BATCH, SEQ = 16, 1024


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--batch", type=int, default=MICRO_BATCH)
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, f"/tmp/dptb_clocks_{os.getpid()}.csv"
        self.first_line = 0

    def start(self):
        """Starts sampling if it is not running yet (nvidia-smi needs a few hundred ms before its first line: a caller
        with a short timed region starts it during warm-up and calls ``mark()`` where the region begins)."""
        if self.proc is not None:
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def mark(self):
        """The timed region begins here: only lines written from now on are summarised."""
        self.start()
        try:
            with open(self.path) as f:
                self.first_line = sum(1 for _ in f)
        except OSError:
            self.first_line = 0

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            lines = open(self.path).read().splitlines()
            # the timed window; if it was too short to catch a line, the last samples before it (same load: warm-up)
            window = lines[self.first_line:] or lines[max(0, self.first_line - 3):]
            for line in window:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[3:7]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus: int):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world: int):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def make_batches(n: int, batch: int, seed: int):
    """n synthetic (tokens, targets) batches in pinned host memory (uniform ids, next-token targets)."""
    import torch
    g = torch.Generator().manual_seed(seed)
    xs = torch.randint(0, MODEL["vocab_size"], (n, batch, SEQ + 1), generator=g, dtype=torch.long)
    x = xs[:, :, :-1].contiguous().pin_memory()
    y = xs[:, :, 1:].contiguous().pin_memory()
    return x, y


def run_ours(args):
    import torch
    import dart_pytorch_b200 as dp
    from dart_pytorch_b200 import _native
    from dart_pytorch_b200.nn.transformer import Activation
    from dart_pytorch_b200.utils.trainer import Trainer

    rank, world, local = dist_setup(args.gpus)
    lib = _native.load(required=True)
    lib.dptb_launch_count.restype = ctypes.c_longlong
    cfg = dp.GPTConfig(attn_bias=True, activation=Activation.geluTanh, init_std=0.02, tie_weights=True, seed=0, **MODEL)
    model = dp.GPT(cfg).to("cuda", torch.bfloat16)
    total_steps = max(1000, args.steps + args.warmup)
    opt = dp.Adam(model.parameters(), lr=6e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)
    sched = dp.LinearWarmupCosineDecay(opt, warmup_steps=100, total_steps=total_steps, max_lr=6e-4, min_lr=6e-5)
    reducer = None
    if world > 1:
        from dart_pytorch_b200.parallel.dp import GradReducer
        overlap = os.environ.get("DPTB200_DP_OVERLAP", "1") not in ("0", "false", "False")
        reducer = GradReducer(opt.arena, world, overlap=overlap)
    trainer = Trainer(model, opt, sched, clip_norm=1.0, use_graph=not args.no_graph, reducer=reducer)

    n_batches = args.warmup + 2 * args.steps
    hx, hy = make_batches(n_batches, args.batch, seed=1234 + rank)
    dx, dy = hx.cuda(), hy.cuda()
    tokens_per_step = args.batch * SEQ * world

    # Warm-up (eager steps, then graph capture); the clock sampler is already running, the timed region is marked below.
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(max(args.warmup, 3)):
        loss = trainer.step(dx[i % n_batches], dy[i % n_batches])
    barrier(world)
    first_loss = float(loss)

    # ---- device-timed region: inputs already on the device -------------------------------------------
    launches_before = lib.dptb_launch_count()
    barrier(world)
    if rank == 0:
        sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        j = (args.warmup + i) % n_batches
        loss = trainer.step(dx[j], dy[j])
    e1.record()
    barrier(world)
    dev_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    eager_launches = int(lib.dptb_launch_count() - launches_before)
    dev_ms = max_over_ranks(dev_ms, world)

    # ---- end-to-end region: pinned host inputs in, loss value out, every step -----------------------------
    barrier(world)
    t0 = time.perf_counter()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    last = 0.0
    for i in range(args.steps):
        j = (args.warmup + args.steps + i) % n_batches
        loss = trainer.step(hx[j], hy[j])
        last = float(loss)  # device -> host read of the step's result
    e3.record()
    barrier(world)
    e2e_ms = max(e2.elapsed_time(e3), (time.perf_counter() - t0) * 1e3)
    e2e_ms = max_over_ranks(e2e_ms, world)
    _native.raise_on_device_error()

    # ---- two more device-timed blocks of K steps: the spread shows how much of a small difference is noise ----------
    block_ms = [dev_ms / args.steps]
    for _ in range(2):
        barrier(world)
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for i in range(args.steps):
            j = (args.warmup + i) % n_batches
            trainer.step(dx[j], dy[j])
        b1.record()
        barrier(world)
        block_ms.append(max_over_ranks(b0.elapsed_time(b1), world) / args.steps)

    # ---- library baseline of the same step at the same N (plain PyTorch, CUDA-graphed), for vs_baseline ------------
    baseline = None
    if os.environ.get("DPTB200_BENCH_BASELINE", "1") not in ("0", "false"):
        try:
            from benchmarks.torch_baseline import measure as torch_measure
            baseline = torch_measure(MODEL, SEQ, world, local, args.batch, args.steps, args.warmup, hx, hy, dx, dy,
                                     max_over_ranks, barrier, use_graph=True)
        except Exception as e:      # the baseline must never take the primary number down with it
            baseline = {"error": repr(e)[:200]}

    # ---- second half of the metric: Llama-3-8B-shaped tensor-parallel decode on the same N GPUs -------------------
    secondary = None
    if world >= 2 and os.environ.get("DPTB200_BENCH_SECONDARY", "1") not in ("0", "false"):
        try:
            from benchmarks.tp_decode_bench import measure as tp_measure
            layers = max(1, 32 * world // 8)     # the full 32 layers at TP = 8; proportionally fewer on smaller groups
            r = tp_measure("ours", layers, 32, 2048, 256, prefill_modes=("ar", "sp"))
            secondary = {"metric": "llama8b_tp8_decode_tokens_per_s" if world == 8 else
                         f"llama8b_shaped_{layers}layer_tp{world}_decode_tokens_per_s",
                         "value": r["value"], "unit": "tokens/s", "ttft_ms_p50": r["ttft_ms_p50"],
                         "ttft_ms_p50_by_prefill_mode": r["ttft_ms_p50_by_prefill_mode"],
                         "decode_ms_per_step": r["decode_ms_per_step"], "config": r["config"], "nvls": r.get("nvls")}
        except Exception as e:
            secondary = {"error": repr(e)[:200]}

    if rank == 0:
        kernels = trainer.kernels_per_step * args.steps if trainer.kernels_per_step else eager_launches
        value = tokens_per_step * args.steps / (dev_ms / 1e3)
        e2e = tokens_per_step * args.steps / (e2e_ms / 1e3)
        base_value = None
        if baseline and "ms_per_step" in baseline:
            base_value = tokens_per_step / (baseline["ms_per_step"] / 1e3)
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / base_value) if base_value else None, "dtype": "bf16", "data": "synthetic",
            "impl": "ours",
            "config": {"model": "gpt2-124m", "global_batch": args.batch * world, "seq_len": SEQ,
                       "parallelism": f"dp{world}", "optimizer": "adamw lr6e-4 wd0.1 clip1.0 warmup-cosine",
                       "cache_policy": "per-step working set (>2 GB of activations and logits) exceeds the 126 MB L2",
                       "cuda_graph": trainer._graph is not None,
                       "grad_reduce_overlap": bool(reducer is not None and getattr(reducer, "overlap", False)),
                       "grad_reduce": "none" if reducer is None else
                       (reducer.mode + ("+multimem" if getattr(reducer.impl, "use_nvls", False) else ""))},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": int(hx[0].numel() * 8 + hy[0].numel() * 8), "d2h_bytes_per_step": 4},
            "gpu_launches": int(kernels),
            "loss_first": first_loss, "loss_last": last,
            "ms_per_step_blocks": block_ms, "ms_per_step_median_of_blocks": statistics.median(block_ms),
            # what vs_baseline divides by: the same model and step in plain PyTorch (cuBLAS + SDPA + fused AdamW +
            # clip_grad_norm_ + DDP over NCCL), captured in a CUDA graph like this package's step, timed in this run
            "baseline": None if baseline is None else dict(
                baseline, impl="torch", value=base_value,
                e2e_value=(tokens_per_step / (baseline["e2e_ms_per_step"] / 1e3)) if "e2e_ms_per_step" in baseline else None),
            "secondary": secondary,
        }
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def run_torch(args):
    """Plain PyTorch (cuBLAS + SDPA + fused AdamW, DDP over NCCL) arm of the same model: the library baseline."""
    from benchmarks.torch_baseline import run
    run(args, METRIC, MODEL, SEQ, ClockSampler, dist_setup, max_over_ranks, barrier, make_batches)


def run_reference(args):
    from baseline.reference_arm import run
    run(args, METRIC, MODEL, SEQ, ClockSampler)


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    elif a.impl == "torch":
        run_torch(a)
    else:
        run_ours(a)
