"""Library baseline for the headline benchmark: the same GPT-2 124M training step written in plain PyTorch
(cuBLAS GEMMs, SDPA attention, fused AdamW, ``clip_grad_norm_``, DDP over NCCL for N > 1).  It is the number the
hand-written kernels are compared against; none of this package's kernels run here."""
from __future__ import annotations

import json
import math
import os
import time

import torch
import torch.nn as nn
import torch.nn.functional as F


class Block(nn.Module):
    def __init__(self, d, h):
        super().__init__()
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.fc, self.fc2 = nn.Linear(d, 4 * d), nn.Linear(4 * d, d)
        self.h = h

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).split(d, dim=2)
        q, k, v = (t.view(b, s, self.h, d // self.h).transpose(1, 2) for t in (q, k, v))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(b, s, d)
        x = x + self.proj(a)
        return x + self.fc2(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


class TorchGPT(nn.Module):
    def __init__(self, vocab_size, max_ctx, embed_dim, num_layers, num_heads):
        super().__init__()
        self.wte, self.wpe = nn.Embedding(vocab_size, embed_dim), nn.Embedding(max_ctx, embed_dim)
        self.blocks = nn.ModuleList(Block(embed_dim, num_heads) for _ in range(num_layers))
        self.lnf = nn.LayerNorm(embed_dim)
        self.apply(lambda m: nn.init.normal_(m.weight, std=0.02) if isinstance(m, (nn.Linear, nn.Embedding)) else None)

    def forward(self, x, y):
        h = self.wte(x) + self.wpe(torch.arange(x.shape[1], device=x.device))
        for blk in self.blocks:
            h = blk(h)
        logits = F.linear(self.lnf(h), self.wte.weight)
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), y.reshape(-1))


def run(args, metric, model_cfg, seq, ClockSampler, dist_setup, max_over_ranks, barrier, make_batches):
    rank, world, local = dist_setup(args.gpus)
    torch.backends.cuda.matmul.allow_tf32 = True
    model = TorchGPT(**model_cfg).cuda()
    ddp = model
    if world > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP
        ddp = DDP(model, device_ids=[local], gradient_as_bucket_view=True)
    opt = torch.optim.AdamW(model.parameters(), lr=6e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    n_batches = args.warmup + 2 * args.steps
    hx, hy = make_batches(n_batches, args.batch, seed=1234 + rank)
    dx, dy = hx.cuda(), hy.cuda()

    def step(x, y):
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = ddp(x, y)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        return loss

    for i in range(max(args.warmup, 3)):
        loss = step(dx[i % n_batches], dy[i % n_batches])
    barrier(world)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        j = (args.warmup + i) % n_batches
        loss = step(dx[j], dy[j])
    e1.record()
    barrier(world)
    dev_ms = max_over_ranks(e0.elapsed_time(e1), world)
    clocks = sampler.stop() if rank == 0 else None
    barrier(world)
    t0 = time.perf_counter()
    last = 0.0
    for i in range(args.steps):
        j = (args.warmup + args.steps + i) % n_batches
        loss = step(hx[j].cuda(non_blocking=True), hy[j].cuda(non_blocking=True))
        last = float(loss)
    barrier(world)
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3, world)
    if rank == 0:
        toks = args.batch * seq * world * args.steps
        print(json.dumps({
            "metric": metric, "value": toks / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "torch",
            "config": {"model": "gpt2-124m", "global_batch": args.batch * world, "seq_len": seq,
                       "parallelism": f"dp{world}", "stack": "torch autocast bf16 + cuBLAS + SDPA + fused AdamW + DDP"},
            "clocks": clocks,
            "e2e": {"value": toks / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": int(hx[0].numel() * 16), "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "loss_last": last}))
    if world > 1:
        torch.distributed.destroy_process_group()
