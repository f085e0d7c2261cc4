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


class TorchTrainer:
    """The library training step, eager or captured in a CUDA graph (whole step: forward, backward, DDP all-reduce,
    ``clip_grad_norm_``, fused capturable AdamW), so that the comparison with this package's graph-captured step is
    like for like.  ``graph_note`` says what ran: "cuda graph" or why capture was not possible."""

    def __init__(self, model_cfg, world, local, batch, seq, use_graph=True):
        self.world = world
        torch.backends.cuda.matmul.allow_tf32 = True
        self.side = torch.cuda.Stream()
        self.side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.side):      # DDP built and warmed on the stream the capture will use
            self.model = TorchGPT(**model_cfg).cuda()
            self.ddp = self.model
            if world > 1:
                from torch.nn.parallel import DistributedDataParallel as DDP
                self.ddp = DDP(self.model, device_ids=[local], gradient_as_bucket_view=True)
            self.opt = torch.optim.AdamW(self.model.parameters(), lr=6e-4, betas=(0.9, 0.95), weight_decay=0.1,
                                         fused=True, capturable=use_graph)
        torch.cuda.current_stream().wait_stream(self.side)
        self.graph = None
        self.graph_note = "eager"
        self.sx = torch.zeros(batch, seq, dtype=torch.long, device="cuda")
        self.sy = torch.zeros(batch, seq, dtype=torch.long, device="cuda")
        self.sloss = None
        self.want_graph = use_graph

    def _eager(self, x, y):
        self.opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = self.ddp(x, y)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(self.model.parameters(), 1.0)
        self.opt.step()
        return loss

    def warm_and_capture(self, x, y, warm=11):
        """DDP needs about ten eager iterations on the capture stream before its buckets are stable."""
        self.side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.side):
            for _ in range(warm):
                self.sx.copy_(x)
                self.sy.copy_(y)
                self._eager(self.sx, self.sy)
        torch.cuda.current_stream().wait_stream(self.side)
        torch.cuda.synchronize()
        if not self.want_graph:
            return
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.side):
                self.sloss = self._eager(self.sx, self.sy)
            self.graph, self.graph_note = g, "cuda graph"
        except Exception as e:          # capture of this stack is not possible here: keep the eager step and say so
            torch.cuda.synchronize()
            self.graph = None
            self.graph_note = "eager (capture failed: " + repr(e)[:160] + ")"
            self.opt = torch.optim.AdamW(self.model.parameters(), lr=6e-4, betas=(0.9, 0.95), weight_decay=0.1,
                                         fused=True)

    def step(self, x, y):
        if self.graph is not None:
            self.sx.copy_(x, non_blocking=True)
            self.sy.copy_(y, non_blocking=True)
            self.graph.replay()
            return self.sloss
        return self._eager(x, y)


def measure(model_cfg, seq, world, local, batch, steps, warmup, hx, hy, dx, dy, max_over_ranks, barrier,
            use_graph=True, sampler=None):
    """Times the library step: device-timed (inputs on the device) and end to end (pinned host inputs, loss read back
    every step).  Returns a dict with ms per step for both and the graph note."""
    tr = TorchTrainer(model_cfg, world, local, batch, seq, use_graph=use_graph)
    n_batches = dx.shape[0]
    tr.warm_and_capture(dx[0], dy[0])
    if sampler is not None:
        sampler.start()          # running through the warm-up; the timed region is marked below
    for i in range(max(warmup, 3)):
        loss = tr.step(dx[i % n_batches], dy[i % n_batches])
    barrier(world)
    if sampler is not None:
        sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        j = (warmup + i) % n_batches
        loss = tr.step(dx[j], dy[j])
    e1.record()
    barrier(world)
    dev_ms = max_over_ranks(e0.elapsed_time(e1), world)
    clocks = sampler.stop() if sampler is not None else None
    barrier(world)
    t0 = time.perf_counter()
    last = 0.0
    for i in range(steps):
        j = (warmup + steps + i) % n_batches
        loss = tr.step(hx[j], hy[j]) if tr.graph is not None else \
            tr.step(hx[j].cuda(non_blocking=True), hy[j].cuda(non_blocking=True))
        last = float(loss)
    barrier(world)
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3, world)
    out = {"ms_per_step": dev_ms / steps, "e2e_ms_per_step": e2e_ms / steps, "graph": tr.graph_note, "loss_last": last,
           "clocks": clocks}
    del tr
    torch.cuda.empty_cache()
    return out


def run(args, metric, model_cfg, seq, ClockSampler, dist_setup, max_over_ranks, barrier, make_batches):
    rank, world, local = dist_setup(args.gpus)
    n_batches = args.warmup + 2 * args.steps
    hx, hy = make_batches(n_batches, args.batch, seed=1234 + rank)
    dx, dy = hx.cuda(), hy.cuda()
    m = measure(model_cfg, seq, world, local, args.batch, args.steps, args.warmup, hx, hy, dx, dy, max_over_ranks,
                barrier, use_graph=not getattr(args, "no_graph", False), sampler=ClockSampler(local) if rank == 0 else None)
    if rank == 0:
        toks = args.batch * seq * world
        print(json.dumps({
            "metric": metric, "value": toks / (m["ms_per_step"] / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": m["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "torch",
            "config": {"model": "gpt2-124m", "global_batch": args.batch * world, "seq_len": seq,
                       "parallelism": f"dp{world}", "step": m["graph"],
                       "stack": "torch autocast bf16 + cuBLAS + SDPA + fused AdamW + clip_grad_norm_ + DDP"},
            "clocks": m["clocks"],
            "e2e": {"value": toks / (m["e2e_ms_per_step"] / 1e3), "unit": "tokens/s",
                    "ms_per_step": m["e2e_ms_per_step"], "h2d_bytes_per_step": int(hx[0].numel() * 16),
                    "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "loss_last": m["loss_last"]}))
    if world > 1:
        torch.distributed.destroy_process_group()
    return

