"""Tiny character-level GPT on the CPU in fp32: the smallest end-to-end workload of the framework.

Vocabulary 65, d_model 64, 2 pre-LN blocks, 4 heads, MLP 4x, learned positions, context 32, weight-tied head, dropout
0.1; batch 8 of token ids uniform in [0, 65) from seed 0, weights N(0, 0.02).  200 steps of Adam (lr 3e-3, 20-step linear
warm-up then cosine, gradient clipping at 1.0), then a DPTC checkpoint is written, loaded into a fresh model and both
generate 32 tokens greedily through the KV cache (the recipe of the reference's trainer, bin/gpt_train.dart:111-131,
and of its cached generate, lib/core/nn/gpt.dart:185-259).

``--impl torch`` runs the same model restated in plain PyTorch modules on the CPU (the timed CPU baseline).

    python benchmarks/tiny_gpt_cpu.py [--impl ours|torch] [--steps 200]
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import tempfile
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

V, D, L, H, CTX, B = 65, 64, 2, 4, 32, 8
LR, WARM, CLIP = 3e-3, 20, 1.0


def batches(steps: int):
    g = torch.Generator().manual_seed(0)
    for _ in range(steps):
        tok = torch.randint(0, V, (B, CTX + 1), generator=g)
        yield tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


def run_ours(steps: int) -> dict:
    from dart_pytorch_b200 import Adam, Checkpoint, clip_grad_norm
    from dart_pytorch_b200.models.gpt import GPT, GPTConfig
    from dart_pytorch_b200.nn.transformer import Activation
    from dart_pytorch_b200.optim.lr_scheduler import LinearWarmupCosineDecay

    def make(seed):
        return GPT(GPTConfig(vocab_size=V, max_ctx=CTX, embed_dim=D, num_layers=L, num_heads=H, ffn_dim=4 * D,
                             dropout_p=0.1, tie_weights=True, activation=Activation.geluTanh, seed=seed, init_std=0.02))
    model = make(0)
    opt = Adam(model.parameters(), lr=LR)
    sched = LinearWarmupCosineDecay(opt, warmup_steps=WARM, total_steps=steps, max_lr=LR)
    model.train()
    losses, step_s = [], []
    t0 = time.perf_counter()
    for x, y in batches(steps):
        t_step = time.perf_counter()
        opt.zero_grad()
        loss = model.loss(x, y)
        loss.backward()
        clip_grad_norm(model.parameters(), CLIP)
        opt.step()
        sched.step()
        losses.append(float(loss.detach()))
        step_s.append(time.perf_counter() - t_step)
    train_s = time.perf_counter() - t0
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "tiny.dptc")
        Checkpoint.save_file(model, path)
        size = os.path.getsize(path)
        clone = make(123)
        Checkpoint.load_into_file(clone, path)
    same = all(torch.equal(a.detach(), b.detach()) for a, b in zip(model.parameters(), clone.parameters()))
    t0 = time.perf_counter()
    out_a = model.generate([1.0, 2.0, 3.0], 32, temperature=0.0)
    gen_s = time.perf_counter() - t0
    out_b = clone.generate([1.0, 2.0, 3.0], 32, temperature=0.0)
    out_nc = model.generate([1.0, 2.0, 3.0], 29, temperature=0.0, use_cache=False)
    return {"impl": "ours", "ms_per_step": 1e3 * train_s / steps, "median_ms_per_step": 1e3 * sorted(step_s)[len(step_s) // 2], "loss_first": losses[0], "loss_last": losses[-1],
            "checkpoint_bytes": size, "checkpoint_round_trip": bool(same),
            "generate_matches_after_reload": out_a == out_b, "cache_matches_no_cache": out_a[:len(out_nc)] == out_nc,
            "generate_ms_per_token": 1e3 * gen_s / 32, "generated": [int(t) for t in out_a]}


def run_torch(steps: int) -> dict:
    import torch.nn as nn
    import torch.nn.functional as F

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.ln1, self.ln2 = nn.LayerNorm(D), nn.LayerNorm(D)
            self.qkv, self.proj = nn.Linear(D, 3 * D, bias=False), nn.Linear(D, D, bias=False)
            self.fc1, self.fc2 = nn.Linear(D, 4 * D), nn.Linear(4 * D, D)
            self.drop = nn.Dropout(0.1)

        def forward(self, x):
            b, t, _ = x.shape
            q, k, v = self.qkv(self.ln1(x)).view(b, t, 3, H, D // H).permute(2, 0, 3, 1, 4)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(b, t, D)
            x = x + self.drop(self.proj(a))
            return x + self.drop(self.fc2(F.gelu(self.fc1(self.ln2(x)), approximate="tanh")))

    class Tiny(nn.Module):
        def __init__(self):
            super().__init__()
            self.tok, self.pos = nn.Embedding(V, D), nn.Embedding(CTX, D)
            self.blocks = nn.ModuleList(Block() for _ in range(L))
            self.lnf = nn.LayerNorm(D)
            self.drop = nn.Dropout(0.1)

        def forward(self, x):
            h = self.drop(self.tok(x) + self.pos(torch.arange(x.shape[1])))
            for blk in self.blocks:
                h = blk(h)
            return self.lnf(h) @ self.tok.weight.t()

    torch.manual_seed(0)
    model = Tiny()
    for p in model.parameters():
        if p.dim() > 1:
            nn.init.normal_(p, std=0.02)
    opt = torch.optim.Adam(model.parameters(), lr=LR)

    def lr_at(step):
        if step <= WARM:
            return LR * step / WARM
        return 0.5 * LR * (1.0 + math.cos(math.pi * (step - WARM) / (steps - WARM)))
    losses, step_s = [], []
    t0 = time.perf_counter()
    for i, (x, y) in enumerate(batches(steps)):
        t_step = time.perf_counter()
        for g in opt.param_groups:
            g["lr"] = lr_at(i + 1)
        opt.zero_grad(set_to_none=True)
        loss = F.cross_entropy(model(x).reshape(-1, V), y.reshape(-1))
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), CLIP)
        opt.step()
        losses.append(float(loss.detach()))
        step_s.append(time.perf_counter() - t_step)
    train_s = time.perf_counter() - t0
    return {"impl": "torch", "ms_per_step": 1e3 * train_s / steps, "median_ms_per_step": 1e3 * sorted(step_s)[len(step_s) // 2], "loss_first": losses[0], "loss_last": losses[-1]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "torch"])
    ap.add_argument("--steps", type=int, default=200)
    args = ap.parse_args()
    torch.set_num_threads(max(1, min(8, os.cpu_count() or 1)))
    res = run_ours(args.steps) if args.impl == "ours" else run_torch(args.steps)
    res.update({"metric": "tiny_char_gpt_cpu_ms_per_step", "steps": args.steps, "dtype": "fp32", "device": "cpu",
                "config": {"vocab": V, "d_model": D, "layers": L, "heads": H, "ctx": CTX, "batch": B}})
    print(json.dumps(res))


if __name__ == "__main__":
    main()
