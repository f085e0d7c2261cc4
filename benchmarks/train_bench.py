"""Training-step benchmarks of the two other training configurations: ViT-B/16 data-parallel and the MoE causal LM
with expert parallelism.  One rank per GPU; CUDA-event timing, max over ranks; rank 0 prints one JSON line.

    python benchmarks/train_bench.py --workload vit_b16 --impl ours            # 1 GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29650 \\
        benchmarks/train_bench.py --workload moe_ep --impl ours

vit_b16: images 224x224x3 ~ N(0,1), 16x16 patches, 12 layers, d 768, 12 heads, MLP 3072, CLS token, 1000 classes,
         batch 128 per GPU, AdamW lr 1e-3, clip 1.0, bf16.
moe_ep:  16 layers, d 1024, 16 heads, RMSNorm, RoPE 10000; every MLP is an MoE of 8 SwiGLU experts (ffn 4096), softmax
         top-2, capacity factor 1.25, aux loss 0.01; seq 2048, 8 sequences per GPU, vocab 32000; experts sharded over
         the ranks, everything else data-parallel.

``--impl torch`` is the library baseline of the same model: PyTorch modules in bf16 autocast with SDPA, fused AdamW,
DDP; the MoE baseline exchanges tokens with ``all_to_all_single`` and runs the experts with cuBLAS.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

VIT = dict(image_size=224, patch_size=16, embed_dim=768, num_layers=12, num_heads=12, ffn_dim=3072, num_classes=1000)
MOE = dict(vocab=32000, d=1024, layers=16, heads=16, experts=8, ffn=4096, top_k=2, cf=1.25, aux=0.01, seq=2048)


def setup():
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29650")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), rank=rank, world_size=world)
    return rank, world


def timed_steps(step_fn, steps, warmup, world):
    for _ in range(warmup):
        step_fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step_fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()) / steps


# ------------------------------------------------------------------------------------------------- ViT-B/16 ---
def vit_ours(args, rank, world):
    import dart_pytorch_b200 as dp
    from dart_pytorch_b200.models import ViTClassifier
    from dart_pytorch_b200.nn.transformer import Activation
    from dart_pytorch_b200.parallel.dp import GradReducer
    from dart_pytorch_b200.utils.trainer import Trainer
    model = ViTClassifier(activation=Activation.geluTanh, attn_bias=True, device="cuda", dtype=torch.bfloat16,
                          init_std=0.02, **VIT)
    opt = dp.Adam(model.parameters(), lr=1e-3, beta1=0.9, beta2=0.999, weight_decay=0.05)
    reducer = GradReducer(opt.arena, world, overlap=True) if world > 1 else None
    tr = Trainer(model, opt, None, clip_norm=1.0, use_graph=not args.no_graph, reducer=reducer)
    g = torch.Generator(device="cuda").manual_seed(rank)
    xs = [torch.randn(args.batch, 3, 224, 224, device="cuda", generator=g).bfloat16() for _ in range(4)]
    ys = [torch.randint(0, 1000, (args.batch,), device="cuda", generator=g) for _ in range(4)]
    i = [0]

    def step():
        i[0] += 1
        return tr.step(xs[i[0] % 4], ys[i[0] % 4])
    return step


class _TorchViT(torch.nn.Module):
    def __init__(self):
        super().__init__()
        d = VIT["embed_dim"]
        self.patch = torch.nn.Conv2d(3, d, 16, 16)
        self.cls = torch.nn.Parameter(torch.zeros(1, 1, d))
        self.pos = torch.nn.Parameter(torch.randn(1, 197, d) * 0.02)
        layer = torch.nn.TransformerEncoderLayer(d, VIT["num_heads"], VIT["ffn_dim"], dropout=0.0, activation="gelu",
                                                 batch_first=True, norm_first=True)
        self.enc = torch.nn.TransformerEncoder(layer, VIT["num_layers"], norm=torch.nn.LayerNorm(d),
                                               enable_nested_tensor=False)
        self.head = torch.nn.Linear(d, VIT["num_classes"])

    def forward(self, x):
        t = self.patch(x).flatten(2).transpose(1, 2)
        h = torch.cat([self.cls.expand(t.shape[0], -1, -1), t], 1) + self.pos
        return self.head(self.enc(h)[:, 0])


def vit_torch(args, rank, world):
    model = _TorchViT().cuda()
    ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[torch.cuda.current_device()]) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.05, fused=True)
    g = torch.Generator(device="cuda").manual_seed(rank)
    xs = [torch.randn(args.batch, 3, 224, 224, device="cuda", generator=g) for _ in range(4)]
    ys = [torch.randint(0, 1000, (args.batch,), device="cuda", generator=g) for _ in range(4)]
    i = [0]

    def step():
        i[0] += 1
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(ddp(xs[i[0] % 4]).float(), ys[i[0] % 4])
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        return loss
    return step


# --------------------------------------------------------------------------------------------------- MoE EP ---
def moe_ours(args, rank, world):
    import dart_pytorch_b200 as dp
    from dart_pytorch_b200.models import MoELanguageModel
    from dart_pytorch_b200.nn.moe import ExpertVariant
    from dart_pytorch_b200.parallel.dp import GradReducer
    from dart_pytorch_b200.utils.trainer import Trainer
    m = MOE
    model = MoELanguageModel(m["vocab"], m["d"], args.layers or m["layers"], m["heads"], m["seq"],
                             num_routed_experts=m["experts"], num_shared_experts=0, top_k=m["top_k"],
                             expert_hidden_dim=m["ffn"], expert_variant=ExpertVariant.swiGlu, norm="rms",
                             rope_base=10000.0, capacity_factor=m["cf"], aux_loss_coef=m["aux"], expert_bias=False,
                             head_bias=False, device="cuda", dtype=torch.bfloat16, init_std=0.02,
                             ep_group=dist.group.WORLD)
    opt = dp.Adam(model.parameters(), lr=3e-4, beta1=0.9, beta2=0.95, weight_decay=0.1)
    reducer = GradReducer(opt.arena, world, overlap=False, exclude=model.expert_parameters()) if world > 1 else None
    tr = Trainer(model, opt, None, clip_norm=1.0, use_graph=False, reducer=reducer)
    g = torch.Generator(device="cuda").manual_seed(rank)
    toks = [torch.randint(0, m["vocab"], (args.batch, m["seq"] + 1), device="cuda", generator=g) for _ in range(4)]
    i = [0]

    def step():
        i[0] += 1
        t = toks[i[0] % 4]
        return tr.step(t[:, :-1].contiguous(), t[:, 1:].contiguous())
    return step


class _TorchMoEBlock(torch.nn.Module):
    def __init__(self, world):
        super().__init__()
        m = MOE
        d = m["d"]
        self.n1, self.n2 = torch.nn.RMSNorm(d), torch.nn.RMSNorm(d)
        self.qkv, self.wo = torch.nn.Linear(d, 3 * d, bias=False), torch.nn.Linear(d, d, bias=False)
        self.gate = torch.nn.Linear(d, m["experts"], bias=False)
        self.El = m["experts"] // world
        self.w1 = torch.nn.Parameter(torch.randn(self.El, 2 * m["ffn"], d) * 0.02)
        self.w2 = torch.nn.Parameter(torch.randn(self.El, d, m["ffn"]) * 0.02)
        self.world = world

    def moe(self, x):
        m = MOE
        T, d = x.shape
        E, k, W = m["experts"], m["top_k"], self.world
        C = int(math.ceil(m["cf"] * T * k / E))
        probs = torch.softmax(self.gate(x).float(), -1)
        w, idx = torch.topk(probs, k, -1)
        flat_e = idx.reshape(-1)
        onehot = torch.nn.functional.one_hot(flat_e, E)
        slot = (onehot.cumsum(0) - 1).gather(1, flat_e[:, None])[:, 0]
        keep = slot < C
        send = x.new_zeros(E * C, d)
        pos = flat_e * C + slot
        src_rows = torch.arange(T, device=x.device).repeat_interleave(k)
        send.index_copy_(0, pos[keep], x[src_rows[keep]])
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send)                       # [W][El][C][d] rows for my experts
        r = recv.view(W, self.El, C, d).transpose(0, 1).reshape(self.El, W * C, d)
        h = torch.bmm(r, self.w1.transpose(1, 2).to(r.dtype))
        F_ = m["ffn"]
        h = torch.nn.functional.silu(h[..., :F_]) * h[..., F_:]
        o = torch.bmm(h, self.w2.transpose(1, 2).to(h.dtype))
        back_in = o.view(self.El, W, C, d).transpose(0, 1).reshape(E * C, d).contiguous()
        back = torch.empty_like(back_in)
        dist.all_to_all_single(back, back_in)
        gathered = back[pos.clamp(max=E * C - 1)] * (w.reshape(-1, 1) * keep[:, None]).to(back.dtype)
        y = x.new_zeros(T, d).index_add_(0, src_rows, gathered.to(x.dtype))
        f = onehot.float().mean(0)
        return y, m["aux"] * E * (f * probs.mean(0)).sum()

    def forward(self, x, cos, sin):
        B, S, d = x.shape
        H = MOE["heads"]
        q, k, v = self.qkv(self.n1(x)).view(B, S, 3, H, d // H).permute(2, 0, 3, 1, 4)

        def rope(t):
            a, b = t[..., :d // H // 2], t[..., d // H // 2:]
            return torch.cat([a * cos - b * sin, b * cos + a * sin], -1).to(t.dtype)
        o = torch.nn.functional.scaled_dot_product_attention(rope(q), rope(k), v, is_causal=True)
        x = x + self.wo(o.transpose(1, 2).reshape(B, S, d))
        y, aux = self.moe(self.n2(x).reshape(B * S, d))
        return x + y.view(B, S, d), aux


class _TorchMoE(torch.nn.Module):
    def __init__(self, world, layers):
        super().__init__()
        m = MOE
        self.emb = torch.nn.Embedding(m["vocab"], m["d"])
        self.blocks = torch.nn.ModuleList([_TorchMoEBlock(world) for _ in range(layers)])
        self.norm = torch.nn.RMSNorm(m["d"])
        self.head = torch.nn.Linear(m["d"], m["vocab"], bias=False)
        hd = m["d"] // m["heads"]
        inv = 10000.0 ** (-2.0 * torch.arange(hd // 2).float() / hd)
        ang = torch.arange(m["seq"]).float()[:, None] * inv[None]
        self.register_buffer("cos", torch.cos(ang)[None, None])
        self.register_buffer("sin", torch.sin(ang)[None, None])

    def forward(self, tok):
        x = self.emb(tok)
        aux = 0.0
        for b in self.blocks:
            x, a = b(x, self.cos, self.sin)
            aux = aux + a
        return self.head(self.norm(x)), aux


def moe_torch(args, rank, world):
    m = MOE
    model = _TorchMoE(world, args.layers or m["layers"]).cuda()
    shared = [p for n, p in model.named_parameters() if not (n.endswith(".w1") or n.endswith(".w2"))]
    expert = [p for n, p in model.named_parameters() if n.endswith(".w1") or n.endswith(".w2")]
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    g = torch.Generator(device="cuda").manual_seed(rank)
    toks = [torch.randint(0, m["vocab"], (args.batch, m["seq"] + 1), device="cuda", generator=g) for _ in range(4)]
    i = [0]

    def step():
        i[0] += 1
        t = toks[i[0] % 4]
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits, aux = model(t[:, :-1])
            loss = torch.nn.functional.cross_entropy(logits.float().view(-1, m["vocab"]), t[:, 1:].reshape(-1)) + aux
        loss.backward()
        if world > 1:
            live = [p for p in shared if p.grad is not None]
            flat = torch.cat([p.grad.reshape(-1) for p in live])
            dist.all_reduce(flat, op=dist.ReduceOp.AVG)
            off = 0
            for p in live:
                p.grad.copy_(flat[off:off + p.numel()].view_as(p))
                off += p.numel()
            for p in expert:
                if p.grad is not None:
                    p.grad.div_(world)
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        return loss
    return step


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", required=True, choices=["vit_b16", "moe_ep"])
    ap.add_argument("--impl", default="ours", choices=["ours", "torch"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    rank, world = setup()
    if args.workload == "vit_b16":
        args.batch = args.batch or 128
        step = (vit_ours if args.impl == "ours" else vit_torch)(args, rank, world)
        per_gpu, unit = args.batch, "images/s"
    else:
        args.batch = args.batch or 8
        step = (moe_ours if args.impl == "ours" else moe_torch)(args, rank, world)
        per_gpu, unit = args.batch * MOE["seq"], "tokens/s"
    ms = timed_steps(step, args.steps, args.warmup, world)
    loss = float(step())
    if args.impl == "ours":
        from dart_pytorch_b200 import _native
        _native.raise_on_device_error()
    if rank == 0:
        print(json.dumps({"metric": f"{args.workload}_train_{unit.split('/')[0]}_per_s", "value": per_gpu * world / (ms / 1e3),
                          "unit": unit, "impl": args.impl, "n_gpus": world, "ms_per_step": ms, "steps": args.steps,
                          "warmup": args.warmup, "dtype": "bf16", "data": "synthetic", "loss": loss,
                          "config": {"workload": args.workload, "per_gpu_batch": args.batch,
                                     "layers": args.layers or (MOE["layers"] if args.workload == "moe_ep" else VIT["num_layers"])}}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
