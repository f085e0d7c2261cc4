"""Llama-3-8B-shaped tensor-parallel inference benchmark: batched prefill (TTFT) and greedy decode throughput.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29600 \\
        benchmarks/tp_decode_bench.py --impl ours

Config (random N(0, 0.02) weights, uniform random prompts, bf16): 32 layers, d 4096, 32 query / 8 KV heads, head 128,
RoPE theta 500000, RMSNorm eps 1e-5, SwiGLU ffn 14336, vocab 128256; batch 32 prompts x 2048 tokens prefill, then 256
greedy decode steps.  ``--impl ours`` runs ``TPLlamaEngine`` (fused GEMM + all-reduce kernels, CUDA-graph decode);
``--impl torch`` runs the same sharding with cuBLAS matmuls, SDPA and NCCL all-reduces (the library baseline), its
decode step with static shapes replayed as a CUDA graph like ours (``--no-graph`` times it eagerly).
Times are CUDA events on the launching stream, max over ranks; rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def llama8b_config(layers: int, max_ctx: int):
    from dart_pytorch_b200.models.llama import LlamaConfig
    return LlamaConfig(vocab_size=128256, max_ctx=max_ctx, embed_dim=4096, num_layers=layers, num_heads=32,
                       num_kv_heads=8, ffn_dim=14336, rope_base=500000.0, rms_norm_eps=1e-5, tie_weights=False)


class TorchTPLlama:
    """Library baseline: cuBLAS GEMMs, SDPA, NCCL all-reduce after every row-parallel projection, eager launches."""

    def __init__(self, cfg, max_batch, max_ctx, group):
        self.c, self.T, self.rank = cfg, dist.get_world_size(group), dist.get_rank(group)
        self.group = group
        T, d, hd = self.T, cfg.embed_dim, cfg.head_dim
        self.Hq, self.Hkv, self.F, self.Vl = cfg.num_heads // T, cfg.num_kv_heads // T, cfg.ffn_dim // T, cfg.vocab_size // T
        dev = torch.device("cuda", torch.cuda.current_device())
        g = torch.Generator(device=dev).manual_seed(1000 + self.rank)
        rnd = lambda r, c_: (torch.randn(r, c_, device=dev, generator=g) * 0.02).bfloat16()  # noqa: E731
        self.embed = rnd(cfg.vocab_size, d)
        self.head = rnd(self.Vl, d)
        self.layers = []
        for _ in range(cfg.num_layers):
            self.layers.append(dict(qkv=rnd((self.Hq + 2 * self.Hkv) * hd, d), wo=rnd(d, self.Hq * hd),
                                    gu=rnd(2 * self.F, d), down=rnd(d, self.F),
                                    n1=torch.ones(d, device=dev, dtype=torch.bfloat16),
                                    n2=torch.ones(d, device=dev, dtype=torch.bfloat16),
                                    k=torch.zeros(max_batch, self.Hkv, max_ctx, hd, device=dev, dtype=torch.bfloat16),
                                    v=torch.zeros(max_batch, self.Hkv, max_ctx, hd, device=dev, dtype=torch.bfloat16)))
        self.nf = torch.ones(d, device=dev, dtype=torch.bfloat16)
        half = hd // 2
        inv = cfg.rope_base ** (-2.0 * torch.arange(half, device=dev, dtype=torch.float32) / hd)
        ang = torch.arange(max_ctx, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = torch.cos(ang), torch.sin(ang)

    def _rope(self, t, pos0):
        S, half = t.shape[2], t.shape[-1] // 2
        cs, sn = self.cos[pos0:pos0 + S].view(1, 1, S, half), self.sin[pos0:pos0 + S].view(1, 1, S, half)
        a, b = t[..., :half].float(), t[..., half:].float()
        return torch.cat([a * cs - b * sn, b * cs + a * sn], -1).to(t.dtype)

    @torch.no_grad()
    def forward(self, tokens, pos0, b0=0):
        import torch.nn.functional as Fn
        c, hd = self.c, self.c.head_dim
        B, S = tokens.shape
        x = self.embed[tokens]
        for L in self.layers:
            y = Fn.rms_norm(x, (c.embed_dim,), L["n1"], c.rms_norm_eps)
            qkv = y @ L["qkv"].t()
            q, k, v = qkv.split([self.Hq * hd, self.Hkv * hd, self.Hkv * hd], -1)
            q = self._rope(q.view(B, S, self.Hq, hd).transpose(1, 2), pos0)
            k = self._rope(k.view(B, S, self.Hkv, hd).transpose(1, 2), pos0)
            v = v.view(B, S, self.Hkv, hd).transpose(1, 2)
            L["k"][b0:b0 + B, :, pos0:pos0 + S] = k
            L["v"][b0:b0 + B, :, pos0:pos0 + S] = v
            kk, vv = L["k"][b0:b0 + B, :, :pos0 + S], L["v"][b0:b0 + B, :, :pos0 + S]
            if S == 1:
                # one new token: the G query heads that share a KV head become G query rows of that head, which lets
                # the fused SDPA kernels run without materialising repeated keys
                qg = q.reshape(B, self.Hkv, self.Hq // self.Hkv, hd)
                o = Fn.scaled_dot_product_attention(qg, kk, vv).reshape(B, 1, self.Hq * hd)
            else:
                o = Fn.scaled_dot_product_attention(q, kk, vv, is_causal=True, enable_gqa=True)
                o = o.transpose(1, 2).reshape(B, S, self.Hq * hd)
            part = o @ L["wo"].t()
            dist.all_reduce(part, group=self.group)
            x = x + part
            y = Fn.rms_norm(x, (c.embed_dim,), L["n2"], c.rms_norm_eps)
            gu = y @ L["gu"].t()
            h = Fn.silu(gu[..., :self.F]) * gu[..., self.F:]
            part = h @ L["down"].t()
            dist.all_reduce(part, group=self.group)
            x = x + part
        xf = Fn.rms_norm(x[:, -1], (c.embed_dim,), self.nf, c.rms_norm_eps)
        logits = xf @ self.head.t()
        val, idx = logits.float().max(-1)
        vals = [torch.empty_like(val) for _ in range(self.T)]
        idxs = [torch.empty_like(idx) for _ in range(self.T)]
        dist.all_gather(vals, val, group=self.group)
        dist.all_gather(idxs, idx + self.rank * self.Vl, group=self.group)
        best = torch.stack(vals).argmax(0)
        return torch.stack(idxs).gather(0, best[None])[0]

    @torch.no_grad()
    def decode_static(self, tok, pos):
        """One decode step with static shapes, so that it can be captured in a CUDA graph: the position is a device
        tensor, the new K / V rows are written with ``index_copy_`` and attention runs over the whole cache under a
        length mask.  ``tok [B]`` and ``pos [1]`` (int64) are updated in place."""
        import torch.nn.functional as Fn
        c, hd = self.c, self.c.head_dim
        B = tok.shape[0]
        max_ctx = self.layers[0]["k"].shape[2]
        x = self.embed[tok].view(B, 1, -1)
        cs, sn = self.cos.index_select(0, pos).view(1, 1, 1, -1), self.sin.index_select(0, pos).view(1, 1, 1, -1)
        mask = (torch.arange(max_ctx, device=tok.device) <= pos).view(1, 1, 1, max_ctx)

        def rope(t):
            half = t.shape[-1] // 2
            a, b = t[..., :half].float(), t[..., half:].float()
            return torch.cat([a * cs - b * sn, b * cs + a * sn], -1).to(t.dtype)
        for L in self.layers:
            y = Fn.rms_norm(x, (c.embed_dim,), L["n1"], c.rms_norm_eps)
            qkv = y @ L["qkv"].t()
            q, k, v = qkv.split([self.Hq * hd, self.Hkv * hd, self.Hkv * hd], -1)
            q = rope(q.view(B, 1, self.Hq, hd).transpose(1, 2))
            k = rope(k.view(B, 1, self.Hkv, hd).transpose(1, 2))
            v = v.view(B, 1, self.Hkv, hd).transpose(1, 2)
            L["k"][:B].index_copy_(2, pos, k)
            L["v"][:B].index_copy_(2, pos, v)
            qg = q.reshape(B, self.Hkv, self.Hq // self.Hkv, hd)
            o = Fn.scaled_dot_product_attention(qg, L["k"][:B], L["v"][:B], attn_mask=mask).reshape(B, 1, self.Hq * hd)
            part = o @ L["wo"].t()
            dist.all_reduce(part, group=self.group)
            x = x + part
            y = Fn.rms_norm(x, (c.embed_dim,), L["n2"], c.rms_norm_eps)
            gu = y @ L["gu"].t()
            h = Fn.silu(gu[..., :self.F]) * gu[..., self.F:]
            part = h @ L["down"].t()
            dist.all_reduce(part, group=self.group)
            x = x + part
        xf = Fn.rms_norm(x[:, -1], (c.embed_dim,), self.nf, c.rms_norm_eps)
        logits = xf @ self.head.t()
        val, idx = logits.float().max(-1)
        vals = torch.empty(self.T, B, device=tok.device)
        idxs = torch.empty(self.T, B, dtype=torch.long, device=tok.device)
        dist.all_gather_into_tensor(vals, val, group=self.group)
        dist.all_gather_into_tensor(idxs, idx + self.rank * self.Vl, group=self.group)
        tok.copy_(idxs.gather(0, vals.argmax(0)[None])[0])
        pos.add_(1)


def measure(impl: str, layers: int, B: int, S: int, NEW: int, prefill_rows: int = 65536, prefill_reps: int = 3,
            use_graph: bool = True, group=None, prefill_modes=("ar",)):
    """Prefill (TTFT) and greedy-decode throughput of the Llama-3-8B-shaped model on the ranks of ``group``
    (``torch.distributed`` must be initialised).  Returns the result dict on every rank (times are the max over
    ranks).  ``prefill_modes``: which prefill schedules of ``TPLlamaEngine`` to time ("ar": replicated activations,
    GEMM + all-reduce; "sp": row-sharded activations, GEMM + reduce-scatter / all-gather + GEMM); the fastest is the
    reported TTFT."""
    group = group if group is not None else dist.group.WORLD
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    max_ctx = S + NEW
    cfg = llama8b_config(layers, max_ctx)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (B, S), generator=g).cuda()
    chunk = max(1, prefill_rows // S)
    note = {}
    if impl == "ours":
        from dart_pytorch_b200 import _native
        from dart_pytorch_b200.parallel.tp_llama import TPLlamaEngine
        eng = TPLlamaEngine(cfg, max_batch=B, max_ctx=max_ctx, max_rows=max(prefill_rows, B), group=group)

        def prefill(mode="ar"):
            eng.reset()
            return eng.prefill(prompts, chunk=chunk, mode=mode)

        def step():
            return eng.decode_step(B, use_graph=use_graph)
        note["cuda_graph_decode"] = bool(use_graph)
    else:
        eng = TorchTPLlama(cfg, B, max_ctx, group)
        state = {"tok": None, "pos": 0, "graph": None}
        stok = torch.zeros(B, dtype=torch.long, device="cuda")
        spos = torch.zeros(1, dtype=torch.long, device="cuda")

        def prefill(mode="ar"):
            outs = [eng.forward(prompts[b0:b0 + chunk], 0, b0) for b0 in range(0, B, chunk)]
            state["tok"], state["pos"] = torch.cat(outs), S
            stok.copy_(state["tok"])
            spos.fill_(S)
            return state["tok"]

        def capture():
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            saved = (stok.clone(), spos.clone())
            try:
                with torch.cuda.stream(side):
                    for _ in range(3):
                        eng.decode_static(stok, spos)
                    torch.cuda.synchronize()
                    dist.barrier(group=group)
                    gr = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gr, stream=side):
                        eng.decode_static(stok, spos)
                state["graph"] = gr
                note["cuda_graph_decode"] = True
            except Exception as e:      # keep the eager step and say why
                torch.cuda.synchronize()
                note["cuda_graph_decode"] = False
                note["graph_error"] = repr(e)[:160]
            torch.cuda.current_stream().wait_stream(side)
            stok.copy_(saved[0])
            spos.copy_(saved[1])

        def step():
            if state["graph"] is not None:
                state["graph"].replay()
                return stok
            state["tok"] = eng.forward(state["tok"].view(B, 1), state["pos"])
            state["pos"] += 1
            return state["tok"]
        prefill_modes = ("ar",)

    def timed(fn):
        dist.barrier(group=group)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return float(t.item())

    ttft = {}
    for mode in prefill_modes:
        prefill(mode)                                     # warm-up (allocations, descriptor caches)
        ttft[mode] = sorted(timed(lambda: prefill(mode)) for _ in range(prefill_reps))
    best_mode = min(ttft, key=lambda m: ttft[m][len(ttft[m]) // 2])
    prefill(best_mode)
    if impl == "torch" and use_graph:
        capture()
    for _ in range(3):                                    # decode warm-up; builds the CUDA graph for `ours`
        step()
    steps = NEW - 4

    def run_decode():
        for _ in range(steps):
            step()
    ms = timed(run_decode)
    if impl == "ours":
        _native.raise_on_device_error()
    med = {m: v[len(v) // 2] for m, v in ttft.items()}
    out = {"metric": "llama8b_tp_decode_tokens_per_s", "value": B * steps / (ms / 1e3), "unit": "tokens/s",
           "impl": impl, "n_gpus": world, "ttft_ms_p50": med[best_mode], "ttft_ms_all": ttft[best_mode],
           "ttft_ms_p50_by_prefill_mode": med, "prefill_mode": best_mode,
           "decode_ms_per_step": ms / steps, "decode_steps": steps, "dtype": "bf16", "data": "synthetic",
           "config": dict({"model": f"llama-3-8b-shaped ({layers} layers)", "batch": B, "prompt": S, "new": NEW,
                           "parallelism": f"tp{world}", "prefill_rows_per_call": prefill_rows}, **note)}
    if impl == "ours":
        out["nvls"] = bool(eng.comm.use_nvls)
    del eng
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "torch"])
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--prefill-rows", type=int, default=65536,
                    help="token rows per prefill call (whole sequences); both implementations use the same chunking")
    ap.add_argument("--prefill-reps", type=int, default=3)
    ap.add_argument("--prefill-modes", default="ar,sp")
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    rank, local = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    out = measure(args.impl, args.layers, args.batch, args.prompt, args.new, args.prefill_rows, args.prefill_reps,
                  use_graph=not args.no_graph, prefill_modes=tuple(m for m in args.prefill_modes.split(",") if m))
    if rank == 0:
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
