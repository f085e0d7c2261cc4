"""Per-kernel timing at the GPT-2 124M training shapes (16 x 1024 tokens, d 768), one row per kernel.

Each case is timed with CUDA events on the launching stream after warm-up, with an L2 flush (a 256 MiB write) before
every timed launch and a short device-side sleep queued ahead of it (so host launch latency is hidden and the
events bracket device time only), and reported against the measured copy bandwidth / bf16 GEMM throughput of the machine
(``MEASURED_PEAKS.json`` at the repository root when present, else 6.65 TB/s and 1.59 PFLOP/s).

    python benchmarks/kernel_bench.py                       # table of all cases
    python benchmarks/kernel_bench.py --only norm_bwd --iters 1 --warmup 1     # what a profiler run wraps

``--json PATH`` also writes the rows as JSON.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dart_pytorch_b200.ops import flash as A  # noqa: E402
from dart_pytorch_b200.ops import kernels as K  # noqa: E402


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    hbm, tf, src = 6650.0, 1590.0, "fallback"
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            hbm = float(d.get("hbm_gbs", hbm))
            tf = float(d.get("bf16_tflops", tf))
            src = "measured"
        except Exception:
            pass
    return hbm, tf, src


def build_cases(dev, want=()):
    """Cases are built only when their group is selected, so a profiler run of one kernel holds little memory."""
    def on(group):
        return not want or any(w in group or group in w for w in want)
    M, D, H, hd, B, S, V = 16384, 768, 12, 64, 16, 1024, 50257
    VP = (V + 127) // 128 * 128
    bf = dict(device=dev, dtype=torch.bfloat16)
    x = torch.randn(M, D, **bf)
    dy = torch.randn(M, D, **bf)
    dres = torch.randn(M, D, **bf)
    gamma = torch.ones(D, **bf)
    beta = torch.zeros(D, **bf)
    cases = {}

    def gemm_case(name, m, n, k, ta, tb, **kw):
        if want and not any(w in name for w in want):
            return
        a = torch.randn((k, m) if ta else (m, k), **bf)
        b = torch.randn((n, k) if tb else (k, n), **bf)
        c = torch.empty(m, n, **bf)
        extra = {}
        nbytes = 2 * (m * k + n * k + m * n)
        if kw.get("bias"):
            extra["bias"] = torch.randn(n, **bf)
        if kw.get("residual"):
            extra["residual"] = torch.randn(m, n, **bf)
            nbytes += 2 * m * n
        if kw.get("act"):
            extra["act"] = kw["act"]
        if kw.get("aux_out"):          # pre-activation copy kept for the backward pass
            extra["aux_out"] = torch.empty(m, n, **bf)
            nbytes += 2 * m * n
        if kw.get("act_bwd"):          # multiply by act'(pre-activation) in the epilogue
            extra["aux_in"] = torch.randn(m, n, **bf)
            extra["act_bwd"] = kw["act_bwd"]
            nbytes += 2 * m * n
        if kw.get("accumulate"):       # weight gradients add into the flat gradient buffer
            extra["accumulate"] = True
            c.zero_()
            nbytes += 2 * m * n
        cases[name] = (lambda: K.gemm(a, b, c, trans_a=ta, trans_b=tb, **extra), nbytes, 2.0 * m * n * k)

    gemm_case("gemm_qkv_fwd", M, 3 * D, D, False, True, bias=True)
    gemm_case("gemm_proj_fwd", M, D, D, False, True, bias=True, residual=True)
    gemm_case("gemm_fc1_fwd_gelu", M, 4 * D, D, False, True, bias=True, act="gelu_tanh_d", aux_out=True)
    gemm_case("gemm_fc2_fwd", M, D, 4 * D, False, True, bias=True, residual=True)
    gemm_case("gemm_lmhead_fwd", M, VP, D, False, True)
    gemm_case("gemm_fc1_dgrad", M, D, 4 * D, False, False)
    gemm_case("gemm_fc2_dgrad", M, 4 * D, D, False, False, act_bwd="mul")
    gemm_case("gemm_qkv_dgrad", M, D, 3 * D, False, False)
    gemm_case("gemm_fc1_wgrad", 4 * D, D, M, True, False, accumulate=True)
    gemm_case("gemm_fc2_wgrad", D, 4 * D, M, True, False, accumulate=True)
    gemm_case("gemm_qkv_wgrad", 3 * D, D, M, True, False, accumulate=True)
    gemm_case("gemm_proj_wgrad", D, D, M, True, False, accumulate=True)
    gemm_case("gemm_8192", 8192, 8192, 8192, False, True)
    # decode-sized rows: the per-GPU projections of a Llama-3-8B layer at TP = 8, batch 32 (weight streaming)
    gemm_case("gemm_dec_qkv", 32, 768, 4096, False, True)
    gemm_case("gemm_dec_wo", 32, 4096, 512, False, True)
    gemm_case("gemm_dec_gateup", 32, 3584, 4096, False, True)
    gemm_case("gemm_dec_down", 32, 4096, 1792, False, True)
    gemm_case("gemm_dec_head", 32, 16032, 4096, False, True)

    if on("norm"):
      _, mean, rstd = K.layernorm_fwd(x, gamma, beta, 1e-5)
      _, rrstd = K.rmsnorm_fwd(x, gamma, 1e-5)
    else:
      mean = rstd = rrstd = None
    cases["norm_fwd"] = (lambda: K.layernorm_fwd(x, gamma, beta, 1e-5), 2 * 2 * M * D, 0.0)
    cases["norm_bwd"] = (lambda: K.layernorm_bwd(x, dy, gamma, mean, rstd, dres=dres), 4 * 2 * M * D, 0.0)
    cases["rmsnorm_fwd"] = (lambda: K.rmsnorm_fwd(x, gamma, 1e-5), 2 * 2 * M * D, 0.0)
    cases["rmsnorm_bwd"] = (lambda: K.rmsnorm_bwd(x, dy, gamma, rrstd, dres=dres), 4 * 2 * M * D, 0.0)

    if on("attn"):
        qkv = torch.randn(M, 3 * D, **bf)
        o = torch.empty(M, D, **bf)
        q2, k2, v2 = qkv[:, :D], qkv[:, D:2 * D], qkv[:, 2 * D:]
        _, lse = A.attn_fwd(q2, k2, v2, B, S, S, H, H, hd, True, out=o)
        do = torch.randn(M, D, **bf)
        dqkv = torch.empty(M, 3 * D, **bf)
        att_flops = 4.0 * B * H * S * S * hd / 2  # causal: half of the score matrix
        cases["attn_fwd"] = (lambda: A.attn_fwd(q2, k2, v2, B, S, S, H, H, hd, True, out=o), 2 * 4 * M * D, att_flops)
        cases["attn_bwd"] = (lambda: A.attn_bwd(q2, k2, v2, o, do, lse, dqkv[:, :D], dqkv[:, D:2 * D], dqkv[:, 2 * D:],
                                                B, S, S, H, H, hd, True), 2 * 8 * M * D, 2.5 * att_flops)
    if on("ce"):
        logits = torch.randn(M, VP, **bf)
        tgt = torch.randint(0, V, (M,), device=dev)
        _, lse_ce = K.ce_fwd(logits, tgt, V)
        gone = torch.ones(1, device=dev, dtype=torch.float32)
        cases["ce_fwd"] = (lambda: K.ce_fwd(logits, tgt, V), 2 * M * VP, 0.0)
        cases["ce_bwd"] = (lambda: K.ce_bwd(logits, tgt, lse_ce, gone, 1.0 / M, V, out=logits, pad_to=VP), 4 * M * VP, 0.0)

    for cols in (D, 3 * D, 4 * D) if on("colsum") else ():
        src = torch.randn(M, cols, **bf)
        dst = torch.zeros(cols, **bf)
        cases[f"colsum_{cols}"] = (lambda src=src, dst=dst: K.colsum(src, dst, accumulate=True), 2 * M * cols, 0.0)

    if on("embedding"):
        table = torch.randn(V, D, **bf)
        pos = torch.randn(S, D, **bf)
        idx = torch.randint(0, V, (M,), device=dev)
        dtable = torch.zeros(V, D, **bf)
        cases["embedding_fwd"] = (lambda: K.embedding_fwd(table, idx, pos, 0, S), 2 * 2 * M * D, 0.0)
        cases["embedding_bwd"] = (lambda: K.embedding_bwd(dtable, idx, dy), 2 * 2 * M * D, 0.0)
    if on("adam") or on("grad_norm"):
        n = 124_500_000
        p = torch.randn(n, device=dev)           # fp32 master
        shadow = p.to(torch.bfloat16)            # bf16 working copy
        g = torch.randn(n, **bf)
        m1 = torch.zeros(n, device=dev)
        v1 = torch.zeros(n, device=dev)
        ctrl = torch.zeros(4, device=dev)
        ctrl[1] = 1.0
        ctrl[2] = 1.0
        cases["grad_norm"] = (lambda: K.grad_norm(g, ctrl, 1.0), 2 * n, 0.0)
        cases["adam_flat"] = (lambda: K.adam_flat(p, shadow, g, m1, v1, ctrl, 1e-4, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05),
                              n * (2 + 2 + 4 * 6), 0.0)
    if on("swiglu") or on("softmax"):
        gate = torch.randn(M, 4 * D, **bf)
        up = torch.randn(M, 4 * D, **bf)
        sw = torch.empty(M, 4 * D, **bf)
        cases["swiglu_fwd"] = (lambda: K.swiglu_fwd(gate, up, sw), 3 * 2 * M * 4 * D, 0.0)
        sm = torch.randn(B * H * 64, S, **bf)
        cases["softmax_fwd"] = (lambda: K.softmax_fwd(sm), 2 * 2 * sm.numel(), 0.0)
    if on("decode"):
        from dart_pytorch_b200.ops import decode as Dk
        Bd, Sk, Hq, Hkv, hdd = 32, 2304, 4, 1, 128                    # one rank of Llama-8B TP=8, batch 32
        qd = torch.randn(Bd, Hq * hdd, **bf)
        kc = torch.randn(Bd, Sk, Hkv * hdd, **bf)
        vc = torch.randn(Bd, Sk, Hkv * hdd, **bf)
        od = torch.empty(Bd, Hq * hdd, **bf)
        cases["attn_decode"] = (lambda: Dk.attn_decode(qd, kc, vc, Bd, 1, Sk, Hq, Hkv, hdd, Sk - 1, out=od),
                                2 * 2 * Bd * Sk * Hkv * hdd, 0.0)
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="", help="comma-separated substrings of case names")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    hbm, tf, src = peaks()
    want = [w for w in args.only.split(",") if w]
    cases = build_cases(dev, want)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    print(f"{'kernel':24s} {'us':>9s} {'GB/s':>8s} {'TF/s':>8s}  frac of {src} peak")
    for name, (fn, nbytes, flops) in cases.items():
        if want and not any(w in name for w in want):
            continue
        for _ in range(args.warmup):
            fn()
        ts = []
        for _ in range(args.iters):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            torch.cuda._sleep(400_000)   # the GPU idles ~0.2 ms while the host queues the launches behind it
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        us = ts[len(ts) // 2]
        gbs = nbytes / us / 1e3
        tfs = flops / us / 1e6
        frac = max(gbs / hbm, tfs / tf)
        bound = "mem" if gbs / hbm >= tfs / tf else "mma"
        print(f"{name:24s} {us:9.1f} {gbs:8.0f} {tfs:8.0f}  {frac:5.2f} ({bound})")
        rows.append(dict(kernel=name, us=us, gbs=gbs, tflops=tfs, frac=frac, bound=bound, peaks=src))
    K.N.raise_on_device_error()
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
