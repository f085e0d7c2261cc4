"""Kernel-for-kernel timing of the reference's own native CUDA library against this package's kernels.

The reference library (lib/native/src/engine.cu and kernels/*.cuh, fp32, one freshly allocated result handle per op) is
compiled unmodified by ``python -m baseline.reference_native --build <reference root>`` and driven through ctypes the way
its Dart FFI layer drives it.  Each row runs the same operation at the same shape (GPT-2 124M training shapes at
16 x 1024 tokens) through both, checks that the results agree, and reports device time from CUDA events on the stream
both use (the reference launches on the default stream).  The reference time includes what its entry point does per
call -- two ``cudaMalloc`` + two ``cudaMemset`` for the result handle -- because that is its stock code path.

    python benchmarks/reference_kernels_bench.py [--only NAME] [--iters N] [--json PATH]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from baseline.reference_native import RefLib  # noqa: E402
from dart_pytorch_b200.ops import kernels as K  # noqa: E402
from dart_pytorch_b200.ops.aft import aft_full_cuda  # noqa: E402

FLUSH = None


def flush_l2():
    global FLUSH
    if FLUSH is None:
        FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    FLUSH.add_(1)


def time_ms(fn, iters: int, warmup: int = 3, cleanup=None) -> float:
    for _ in range(warmup):
        r = fn()
        if cleanup:
            cleanup(r)
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        r = fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
        if cleanup:
            cleanup(r)
    return total / iters


def rel_err(a: np.ndarray, b: np.ndarray) -> float:
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-12))


def cases(ref: RefLib):
    rng = np.random.default_rng(0)
    M, D, F, V = 16384, 768, 3072, 50257
    bf = torch.bfloat16

    def dev(a, dtype=bf):
        return torch.from_numpy(a).cuda().to(dtype)

    def matmul():
        a = (rng.standard_normal((M, D)) * 0.5).astype(np.float32)
        b = (rng.standard_normal((D, F)) * 0.05).astype(np.float32)
        ha, hb = ref.tensor(a), ref.tensor(b)
        ta, tb = dev(a), dev(b)
        out = torch.empty(M, F, dtype=bf, device="cuda")
        return dict(name="matmul_16384x768x3072", flops=2.0 * M * D * F,
                    ref=lambda: ref.lib.matmul_tensors(ha, hb), ref_shape=(M, F),
                    ours=lambda: K.gemm(ta, tb, out), tol=2e-2, keep=(ha, hb))

    def layernorm():
        x = rng.standard_normal((M, D)).astype(np.float32)
        g = (1.0 + 0.1 * rng.standard_normal((1, D))).astype(np.float32)
        b = (0.1 * rng.standard_normal((1, D))).astype(np.float32)
        hx, hg, hb = ref.tensor(x), ref.tensor(g), ref.tensor(b)
        tx, tg, tb = dev(x), dev(g.reshape(-1)), dev(b.reshape(-1))
        return dict(name="layernorm_fwd_16384x768", bytes_=M * D * 2 * 2,
                    ref=lambda: ref.lib.layernorm_forward(hx, hg, hb, 1e-5), ref_shape=(M, D),
                    ours=lambda: K.layernorm_fwd(tx, tg, tb, 1e-5)[0], tol=3e-2, keep=(hx, hg, hb))

    def cross_entropy():
        R = 4096
        x = rng.standard_normal((R, V)).astype(np.float32)
        t = rng.integers(0, V, size=(R, 1))
        hx, ht = ref.tensor(x), ref.tensor(t.astype(np.float32))
        tx = dev(x)
        tt = torch.from_numpy(t.reshape(-1)).cuda()
        return dict(name="cross_entropy_fwd_4096x50257", bytes_=R * V * 2,
                    ref=lambda: ref.lib.cross_entropy_forward(hx, ht), ref_shape=(R, 1),
                    ours=lambda: K.ce_fwd(tx, tt, V)[0].reshape(R, 1), tol=3e-2, keep=(hx, ht))

    def softmax():
        R, C = 16384, 1024
        x = rng.standard_normal((R, C)).astype(np.float32)
        hx = ref.tensor(x)
        tx = dev(x)
        return dict(name="softmax_fwd_16384x1024", bytes_=R * C * 2 * 2,
                    ref=lambda: ref.lib.softmax_forward(hx), ref_shape=(R, C),
                    ours=lambda: K.softmax_fwd(tx), tol=3e-2, keep=(hx,))

    def embedding():
        table = (rng.standard_normal((V, D)) * 0.02).astype(np.float32)
        idx = rng.integers(0, V, size=(M, 1))
        ht, hi = ref.tensor(table), ref.tensor(idx.astype(np.float32))
        tt = dev(table)
        ti = torch.from_numpy(idx.reshape(-1)).cuda()
        return dict(name="embedding_fwd_16384x768", bytes_=M * D * 2 * 2,
                    ref=lambda: ref.lib.embedding_forward(ht, hi, M), ref_shape=(M, D),
                    ours=lambda: K.embedding_fwd(tt, ti), tol=1e-2, keep=(ht, hi))

    def add():
        a = rng.standard_normal((M, F)).astype(np.float32)
        b = rng.standard_normal((M, F)).astype(np.float32)
        ha, hb = ref.tensor(a), ref.tensor(b)
        ta, tb = dev(a), dev(b)
        return dict(name="add_16384x3072", bytes_=M * F * 2 * 3,
                    ref=lambda: ref.lib.add_tensors(ha, hb), ref_shape=(M, F),
                    ours=lambda: K.binary(ta, tb, "add"), tol=2e-2, keep=(ha, hb))

    def aft():
        T, Dm = 1024, 768
        q, k, v = (rng.standard_normal((T, Dm)).astype(np.float32) for _ in range(3))
        w = (0.1 * rng.standard_normal((T, T))).astype(np.float32)
        hq, hk, hv, hw = ref.tensor(q), ref.tensor(k), ref.tensor(v), ref.tensor(w)
        tq, tk, tv, tw = dev(q), dev(k), dev(v), dev(w)
        return dict(name="aft_full_fwd_T1024_D768", flops=4.0 * T * T * Dm / 2,
                    ref=lambda: ref.lib.aft_full_forward(hq, hk, hv, hw, 1), ref_shape=(T, Dm),
                    ours=lambda: aft_full_cuda(tq, tk, tv, tw, True), tol=5e-2, keep=(hq, hk, hv, hw))

    return {"matmul": matmul, "layernorm": layernorm, "cross_entropy": cross_entropy, "softmax": softmax,
            "embedding": embedding, "add": add, "aft": aft}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    ref = RefLib()
    rows = []
    for key, make in cases(ref).items():
        if args.only and args.only not in key:
            continue
        c = make()
        h = c["ref"]()
        torch.cuda.synchronize()
        want = ref.read(h, *c["ref_shape"])
        ref.free(h)
        with torch.no_grad():
            got = c["ours"]().float().cpu().numpy().reshape(c["ref_shape"])
            err = rel_err(got, want)
            t_ref = time_ms(c["ref"], args.iters, cleanup=ref.free)
            t_ours = time_ms(c["ours"], args.iters)
        row = {"name": c["name"], "reference_ms": round(t_ref, 4), "ours_ms": round(t_ours, 4),
               "speedup": round(t_ref / t_ours, 1), "max_rel_err": err, "agree": bool(err < c["tol"])}
        if "flops" in c:
            row["reference_tflops"] = round(c["flops"] / t_ref / 1e9, 2)
            row["ours_tflops"] = round(c["flops"] / t_ours / 1e9, 2)
        if "bytes_" in c:
            row["ours_gbs"] = round(c["bytes_"] / t_ours / 1e6, 1)
        print(json.dumps(row), flush=True)
        rows.append(row)
        ref.free(*c["keep"])
        torch.cuda.empty_cache()
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    if not all(r["agree"] for r in rows):
        sys.exit(1)


if __name__ == "__main__":
    main()
