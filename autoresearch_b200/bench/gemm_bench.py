"""Times the tcgen05 GEMM on one shape with CUDA events and compares with torch.matmul (cuBLAS).

    python -m autoresearch_b200.bench.gemm_bench --M 131072 --N 3072 --K 1024 --layout nt --mode 0
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import kernels as K


def timeit(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


HEADLINE_SHAPES = [  # (name, M, N, K, layout) at the 428 M config, 131072 tokens per micro-batch
    ("qkv fwd", 131072, 3072, 1024, "nt"), ("o-proj fwd", 131072, 1024, 1024, "nt"),
    ("fc1 fwd", 131072, 4096, 1024, "nt"), ("fc2 fwd", 131072, 1024, 4096, "nt"),
    ("fc2 dX", 131072, 4096, 1024, "nn"), ("qkv dX", 131072, 1024, 3072, "nn"),
    ("fc1 dW", 4096, 1024, 131072, "tn"), ("o-proj dW", 1024, 1024, 131072, "tn"),
    ("lm head chunk", 16384, 8192, 1024, "nt"),
]


PHASE1_SHAPES = [  # the 119.5 M config (D=512): 64 sequences of 2048 tokens per micro-batch
    ("qkv fwd", 131072, 1536, 512, "nt"), ("o-proj fwd", 131072, 512, 512, "nt"),
    ("fc1 fwd", 131072, 2048, 512, "nt"), ("fc2 fwd", 131072, 512, 2048, "nt"),
    ("fc2 dX", 131072, 2048, 512, "nn"), ("qkv dX", 131072, 512, 1536, "nn"),
    ("fc1 dW", 2048, 512, 131072, "tn"), ("o-proj dW", 512, 512, 131072, "tn"),
    ("lm head chunk", 16384, 8192, 512, "nt"),
]


def table(iters=10, warmup=3, shapes=None):
    """Markdown table of the headline shapes: own kernel vs torch.matmul, CUDA events."""
    rows = ["| GEMM | M | N | K | layout | own ms | own TFLOP/s | cuBLAS ms | cuBLAS TFLOP/s | ratio |", "|---|---|---|---|---|---|---|---|---|---|"]
    g = torch.Generator(device="cuda").manual_seed(0)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
    for name, M, N, Kd, lay in (shapes or HEADLINE_SHAPES):
        if lay == "nt":
            x, w = r(M, Kd), r(N, Kd)
            f, ref = (lambda: K.gemm(x, w)), (lambda: x @ w.t())
        elif lay == "nn":
            x, w = r(M, Kd), r(Kd, N)
            f, ref = (lambda: K.gemm(x, w, trans_b=False)), (lambda: x @ w)
        else:
            x, w = r(Kd, M), r(Kd, N)
            acc = torch.zeros(M, N, device="cuda")
            f, ref = (lambda: K.gemm(x, w, trans_a=True, trans_b=False, out=acc, epi=K.EPI_ATOMIC_F32)), (lambda: x.t() @ w)
        t1, t2 = timeit(f, iters, warmup), timeit(ref, iters, warmup)
        fl = 2.0 * M * N * Kd / 1e9
        rows.append(f"| {name} | {M} | {N} | {Kd} | {lay} | {t1:.3f} | {fl / t1:.0f} | {t2:.3f} | {fl / t2:.0f} | {t2 / t1:.2f} |")
        del x, w
    K.check_err_flag()
    return "\n".join(rows)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--table", action="store_true", help="print the table of one model's GEMM shapes and exit")
    ap.add_argument("--shapes", default="headline", choices=["headline", "phase1"], help="which model's shapes --table times")
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--K", type=int, default=1024)
    ap.add_argument("--layout", default="nt", choices=["nt", "nn", "tn"])
    ap.add_argument("--mode", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-ref", action="store_true")
    a = ap.parse_args()
    if a.table:
        print(table(a.iters, a.warmup, PHASE1_SHAPES if a.shapes == "phase1" else HEADLINE_SHAPES))
        return
    K.gemm_set_mode(a.mode)
    M, N, Kd = a.M, a.N, a.K
    g = torch.Generator(device="cuda").manual_seed(0)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
    if a.layout == "nt":
        x, w = r(M, Kd), r(N, Kd)
        f, ref = (lambda: K.gemm(x, w)), (lambda: x @ w.t())
    elif a.layout == "nn":
        x, w = r(M, Kd), r(Kd, N)
        f, ref = (lambda: K.gemm(x, w, trans_b=False)), (lambda: x @ w)
    else:
        x, w = r(Kd, M), r(Kd, N)
        acc = torch.zeros(M, N, device="cuda")
        f, ref = (lambda: K.gemm(x, w, trans_a=True, trans_b=False, out=acc, epi=K.EPI_ATOMIC_F32)), (lambda: x.t() @ w)
    t = timeit(f, a.iters, a.warmup)
    out = {"M": M, "N": N, "K": Kd, "layout": a.layout, "mode": a.mode, "ms": round(t, 4),
           "tflops": round(2.0 * M * N * Kd / t / 1e9, 1)}
    if not a.no_ref:
        t2 = timeit(ref, a.iters, a.warmup)
        out["cublas_ms"] = round(t2, 4)
        out["cublas_tflops"] = round(2.0 * M * N * Kd / t2 / 1e9, 1)
    K.check_err_flag()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
