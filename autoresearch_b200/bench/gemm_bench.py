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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--K", type=int, default=1024)
    ap.add_argument("--layout", default="nt", choices=["nt", "nn", "tn"])
    ap.add_argument("--mode", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-ref", action="store_true")
    ap.add_argument("--flags", type=int, default=0)
    a = ap.parse_args()
    K.gemm_set_mode(a.mode)
    if a.flags:
        import ctypes
        K.lib().arb_gemm_set_flags(ctypes.c_int(a.flags))
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
