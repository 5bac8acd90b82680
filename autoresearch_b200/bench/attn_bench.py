"""Times the attention kernels on one (B, T, H, window) case with CUDA events.

    python -m autoresearch_b200.bench.attn_bench --B 4 --T 32768 --H 8 --window 32768
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from ..ops import kernels as K
from ..ops import sm100


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--B", type=int, default=1)
    ap.add_argument("--T", type=int, default=4096)
    ap.add_argument("--H", type=int, default=2)
    ap.add_argument("--window", type=int, default=None)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--mode", type=int, default=2,
                    help="2 = wide backward (default), 1 = 64-wide sub-tiles / TMEM operands, 0 = shared-memory operands")
    a = ap.parse_args()
    W = a.window if a.window is not None else a.T
    K.attn_set_mode(a.mode)
    Dl = a.H * 128
    torch.manual_seed(0)
    qkv = torch.randn(a.B * a.T, 3 * Dl, device="cuda").to(torch.bfloat16).requires_grad_(True)
    g = torch.randn(a.B * a.T, Dl, device="cuda").to(torch.bfloat16)

    def run():
        out = sm100.AttentionFn.apply(qkv, a.B, a.T, a.H, W)
        out.backward(g)
        qkv.grad = None

    for _ in range(a.warmup):
        run()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    tf = tb = 0.0
    for _ in range(a.iters):
        ev[0].record()
        out = sm100.AttentionFn.apply(qkv, a.B, a.T, a.H, W)
        ev[1].record()
        out.backward(g)
        ev[2].record()
        torch.cuda.synchronize()
        tf += ev[0].elapsed_time(ev[1])
        tb += ev[1].elapsed_time(ev[2])
        qkv.grad = None
    K.check_err_flag()
    tf /= a.iters
    tb /= a.iters
    keys = sum(min(i, W) + 1 for i in range(a.T))  # visible (query, key) pairs per head
    flops_f = 4.0 * keys * 128 * a.H * a.B
    print(json.dumps({"B": a.B, "T": a.T, "H": a.H, "window": W, "mode": a.mode, "fwd_ms": round(tf, 3), "bwd_ms": round(tb, 3),
                      "fwd_tflops": round(flops_f / tf / 1e9, 1), "bwd_tflops": round(2.5 * flops_f / tb / 1e9, 1)}))


if __name__ == "__main__":
    main()
