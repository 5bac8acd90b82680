"""Times the attention kernels on one (B, T, H, window) case with CUDA events.

    python -m autoresearch_b200.bench.attn_bench --B 4 --T 32768 --H 8 --window 32768
    python -m autoresearch_b200.bench.attn_bench --B 4 --T 32768 --H 8 --modes 1,2     # A/B in one process

The kernels are called through the C interface on preallocated buffers (no autograd, no allocator), the
variants named by ``--modes`` are interleaved round-robin so that clock and temperature drift hits all of
them alike, and the median over ``--iters`` rounds is reported.  Before timing, the GPU is kept busy for
``--warmup-seconds`` so that short cases are not measured while the clocks ramp up.
"""
from __future__ import annotations

import argparse
import json
import math
import statistics
import time

import torch

from ..ops import kernels as K


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--B", type=int, default=1)
    ap.add_argument("--T", type=int, default=4096)
    ap.add_argument("--H", type=int, default=2)
    ap.add_argument("--window", type=int, default=None)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup-seconds", type=float, default=0.5)
    ap.add_argument("--modes", type=str, default="2",
                    help="comma list: 2 = 128x128 tiles, ten warps (default); 1 = six-warp kernels, 64-wide backward "
                         "sub-tiles, TMEM operands; 0 = same with shared-memory operands (forward too)")
    a = ap.parse_args()
    W = a.window if a.window is not None else a.T
    B, T, H = a.B, a.T, a.H
    Dl = H * 128
    modes = [int(m) for m in a.modes.split(",")]
    torch.manual_seed(0)
    qkv = torch.randn(B * T, 3 * Dl, device="cuda").to(torch.bfloat16)
    g = torch.randn(B * T, Dl, device="cuda").to(torch.bfloat16)
    out = torch.empty(B * T, Dl, dtype=torch.bfloat16, device="cuda")
    dqkv = torch.empty_like(qkv)
    lse = torch.empty(B, H, T, dtype=torch.float32, device="cuda")
    delta = torch.empty_like(lse)
    L = K.lib()
    err = K.err_flag().data_ptr()
    st = K._stream()
    b, db = qkv.data_ptr(), dqkv.data_ptr()
    sc = 1.0 / math.sqrt(128)

    def fwd():
        rc = L.arb_attn_fwd(b, b + 2 * Dl, b + 4 * Dl, out.data_ptr(), lse.data_ptr(), B, T, H, 3 * Dl, 3 * Dl, 3 * Dl, Dl, W, sc,
                            err, st)
        assert rc == 0, rc

    def bwd():
        rc = L.arb_attn_bwd(b, b + 2 * Dl, b + 4 * Dl, out.data_ptr(), g.data_ptr(), lse.data_ptr(), db, db + 2 * Dl, db + 4 * Dl,
                            delta.data_ptr(), None, B, T, H, 3 * Dl, 3 * Dl, 3 * Dl, Dl, Dl, 3 * Dl, 3 * Dl, 3 * Dl, W, sc, err, st)
        assert rc == 0, rc

    t0 = time.time()
    while time.time() - t0 < a.warmup_seconds:
        for m in modes:
            K.attn_set_mode(m)
            fwd(); bwd()
        torch.cuda.synchronize()
    K.check_err_flag()
    res = {m: {"fwd": [], "bwd": []} for m in modes}
    reps = max(1, int(20e-3 / max(1e-4, (time.time() - t0) / 50)))  # several launches per event pair for short cases
    reps = min(reps, 20) if T * B * H < 2 ** 20 else 1
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    for _ in range(a.iters):
        for m in modes:
            K.attn_set_mode(m)
            ev[0].record()
            for _r in range(reps):
                fwd()
            ev[1].record()
            for _r in range(reps):
                bwd()
            ev[2].record()
            torch.cuda.synchronize()
            res[m]["fwd"].append(ev[0].elapsed_time(ev[1]) / reps)
            res[m]["bwd"].append(ev[1].elapsed_time(ev[2]) / reps)
    K.check_err_flag()
    K.attn_set_mode(2)
    keys = sum(min(i, W) + 1 for i in range(T))  # visible (query, key) pairs per head
    flops_f = 4.0 * keys * 128 * H * B
    for m in modes:
        tf, tb = statistics.median(res[m]["fwd"]), statistics.median(res[m]["bwd"])
        print(json.dumps({"B": B, "T": T, "H": H, "window": W, "mode": m, "fwd_ms": round(tf, 3), "bwd_ms": round(tb, 3),
                          "fwd_min_ms": round(min(res[m]["fwd"]), 3), "bwd_min_ms": round(min(res[m]["bwd"]), 3),
                          "fwd_tflops": round(flops_f / tf / 1e9, 1), "bwd_tflops": round(2.5 * flops_f / tb / 1e9, 1)}))


if __name__ == "__main__":
    main()
