"""Per-role cycle accounting of the wide attention backward kernels.

    python -m autoresearch_b200.bench.attn_roles --T 32768 --H 8

Compiles ``ops/csrc/attn_wide_sm100.cu`` with ``-DARB_ATTN_PROF`` into a temporary library (the marks are
compiled out of the production library), runs the backward once on random data and prints, for the CTA
with the longest loop, the clock64() cycles per 128 x 128 tile that the MMA-issuing thread and two of the
softmax warps spend in each phase and on each barrier.  A tool for finding the critical path; its totals
carry the overhead of the clock reads (about 5 %).
"""
from __future__ import annotations

import argparse
import ctypes as C
import math
import subprocess
import tempfile
from pathlib import Path

import torch

from ..ops import build as B


def fwd2(a):
    """Cycles per key tile (both query tiles) of the MMA-issuing thread and of one warp of each softmax group."""
    T, H = a.T, a.H
    which = a.kernel          # "fwd2" or "fwd3": same roles, same entry-point signature
    W = a.window if a.window is not None else T
    with tempfile.TemporaryDirectory(prefix="arb_prof_") as td:
        so = Path(td) / "attn_prof.so"
        flags = [f for f in B.NVCC_FLAGS if f not in ("-Xptxas", "-v")]
        subprocess.run([B.nvcc_path()] + flags + ["-DARB_ATTN_PROF", "-shared", str(B.CSRC / f"attn_{which}_sm100.cu"), "-o", str(so),
                        "-lcuda"], check=True)
        lib = C.CDLL(str(so))
        Dl = H * 128
        torch.manual_seed(0)
        qkv = torch.randn(T, 3 * Dl, device="cuda").to(torch.bfloat16)
        o = torch.empty(T, Dl, device="cuda", dtype=torch.bfloat16)
        lse = torch.empty(1, H, T, device="cuda")
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        prof = torch.zeros(64, dtype=torch.int64, device="cuda")
        vp, ll, ci = C.c_void_p, C.c_longlong, C.c_int
        f = getattr(lib, f"arb_attn_prof_{which}")
        f.restype = ci
        f.argtypes = [vp] * 5 + [ci, ci, ci, ll, ll, ci, C.c_float, vp, vp]
        b = qkv.data_ptr()
        for _ in range(2):
            prof.zero_()
            e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(2))
            e1.record()
            rc = f(b, b + 2 * Dl, b + 4 * Dl, o.data_ptr(), lse.data_ptr(), 1, T, H, 3 * Dl, Dl, W, 1 / math.sqrt(128),
                   err.data_ptr(), prof.data_ptr())
            e2.record()
            torch.cuda.synchronize()
            assert rc == 0 and err.item() == 0, (rc, err.item())
        print(f"B=1 T={T} H={H} window={W}: forward (two query tiles per CTA) {e1.elapsed_time(e2):.3f} ms (with the profiling marks)")
        p = prof.cpu()
        nt = (T + 127) // 128 if W >= T else (W // 128 + 2)
        print(f"cycles per key tile, heaviest CTA ({nt} key tiles, two query tiles each)")
        # fwd3: marks inside the issuing thread cost it registers (it runs on 56) and the spills showed up as slow MMAs,
        # so that kernel reports the thread's total only
        issuer = ["total"] + [""] * 7 if which == "fwd3" else ["total", "wait V(t)", "wait P0(t)", "issue PV0(t)", "wait K(t+1)",
                                                               "issue S0(t+1)", "wait P1(t)", "issue PV1(t), S1(t+1)"]
        for role, label, names in (
                (0, "issuer", issuer),
                (2, "softmax g0", ["total", "wait S", "row max", "rescale", "exp + store P", "store wait, arrive", "", ""]),
                (3, "softmax g1", ["total", "wait S", "row max", "rescale", "exp + store P", "store wait, arrive", "", ""])):
            row = p[role * 8: role * 8 + 8].tolist()
            print("   %-11s" % label, "  ".join(f"{n}={v / nt:.0f}" for n, v in zip(names, row) if n))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--T", type=int, default=32768)
    ap.add_argument("--H", type=int, default=8)
    ap.add_argument("--window", type=int, default=None)
    ap.add_argument("--kernel", choices=("bwd", "fwd2", "fwd3"), default="bwd",
                    help="bwd: the wide backward kernels; fwd2: the forward with two query tiles per CTA; fwd3: the same "
                         "with the register file split between the roles and packed softmax arithmetic")
    a = ap.parse_args()
    if a.kernel in ("fwd2", "fwd3"):
        return fwd2(a)
    T, H, Bsz = a.T, a.H, 1
    W = a.window if a.window is not None else T
    with tempfile.TemporaryDirectory(prefix="arb_prof_") as td:
        so = Path(td) / "attn_prof.so"
        flags = [f for f in B.NVCC_FLAGS if f not in ("-Xptxas", "-v")]
        subprocess.run([B.nvcc_path()] + flags + ["-DARB_ATTN_PROF", "-shared", str(B.CSRC / "attn_wide_sm100.cu"), "-o", str(so)],
                       check=True)
        lib = C.CDLL(str(so))
        Dl = H * 128
        torch.manual_seed(0)
        qkv = torch.randn(Bsz * T, 3 * Dl, device="cuda").to(torch.bfloat16)
        g = torch.randn(Bsz * T, Dl, device="cuda").to(torch.bfloat16)
        dqkv = torch.empty_like(qkv)
        lse = torch.randn(Bsz, H, T, device="cuda").abs() + 8.0   # any finite statistics do: only timing matters
        delta = torch.randn(Bsz, H, T, device="cuda")
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        prof = torch.zeros(64, dtype=torch.int64, device="cuda")
        vp, ll, ci = C.c_void_p, C.c_longlong, C.c_int
        f = lib.arb_attn_prof_wide_bwd
        f.restype = ci
        f.argtypes = [vp] * 9 + [ci, ci, ci, ll, ll, ci, C.c_float, vp, vp]
        b, db = qkv.data_ptr(), dqkv.data_ptr()
        for _ in range(2):
            prof.zero_()
            e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(2))
            e1.record()
            rc = f(b, b + 2 * Dl, b + 4 * Dl, g.data_ptr(), db, db + 2 * Dl, db + 4 * Dl, lse.data_ptr(), delta.data_ptr(), Bsz, T, H,
                   3 * Dl, Dl, W, 1 / math.sqrt(128), err.data_ptr(), prof.data_ptr())
            e2.record()
            torch.cuda.synchronize()
            assert rc == 0 and err.item() == 0, (rc, err.item())
        print(f"B=1 T={T} H={H} window={W}: dQ + dK/dV kernels {e1.elapsed_time(e2):.3f} ms (with the profiling marks)")
        p = prof.cpu()
        nt = (T + 127) // 128 if W >= T else (W // 128 + 2)

        def show(title, roles):
            print(f"{title}: cycles per 128x128 tile, heaviest CTA ({nt} tiles)")
            for role, label, names in roles:
                row = p[role * 8: role * 8 + 8].tolist()
                print("   %-11s" % label, "  ".join(f"{n}={v / nt:.0f}" for n, v in zip(names, row) if n))

        sm_q = ["total", "wait S", "phase A", "wait dP", "phase B", "wait dS buffer", "store dS", ""]
        show("dQ kernel", [(0, "issuer", ["total", "wait A(t), K(t+1)", "issue S(t+1)", "wait B(t), V(t+1)", "issue dP(t+1)", "issue dQ(t)", "", ""]),
                           (2, "softmax w2", sm_q), (3, "softmax w7", sm_q)])
        sm_k = ["total", "stat barrier", "wait S^T", "phase A", "wait dP^T", "phase B", "", ""]
        show("dK/dV kernel", [(4, "issuer", ["total", "wait A(t)", "issue dV(t), S^T(t+1)", "wait B(t)", "issue dK(t), dP^T(t+1)", "", "", ""]),
                              (6, "softmax w2", sm_k), (7, "softmax w7", sm_k)])


if __name__ == "__main__":
    main()
