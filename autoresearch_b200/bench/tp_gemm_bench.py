"""Times the two fused tensor-parallel GEMM forms against their NCCL + GEMM baselines and reports the
achieved fraction of the roofline (the slower of FLOPs / measured GEMM peak and NVLink bytes / link rate).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m autoresearch_b200.bench.tp_gemm_bench --rows 16384 --d-model 2048 --cols 8192

``rows`` is the token count of one micro-batch of the TP group, ``cols`` the width of the column-parallel
weight before sharding (3*D for QKV, mlp_dim for FC1).  Device-timed with CUDA events, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--cols", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--peak-tflops", type=float, default=None, help="GEMM peak for the roofline (default: measured file)")
    ap.add_argument("--link-gbs", type=float, default=770.0, help="NVLink rate per direction per GPU")
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from ..ops import kernels as K
    from ..parallel.tp import FusedTPContext, TPContext
    from ..utils.timing import measured_peak_flops
    rank, size = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", local)
    N, D, Cw = a.rows, a.d_model, a.cols // size
    n = N // size
    peak = (a.peak_tflops * 1e12) if a.peak_tflops else measured_peak_flops()
    fused = FusedTPContext(dist.group.WORLD, rank, size, dev, N, D)
    lib = TPContext(dist.group.WORLD, rank, size)
    torch.manual_seed(rank)
    x_shard = torch.randn(n, D, device=dev).to(torch.bfloat16)
    w_col = (torch.randn(Cw, D, device=dev) * 0.02).to(torch.bfloat16)      # column-parallel weight shard [C/tp, D]
    act = torch.randn(N, Cw, device=dev).to(torch.bfloat16)
    w_row = (torch.randn(D, Cw, device=dev) * 0.02).to(torch.bfloat16)      # row-parallel weight shard [D, C/tp]

    def timed(fn):
        for _ in range(3):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # numerics of the fused forms against the library forms
    y_f, _ = fused.ag_gemm(x_shard, w_col)
    y_l = K.gemm(lib.all_gather_rows(x_shard), w_col)
    r_f = fused.gemm_rs(act, w_row)
    r_l = lib.reduce_scatter_rows(K.gemm(act, w_row))
    torch.cuda.synchronize()
    err_ag = ((y_f.float() - y_l.float()).norm() / y_l.float().norm()).item()
    err_rs = ((r_f.float() - r_l.float()).norm() / r_l.float().norm()).item()

    t_ag_f = timed(lambda: fused.ag_gemm(x_shard, w_col))
    t_ag_l = timed(lambda: K.gemm(lib.all_gather_rows(x_shard), w_col))
    t_rs_f = timed(lambda: fused.gemm_rs(act, w_row))
    t_rs_l = timed(lambda: lib.reduce_scatter_rows(K.gemm(act, w_row)))
    x_full = lib.all_gather_rows(x_shard)
    t_gemm_col = timed(lambda: K.gemm(x_full, w_col))
    t_gemm_row = timed(lambda: K.gemm(act, w_row))
    K.check_err_flag()
    flops = 2.0 * N * D * Cw
    bytes_link = (size - 1) * n * D * 2            # received (AG) or sent (RS) per rank, bf16
    roof_ms = max(flops / peak, bytes_link / (a.link_gbs * 1e9)) * 1e3
    if rank == 0:
        print(json.dumps({
            "tp": size, "rows": N, "d_model": D, "cols_per_rank": Cw,
            "roofline_ms": round(roof_ms, 4), "compute_ms_at_peak": round(flops / peak * 1e3, 4),
            "link_ms": round(bytes_link / (a.link_gbs * 1e9) * 1e3, 4),
            "gemm_only_ms": {"column": round(t_gemm_col, 4), "row": round(t_gemm_row, 4)},
            "ag_gemm_ms": {"fused": round(t_ag_f, 4), "nccl_then_gemm": round(t_ag_l, 4),
                           "fused_fraction_of_roofline": round(roof_ms / t_ag_f, 3)},
            "gemm_rs_ms": {"fused": round(t_rs_f, 4), "gemm_then_nccl": round(t_rs_l, 4),
                           "fused_fraction_of_roofline": round(roof_ms / t_rs_f, 3)},
            "rel_err_vs_library": {"ag_gemm": err_ag, "gemm_rs": err_rs}}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
