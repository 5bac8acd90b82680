"""Data-parallel gradient / parameter exchange: this package's peer-memory kernels against NCCL, with the achieved
fraction of the NVLink rate.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m autoresearch_b200.bench.dp_comm_bench --numel 427819008

``numel`` is the size of the flat bf16 gradient bucket (default: the 428 M-parameter headline model).  Timed per
rank with CUDA events, max over ranks:

* reduce-scatter of the bf16 buckets into the owner's fp32 shard: plain peer loads, ``multimem.ld_reduce`` (NVSwitch),
  ``ncclReduceScatter`` (+ cast, which the own kernels include);
* the same reduction fused into the first optimizer kernel (AdamW over the whole shard): fused kernel vs unfused
  AdamW alone - the difference is what the exchange costs when it rides on the optimizer pass;
* all-gather of the updated bf16 shard: peer pull kernel vs ``ncclAllGather``.

The link roofline of every line is (world-1)/world x bucket bytes / 770 GB/s per direction and GPU.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--numel", type=int, default=427819008)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from ..ops import kernels as K
    from ..parallel.symm import SymmBuffer
    rank, world = dist.get_rank(), dist.get_world_size()
    shard = (a.numel + world - 1) // world
    shard = (shard + 255) // 256 * 256
    total = shard * world
    bucket = SymmBuffer(total, torch.bfloat16, dev)
    param = SymmBuffer(total, torch.bfloat16, dev)
    flags = SymmBuffer(64, torch.int32, dev)
    for b in (bucket, param, flags):
        b.rendezvous()
    bucket.tensor.copy_(torch.randn(total, device=dev) * 0.01)
    dist.barrier()
    L = K.lib()
    st = K._stream()
    ptrs_b = (C.c_void_p * (world + 1))(*(bucket.peer_ptrs + [rank]))
    ptrs_plain = (C.c_void_p * world)(*bucket.peer_ptrs)
    ptrs_p = (C.c_void_p * world)(*param.peer_ptrs)
    fl = (C.c_void_p * world)(*flags.peer_ptrs)
    mc = bucket.multicast_ptr
    out32 = torch.empty(shard, dtype=torch.float32, device=dev)
    master = torch.zeros(shard, dtype=torch.float32, device=dev)
    m1 = torch.zeros_like(master); v1 = torch.zeros_like(master)
    shadow = param.tensor[rank * shard:(rank + 1) * shard]
    epoch = [0]

    def barrier():
        epoch[0] += 1
        K._check(L.arb_peer_barrier(fl, world, rank, epoch[0], K.err_flag(dev).data_ptr(), st), "barrier")

    def timed(fn):
        for _ in range(2):
            fn()
        barrier(); torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    res = {}
    res["rs_peer_loads_ms"] = timed(lambda: K._check(L.arb_reduce_scatter_peers(ptrs_b, world, rank * shard, shard, 1, out32.data_ptr(), 1.0, st), "rs"))
    if mc:
        res["rs_multimem_ms"] = timed(lambda: K._check(L.arb_reduce_scatter_multimem(mc, rank * shard, shard, 1, out32.data_ptr(), 1.0, st), "rs_mc"))
    nccl_out = torch.empty(shard, dtype=torch.bfloat16, device=dev)

    def nccl_rs():
        dist.reduce_scatter_tensor(nccl_out, bucket.tensor)
        out32.copy_(nccl_out)
    res["rs_nccl_plus_cast_ms"] = timed(nccl_rs)
    adam = lambda fused: K._check(
        L.arb_adamw_rs(master.data_ptr(), ptrs_plain, world, rank, mc if (mc and fused == 2) else 0, rank * shard, 1.0,
                       m1.data_ptr(), v1.data_ptr(), shadow.data_ptr(), shard, 1e-3, 0.9, 0.95, 1e-8, 0.0, 0.1, 0.05, st), "adamw_rs")
    res["adamw_fused_with_rs_peer_ms"] = timed(lambda: adam(1))
    if mc:
        res["adamw_fused_with_rs_multimem_ms"] = timed(lambda: adam(2))
    grad = out32
    res["adamw_alone_ms"] = timed(lambda: K._check(
        L.arb_adamw(master.data_ptr(), grad.data_ptr(), m1.data_ptr(), v1.data_ptr(), shadow.data_ptr(), shard, 1e-3, 0.9, 0.95,
                    1e-8, 0.0, 0.1, 0.05, st), "adamw"))
    local_copy = torch.empty(total, dtype=torch.bfloat16, device=dev)
    res["ag_peer_pull_ms"] = timed(lambda: K._check(L.arb_all_gather_pull(ptrs_p, world, rank, local_copy.data_ptr(), shard * 2, st), "ag"))
    res["ag_nccl_ms"] = timed(lambda: dist.all_gather_into_tensor(local_copy, shadow))
    K.check_err_flag()
    link_ms = (world - 1) * shard * 2 / (a.link_gbs * 1e9) * 1e3
    if rank == 0:
        out = {"world": world, "bucket_mb": round(total * 2 / 1e6, 1), "remote_mb_per_rank": round((world - 1) * shard * 2 / 1e6, 1),
               "link_roofline_ms": round(link_ms, 4)}
        out.update({k: round(v, 4) for k, v in res.items()})
        out["fraction_of_link"] = {k[:-3]: round(link_ms / v, 3) for k, v in res.items() if k.startswith(("rs_", "ag_"))}
        if "adamw_alone_ms" in res:
            out["rs_cost_when_fused_ms"] = round(res["adamw_fused_with_rs_" + ("multimem" if mc else "peer") + "_ms"] - res["adamw_alone_ms"], 4)
        print(json.dumps(out))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
