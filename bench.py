"""Headline benchmark: training tokens/s of the 428 M GPT (D=1024, L=30, T=32768, 524 288
tokens per optimizer step) on N B200s of one node, device-timed, max over ranks.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                     (the reference arm)

Prints ONE JSON line on rank 0.  ``value`` is timed with CUDA events around exactly K
optimizer steps (each step stages its inputs from pinned host memory); ``e2e`` repeats the
K steps through the public ``Trainer.train_step`` API with a wall clock and a device->host
read of the loss every step.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

BASELINE_TOK_S = 52643.0  # reference, 1x H100 SXM, results/480m_30pct_cooldown/train.log
PUBLISHED = {"phase2": 52643.0, "phase1": 349500.0}   # the reference's published tokens/s on 1x H100 SXM


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="sm100", choices=["sm100", "baseline", "reference"],
                    help="sm100: this package's kernels; baseline: the library arm on the same box (cuBLAS GEMMs, cuDNN / "
                         "flash-attn attention, torch elementwise kernels, NCCL with --comm nccl); reference: the reference "
                         "engine itself (unavailable here, prints why)")
    ap.add_argument("--model", default="phase2")
    ap.add_argument("--attn", default=None, choices=[None, "own", "library"])
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--micro-batch", type=int, default=None,
                    help="sequences per GPU and micro-step; default 4 (64 for phase1, the reference's batch for that model)")
    ap.add_argument("--total-batch", type=int, default=524288)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel group size (world = tp x dp); dense models")
    ap.add_argument("--ep", type=int, default=1, help="expert-parallel group size (MoE models; 1 or the world size)")
    ap.add_argument("--pp", type=int, default=1, help="pipeline stages (world = pp x dp); one process per stage, 1F1B")
    ap.add_argument("--dp-buckets", type=int, default=3,
                    help="gradient buckets of the fused data-parallel exchange (1 = exchange after the backward pass)")
    ap.add_argument("--layers", type=int, default=None, help="debug only: marks the result invalid")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust crate (no setup.py/pyproject at its root, pip refuses it; "
                          "no cargo/rustc in the image) linking a Hopper-only (sm_90a) FlashAttention-3 "
                          "build that needs a network clone"}))
        return 0

    import torch
    import torch.distributed as dist
    from autoresearch_b200.config import ParallelConfig, ScheduleConfig, TrainConfig, model_preset
    from autoresearch_b200.ops import kernels as K
    from autoresearch_b200.trainer import Trainer
    from autoresearch_b200.utils.clocks import ClockSampler

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(f"bench.py --gpus {args.gpus} must be launched by torch.distributed.run", file=sys.stderr)
            return 2
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    over = {}
    if args.seq_len:
        over["seq_len"] = args.seq_len
    if args.layers:
        over["n_layer"] = args.layers
    mcfg = model_preset(args.model, **over)
    sched = ScheduleConfig(peak_lr=0.02, weight_decay=0.3, final_lr_frac=0.02,
                           embedding_lr=0.45, unembedding_lr=0.0025, scalar_lr=0.25)
    if args.micro_batch is None:
        args.micro_batch = 64 if args.model == "phase1" else 4
        if args.impl == "baseline" and args.model != "phase1":
            args.micro_batch = 2   # the library arm keeps every autograd intermediate: 4 x 32768 tokens do not fit
    # MFU denominator: the pool's measured cuBLAS bf16 burst rate when the driver's record is beside this file
    peak, peak_kind = 1.59e15, "fallback"
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as f:
            peak, peak_kind = float(json.load(f)["bf16_tflops"]) * 1e12, "measured"
    except Exception:
        pass
    model_par = max(1, args.tp) * max(1, args.pp)
    tcfg = TrainConfig(device_batch_size=args.micro_batch, total_batch_size=args.total_batch,
                       max_steps=1000, cooldown_steps=300, synthetic_data=True, synthetic_kind="zipf",
                       impl=args.impl, schedule_cfg=sched, cooldown_trigger_file="", peak_flops=peak,
                       parallel=ParallelConfig(dp=world // model_par, tp=args.tp, ep=args.ep, pp=args.pp, comm=args.comm,
                                               dp_buckets=args.dp_buckets))
    if args.tp > 1:
        from autoresearch_b200.parallel.tp import TPTrainer
        tr = TPTrainer(mcfg, tcfg, tp=args.tp, device=f"cuda:{local}", quiet=True)
        comm_name = tr.comm_name
    elif args.pp > 1:
        from autoresearch_b200.parallel.pipeline import PipelineTrainer
        tr = PipelineTrainer(mcfg, tcfg, pp=args.pp, device=f"cuda:{local}", quiet=True)
        comm_name = f"pp-nccl-p2p+dp-{tr.comm.name}"
    else:
        tr = Trainer(mcfg, tcfg, device=f"cuda:{local}", quiet=True)
        comm_name = tr.comm.name
    if args.attn and hasattr(tr.backend, "attn"):
        tr.backend.attn = args.attn

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        tr.train_step()
    sync()
    # ---- device-timed region ---------------------------------------------------------------
    sampler = ClockSampler(local).start()
    n0 = K.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = tr.train_step()
    e1.record()
    sync()
    launches = K.launch_count - n0
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    # ---- end-to-end region (public API, loss read back every step) ------------------------------
    sync()
    t0 = time.perf_counter()
    last = None
    for _ in range(args.steps):
        last = tr.global_loss(tr.train_step()) if model_par > 1 else float(tr.train_step().item())
    sync()
    e2e_s = time.perf_counter() - t0
    K.check_err_flag()
    if world > 1:
        t = torch.tensor([ms, e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0].item()), float(t[1].item())
    tokens_step = tr.tokens_per_step
    value = tokens_step * args.steps / (ms / 1e3)
    e2e = tokens_step * args.steps / e2e_s
    valid = args.layers is None and args.seq_len is None and args.model == "phase2" and args.total_batch == 524288
    published = PUBLISHED.get(args.model) if (args.layers is None and args.seq_len is None and args.total_batch == 524288) else None
    out = {
        "metric": ("train tokens/sec, 428M D1024 L30 T32K (device-timed, max/rank)" if args.model == "phase2"
                   else f"train tokens/sec, {args.model} (device-timed, max/rank)"),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 2), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": (round(value / published, 3) if world == 1 and published else None),
        "dtype": "bf16", "data": "synthetic Zipf(1.1) token ids from a seed; random-init weights",
        "impl": args.impl,
        "config": {"model": f"{mcfg.name} {mcfg.num_params()['total'] / 1e6:.1f}M D{mcfg.d_model} L{mcfg.n_layer} T{mcfg.seq_len}",
                   "global_batch": tokens_step, "seq_len": mcfg.seq_len,
                   "micro_batch_per_gpu": tr.micro_batch, "grad_accum": tr.accum,
                   "parallelism": (f"tp{args.tp}xdp{world // args.tp}" if args.tp > 1 else
                                   (f"pp{args.pp}xdp{world // args.pp}" if args.pp > 1 else
                                    (f"dp{world} ep{args.ep}" if args.ep > 1 else f"dp{world}"))), "comm": comm_name,
                   "attention": (getattr(tr.backend, "attn", None) or
                                 "library: " + json.dumps(getattr(tr.backend, "attention_used", {}))),
                   "dp_buckets": getattr(tr, "n_buckets", 1),
                   "l2": "inputs larger than L2 (per-step working set of tens of GB)",
                   "valid_headline_config": valid},
        "clocks": {k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": tr.h2d_bytes_per_step,
                "d2h_bytes_per_step": 4, "last_loss": last},
        "gpu_launches": launches,
        f"mfu_vs_{peak_kind}_peak": round(mcfg.flops_per_token() * value / (peak * world), 4),
    }
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
