"""Command line: ``python -m autoresearch_b200 [train] [flags]``.

Flags and environment variables are the reference binary's (brain/src/main.rs:6-141):
``--load-checkpoint P --diagnostic N --data-dir D --tokenizer-path|--tokenizer-dir D
--stream-input --distributed --max-steps N --synthetic-data true|1 --pipeline N`` and the legacy
positional ``train``; unknown flags are ignored like there.  ``--max-steps`` beats ``MAX_STEPS``.
Environment: ``SYNTHETIC MAX_STEPS COOLDOWN_STEPS BATCH_SIZE NUM_TRAIN_SHARDS TOTAL_BATCH PEAK_LR
WARMDOWN_RATIO WARMUP_RATIO WEIGHT_DECAY SCHEDULE FINAL_LR_FRAC CHECKPOINT_DIR EVAL_EVERY
CHECKPOINT_EVERY INIT_WEIGHTS_PATH PIPELINE_RANK PIPELINE_WORLD_SIZE``.

Additions (the reference fixes these at compile time): ``--model PRESET`` (or ``MODEL``),
``--impl oracle|baseline|sm100|auto``, ``--synthetic-kind lcg|zipf``, ``--comm fused|nccl``,
``--metrics-jsonl PATH``, ``--resume``, ``--tp N``, ``--ep N`` (expert parallel over the DP ranks).  Under ``torchrun`` the ranks form a
data-parallel group (times ``--pipeline`` stages, times ``--tp``).
"""
from __future__ import annotations

import os
import sys
from typing import List, Optional

from .config import PRESETS, ScheduleConfig, TrainConfig, model_preset


def parse_args(argv: List[str], env=None):
    env = os.environ if env is None else env
    t = TrainConfig.from_env(env)
    model = env.get("MODEL", "phase1")
    max_steps_cli: Optional[int] = None
    tp = 1
    i = 0
    n = len(argv)

    def val():
        nonlocal i
        i += 1
        if i >= n:
            raise SystemExit(f"{argv[i - 1]} expects a value")
        return argv[i]

    while i < n:
        a = argv[i]
        if a == "--load-checkpoint": t.load_checkpoint = val()
        elif a == "--diagnostic": t.diagnostic_steps = int(val())
        elif a == "--data-dir": t.data_dir = val()
        elif a in ("--tokenizer-path", "--tokenizer-dir"): t.tokenizer_dir = val()
        elif a == "--stream-input": t.stream_input = True
        elif a == "--distributed": t.distributed = True
        elif a == "--max-steps": max_steps_cli = int(val())
        elif a == "--synthetic-data": t.synthetic_data = val() in ("true", "1") or t.synthetic_data
        elif a == "--pipeline": t.n_pipeline_stages = int(val())
        elif a == "--model": model = val()
        elif a == "--impl": t.impl = val()
        elif a == "--synthetic-kind": t.synthetic_kind = val()
        elif a == "--comm": t.parallel.comm = val()
        elif a == "--metrics-jsonl": t.metrics_jsonl = val()
        elif a == "--resume": t.resume = True
        elif a == "--tp": tp = int(val())
        elif a == "--ep": t.parallel.ep = int(val())
        elif a == "train": pass
        i += 1
    if max_steps_cli is not None:
        t.max_steps = max_steps_cli
    if model not in PRESETS:
        raise SystemExit(f"unknown --model {model!r}; choose from {', '.join(PRESETS)}")
    t.parallel.tp = tp
    t.parallel.pp = t.n_pipeline_stages
    return model_preset(model), t


def banner(mcfg, t: TrainConfig) -> str:
    s = t.schedule_cfg
    d = ScheduleConfig()
    lines = ["autoresearch-brain"]
    if t.synthetic_data:
        lines.append("  mode:           SYNTHETIC (MFU baseline — no real data)")
    lines.append(f"  max_steps:      {t.max_steps if t.max_steps else '∞'}")
    lines.append(f"  cooldown_steps: {t.cooldown_steps}")
    acc = max(t.total_batch_size // (t.device_batch_size * mcfg.seq_len), 1)
    lines.append(f"  batch:          {t.device_batch_size}x{acc} = {t.total_batch_size} tokens/step")
    lines.append(f"  data:           {t.data_dir}")
    lines.append(f"  peak_lr:        {s.peak_lr}")
    lines.append(f"  warmdown_ratio: {s.warmdown_ratio} (cooldown shape only)")
    lines.append(f"  weight_decay:   {s.weight_decay}")
    lines.append(f"  schedule:       {s.schedule}")
    lines.append(f"  final_lr_frac:  {s.final_lr_frac}")
    scale = s.peak_lr / d.peak_lr
    if scale != 1.0:
        lines.append(f"  (LRs scaled {scale}x: emb={s.embedding_lr:.4f} unemb={s.unembedding_lr:.6f} scalar={s.scalar_lr:.4f})")
    if t.num_train_shards is not None:
        lines.append(f"  train/val split: {t.num_train_shards} train shards, rest = val")
    lines.append(f"  pipeline_stages: {t.n_pipeline_stages}")
    lines.append(f"  model:          {mcfg.name} (D={mcfg.d_model} L={mcfg.n_layer} T={mcfg.seq_len} V={mcfg.vocab})")
    return "\n".join(lines)


def main(argv: Optional[List[str]] = None) -> int:
    import torch
    import torch.distributed as dist
    argv = sys.argv[1:] if argv is None else argv
    mcfg, t = parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", os.environ.get("PIPELINE_WORLD_SIZE", "1")))
    rank = int(os.environ.get("RANK", os.environ.get("PIPELINE_RANK", "0")))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    on_gpu = torch.cuda.is_available()
    if on_gpu:
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        os.environ.setdefault("RANK", str(rank))
        os.environ.setdefault("WORLD_SIZE", str(world))
        dist.init_process_group("nccl" if on_gpu else "gloo")
    if rank == 0:
        print(banner(mcfg, t), flush=True)
    device = f"cuda:{local}" if on_gpu else "cpu"
    pp = max(t.n_pipeline_stages, 1)
    if t.distributed and pp == 1:
        pp = world  # the reference's --distributed mode: every rank is a pipeline stage
    if pp > 1 and world == 1:
        # `--pipeline N` in a single process: this process drives N GPUs (brain/src/main.rs:126-134 -> train_pipeline)
        from .parallel.pipeline_inproc import InProcPipelineTrainer
        n_dev = torch.cuda.device_count() if on_gpu else 0
        if on_gpu and n_dev < pp:
            raise SystemExit(f"--pipeline {pp} needs {pp} GPUs in this process, {n_dev} visible")
        devices = [f"cuda:{i}" for i in range(pp)] if on_gpu else ["cpu"] * pp
        print(f"Launching {pp}-stage pipeline training...", flush=True)
        InProcPipelineTrainer(mcfg, t, devices).run()
    elif pp > 1:
        # one process per stage (launched by torchrun, or with PIPELINE_RANK / PIPELINE_WORLD_SIZE as in
        # brain/src/train.rs:1623-1632); world = pp x dp
        from .parallel.pipeline import PipelineTrainer
        if rank == 0:
            print(f"Launching {pp}-stage pipeline training...", flush=True)
        PipelineTrainer(mcfg, t, pp=pp, device=device).run()
    elif t.parallel.tp > 1:
        from .parallel.tp import TPTrainer
        TPTrainer(mcfg, t, tp=t.parallel.tp, device=device).run()
    else:
        from .trainer import Trainer
        t.parallel.dp = world
        Trainer(mcfg, t, device=device).run()
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0
