"""Parity trainer: run two implementations (e.g. the fp32 oracle and the sm_100a kernels) from the
same initial weights on the same token stream with the same schedule, write one CSV row per step
and report the largest relative loss deviation (role of brain/tools/compare_train.py:58-807,
whose per-step CSV is compared with the engine log by hand).

    python -m autoresearch_b200.tools.compare_train --model small --a oracle --b sm100 --steps 50
"""
from __future__ import annotations

import argparse
import csv

import torch

from ..config import TrainConfig, model_preset
from ..trainer import Trainer


def run(model: str, impl_a: str, impl_b: str, steps: int, batch: int, csv_path: str = None, device: str = None,
        cooldown: int = None):
    cfg = model_preset(model)
    losses = {}
    for impl in (impl_a, impl_b):
        t = TrainConfig(device_batch_size=batch, total_batch_size=batch * cfg.seq_len, max_steps=steps,
                        cooldown_steps=cooldown if cooldown is not None else max(steps // 3, 1), synthetic_data=True,
                        synthetic_kind="zipf", impl=impl, cooldown_trigger_file="")
        dev = device or ("cuda" if torch.cuda.is_available() and impl != "oracle_cpu" else "cpu")
        tr = Trainer(cfg, t, device=dev, quiet=True)
        losses[impl] = [float(tr.train_step()) for _ in range(steps)]
    a, b = losses[impl_a], losses[impl_b]
    rel = [abs(x - y) / max(abs(x), 1e-9) for x, y in zip(a, b)]
    if csv_path:
        with open(csv_path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["step", impl_a, impl_b, "rel_diff"])
            for i, (x, y, r) in enumerate(zip(a, b, rel)):
                w.writerow([i, f"{x:.6f}", f"{y:.6f}", f"{r:.6f}"])
    return {"max_rel": max(rel), "final_rel": rel[-1], "final_a": a[-1], "final_b": b[-1]}


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", default="small")
    ap.add_argument("--a", default="oracle")
    ap.add_argument("--b", default="sm100")
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--csv", default=None)
    a = ap.parse_args()
    print(run(a.model, a.a, a.b, a.steps, a.batch, a.csv))


if __name__ == "__main__":
    main()
