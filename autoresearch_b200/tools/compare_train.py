"""Parity trainer: run implementations (the fp32 oracle, the library arm, the sm_100a kernels) from the same
initial weights on the same token stream with the same WSD schedule, write one CSV row per step and report the
loss deviation (role of brain/tools/compare_train.py:58-807, whose per-step CSV and proxy evaluation are compared
with the engine log by hand).

    python -m autoresearch_b200.tools.compare_train --model small --a oracle --b sm100 --max-steps 50
    python -m autoresearch_b200.tools.compare_train --model phase1 --a baseline --b sm100 --max-steps 1000 \\
        --cooldown-steps 500 --batch 64 --total-batch 131072 --csv steps.csv --report parity.md
    feeder ... | python -m autoresearch_b200.tools.compare_train --stream-input --init-weights init.safetensors ...

Like the reference tool it takes ``--init-weights`` (a safetensors file in engine or Python names, see
tools/generate_init_weights.py), ``--stream-input`` (rows of SEQ+1 little-endian u16 on stdin, as written by the
feeder: the rows are read once and replayed to every implementation), ``--max-steps`` / ``--cooldown-steps``
(step-based WSD identical to the engine's) and evaluates a proxy bits-per-byte every ``--eval-every`` steps on
``--eval-batches`` held-out batches of the same source.  One implementation alone (``--b none``) gives the per-step
CSV to lay beside another engine's log.
"""
from __future__ import annotations

import argparse
import csv
import math
import sys
from typing import List, Optional

import numpy as np
import torch

from ..config import ScheduleConfig, TrainConfig, model_preset
from ..trainer import Trainer


class _ReplayLoader:
    """Batches cut from rows held in memory; every implementation replays the same sequence."""

    def __init__(self, rows: np.ndarray, B: int, T: int):
        self.rows, self.B, self.T, self.pos = rows, B, T, 0

    def next_batch(self, ids_out=None, tgt_out=None):
        if self.pos + self.B > self.rows.shape[0]:
            return None
        t = torch.from_numpy(self.rows[self.pos:self.pos + self.B].astype(np.int32))
        self.pos += self.B
        ids, tgt = t[:, :-1], t[:, 1:]
        if ids_out is not None:
            ids_out.copy_(ids); tgt_out.copy_(tgt)
            return ids_out, tgt_out
        return ids.contiguous(), tgt.contiguous()

    def state_dict(self):
        return {"pos": self.pos}

    def load_state_dict(self, d):
        self.pos = int(d["pos"])


def read_rows(stream, seq_len: int, max_rows: Optional[int]) -> np.ndarray:
    """Rows of seq_len+1 u16 from a binary stream until EOF or max_rows."""
    row_bytes = 2 * (seq_len + 1)
    chunks, n = [], 0
    while max_rows is None or n < max_rows:
        buf = stream.read(row_bytes)
        if len(buf) < row_bytes:
            break
        chunks.append(np.frombuffer(buf, dtype="<u2"))
        n += 1
    if not chunks:
        raise SystemExit("--stream-input: no complete row on stdin")
    return np.stack(chunks)


def _proxy_bpb(tr: Trainer, batches, token_bytes: Optional[torch.Tensor]) -> float:
    """Mean loss in bits per byte over fixed held-out batches (bits per token when no byte table is given)."""
    nats = by = 0.0
    was = tr.model.training
    tr.model.eval()
    with torch.no_grad():
        for ids, tgt in batches:
            ids, tgt = ids.to(tr.device), tgt.to(tr.device)
            _, per_tok = tr.model(ids, tgt)
            if token_bytes is None:
                nats += float(per_tok.double().sum()); by += per_tok.numel()
            else:
                b = token_bytes[tgt.reshape(-1).long()]
                nats += float((per_tok.double() * (b > 0)).sum()); by += float(b.double().sum())
    tr.model.train(was)
    return nats / (math.log(2.0) * by) if by > 0 else float("nan")


def run(model: str, impl_a: str, impl_b: Optional[str], steps: int, batch: int, csv_path: str = None, device: str = None,
        cooldown: int = None, total_batch: int = None, init_weights: str = None, rows: np.ndarray = None,
        eval_every: int = 0, eval_batches: int = 4, tokenizer_dir: str = None, peak_lr: float = None,
        weight_decay: float = None, final_lr_frac: float = None, seed: int = 42, layers: int = None):
    over = {"n_layer": layers} if layers else {}
    cfg = model_preset(model, **over)
    impls = [impl_a] + ([impl_b] if impl_b and impl_b != "none" else [])
    sched = ScheduleConfig()
    if peak_lr is not None:                       # derived learning rates follow PEAK_LR like the CLI (brain/src/main.rs:68-79)
        sched = ScheduleConfig.from_env({"PEAK_LR": str(peak_lr)})
    if weight_decay is not None:
        sched.weight_decay = weight_decay
    if final_lr_frac is not None:
        sched.final_lr_frac = final_lr_frac
    out = {}
    for impl in impls:
        t = TrainConfig(device_batch_size=batch, total_batch_size=total_batch or batch * cfg.seq_len, max_steps=steps,
                        cooldown_steps=cooldown if cooldown is not None else max(steps // 3, 1), synthetic_data=True,
                        synthetic_kind="zipf", impl=impl, cooldown_trigger_file="", init_weights_path=init_weights,
                        schedule_cfg=sched, seed=seed)
        dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
        tr = Trainer(cfg, t, device=dev, quiet=True)
        held = []
        if rows is not None:                      # replay the streamed rows; the tail is held out for the proxy evaluation
            n_eval = eval_batches * tr.micro_batch if eval_every else 0
            train_rows = rows[:rows.shape[0] - n_eval] if n_eval else rows
            tr.prefetch.close()
            tr.train_loader = _ReplayLoader(train_rows, tr.micro_batch, cfg.seq_len)
            from ..data.prefetch import PinnedPrefetcher
            tr.prefetch = PinnedPrefetcher(tr.train_loader, tr.micro_batch, cfg.seq_len, depth=tr.accum + 1,
                                           pin=tr.device.type == "cuda")
            ev = _ReplayLoader(rows[rows.shape[0] - n_eval:], tr.micro_batch, cfg.seq_len) if n_eval else None
        else:
            ev = tr._make_loader("val") if eval_every else None
        if ev is not None:
            for _ in range(eval_batches):
                b = ev.next_batch()
                if b is None:
                    break
                held.append((b[0].clone(), b[1].clone()))
        tb = None
        if tokenizer_dir:
            from ..eval.bpb import load_token_bytes
            tb = load_token_bytes(tokenizer_dir, cfg.vocab, tr.device)
        losses: List[float] = []
        evals = {}
        for s in range(steps):
            l = tr.train_step()
            if l is None:
                break
            losses.append(float(l))
            if eval_every and held and (s + 1) % eval_every == 0:
                evals[s] = _proxy_bpb(tr, held, tb)
        tr.prefetch.close()
        out[impl] = (losses, evals)
        del tr
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
    a = out[impls[0]][0]
    b = out[impls[1]][0] if len(impls) > 1 else None
    n = min(len(a), len(b)) if b is not None else len(a)
    rel = [abs(x - y) / max(abs(x), 1e-9) for x, y in zip(a[:n], b[:n])] if b is not None else []
    if csv_path:
        with open(csv_path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["step"] + [f"loss_{i}" for i in impls] + (["rel_diff"] if b is not None else []) +
                       [f"val_bpb_{i}" for i in impls])
            for i in range(n):
                row = [i] + [f"{out[k][0][i]:.6f}" for k in impls] + ([f"{rel[i]:.6f}"] if b is not None else [])
                row += [(f"{out[k][1][i]:.5f}" if i in out[k][1] else "") for k in impls]
                w.writerow(row)
    res = {"steps": n, "final_a": a[n - 1] if n else None, "impls": impls,
           "evals": {k: out[k][1] for k in impls}, "losses": {k: out[k][0] for k in impls}}
    if b is not None and n:
        # EMA(0.9) with bias correction, the quantity the engines log (brain/src/train.rs:1014-1022)
        def ema(xs):
            e = 0.0
            for j, x in enumerate(xs):
                e = 0.9 * e + 0.1 * x
            return e / (1 - 0.9 ** len(xs))
        res.update(max_rel=max(rel), final_rel=rel[-1], final_b=b[n - 1], ema_a=ema(a[:n]), ema_b=ema(b[:n]),
                   ema_rel=abs(ema(a[:n]) - ema(b[:n])) / ema(a[:n]))
    return res


def write_report(res: dict, path: str, title: str, cmd: str) -> None:
    a, b = res["impls"][0], res["impls"][1]
    la, lb = res["losses"][a], res["losses"][b]
    n = res["steps"]
    marks = sorted(set([0, 1, 2, 5, 10, 25, 50, 100, 200, 300, 500, 700, 900, n - 1]) & set(range(n)))
    lines = [f"# {title}", "", f"command: `{cmd}`", "",
             f"{n} steps; loss of the step (not smoothed) unless stated.", "",
             f"| step | {a} | {b} | relative difference |", "|---|---|---|---|"]
    for s in marks:
        lines.append(f"| {s} | {la[s]:.4f} | {lb[s]:.4f} | {abs(la[s] - lb[s]) / max(abs(la[s]), 1e-9) * 100:.3f} % |")
    lines += ["", f"EMA(0.9) loss at the last step: {a} {res['ema_a']:.4f}, {b} {res['ema_b']:.4f} "
                  f"(difference {res['ema_rel'] * 100:.3f} %); largest single-step difference {res['max_rel'] * 100:.3f} %."]
    for k in res["impls"]:
        if res["evals"][k]:
            lines.append(f"proxy evaluation ({k}): " + ", ".join(f"step {s}: {v:.4f}" for s, v in sorted(res["evals"][k].items())))
    open(path, "w").write("\n".join(lines) + "\n")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="small")
    ap.add_argument("--a", default="oracle")
    ap.add_argument("--b", default="sm100", help="second implementation, or 'none'")
    ap.add_argument("--max-steps", "--steps", dest="steps", type=int, default=50)
    ap.add_argument("--cooldown-steps", type=int, default=None)
    ap.add_argument("--batch", type=int, default=4, help="sequences per micro-step")
    ap.add_argument("--total-batch", type=int, default=None, help="tokens per optimizer step (default: one micro-step)")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--init-weights", default=None)
    ap.add_argument("--stream-input", action="store_true")
    ap.add_argument("--eval-every", type=int, default=0)
    ap.add_argument("--eval-batches", type=int, default=4)
    ap.add_argument("--tokenizer-dir", default=None, help="directory with token_bytes.json (bits per byte instead of per token)")
    ap.add_argument("--peak-lr", type=float, default=None)
    ap.add_argument("--weight-decay", type=float, default=None)
    ap.add_argument("--final-lr-frac", type=float, default=None)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--csv", default=None)
    ap.add_argument("--report", default=None, help="write a Markdown summary table here")
    a = ap.parse_args(argv)
    rows = None
    if a.stream_input:
        cfg = model_preset(a.model)
        per_step = (a.total_batch or a.batch * cfg.seq_len) // cfg.seq_len
        rows = read_rows(sys.stdin.buffer, cfg.seq_len, a.steps * per_step + a.eval_batches * a.batch)
    res = run(a.model, a.a, a.b, a.steps, a.batch, a.csv, cooldown=a.cooldown_steps, total_batch=a.total_batch,
              init_weights=a.init_weights, rows=rows, eval_every=a.eval_every, eval_batches=a.eval_batches,
              tokenizer_dir=a.tokenizer_dir, peak_lr=a.peak_lr, weight_decay=a.weight_decay,
              final_lr_frac=a.final_lr_frac, seed=a.seed, layers=a.layers)
    if a.report and len(res["impls"]) > 1:
        write_report(res, a.report, f"Loss parity, {a.model}: {a.a} vs {a.b}",
                     "python -m autoresearch_b200.tools.compare_train " + " ".join(argv if argv is not None else sys.argv[1:]))
    print({k: v for k, v in res.items() if k not in ("losses", "evals")})
    return res


if __name__ == "__main__":
    main()
