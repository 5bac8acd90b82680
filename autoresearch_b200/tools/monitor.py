"""Training-log scraper: step lines, eval lines and crash markers of a run's stdout
(role of hpc/monitor.sh:143-215 and plot_live.sh, which regex the same fields over ssh).

    python -m autoresearch_b200.tools.monitor train.log [--json curve.json] [--follow]
"""
from __future__ import annotations

import argparse
import json
import re
import sys
import time

STEP = re.compile(r"step\s+(\d+) \| loss ([\d.]+) \| lr ([\d.]+) \| dt ([\d.]+)s \| tok/s (\d+) \| mfu ([\d.]+)% \| vram (\d+)MB \| steps_left (-?\d+)")
EVAL = re.compile(r"\[eval\] (?:step (\d+)|final) \| val_bpb ([\d.]+)")
CRASH = re.compile(r"error|panic|nan|Traceback|blew up", re.IGNORECASE)


def parse(lines):
    steps, evals, crashes = [], [], []
    for ln in lines:
        m = STEP.search(ln)
        if m:
            steps.append(dict(step=int(m[1]), loss=float(m[2]), lr=float(m[3]), dt=float(m[4]), tok_s=int(m[5]),
                              mfu=float(m[6]), vram_mb=int(m[7]), steps_left=int(m[8])))
            continue
        m = EVAL.search(ln)
        if m:
            evals.append(dict(step=int(m[1]) if m[1] else None, val_bpb=float(m[2])))
            continue
        if CRASH.search(ln) and not ln.startswith("timing"):
            crashes.append(ln.strip())
    return {"steps": steps, "evals": evals, "crashes": crashes}


def summary(p) -> str:
    s = p["steps"]
    out = []
    if s:
        last = s[-1]
        out.append(f"step {last['step']} loss {last['loss']:.4f} tok/s {last['tok_s']} mfu {last['mfu']:.1f}% steps_left {last['steps_left']}")
    if p["evals"]:
        out.append("val_bpb " + " ".join(f"{e['val_bpb']:.4f}" for e in p["evals"][-5:]))
    if p["crashes"]:
        out.append(f"CRASH MARKERS: {len(p['crashes'])} (first: {p['crashes'][0][:120]})")
    return "\n".join(out) or "no training lines yet"


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("log")
    ap.add_argument("--json", default=None)
    ap.add_argument("--follow", action="store_true")
    ap.add_argument("--interval", type=float, default=30.0)
    a = ap.parse_args()
    while True:
        with open(a.log, errors="replace") as f:
            p = parse(f)
        print(summary(p), flush=True)
        if a.json:
            with open(a.json, "w") as f:
                json.dump(p["evals"], f)
        if not a.follow or p["crashes"] or (p["steps"] and p["steps"][-1]["steps_left"] == 0):
            return 1 if p["crashes"] else 0
        time.sleep(a.interval)


if __name__ == "__main__":
    sys.exit(main())
