"""Run lifecycle on one multi-GPU box: start a training job, watch it, salvage its results, tear it down.

    python -m autoresearch_b200.tools.launch start --gpus 8 --out results/run1 [--budget-hours 6]
            [--cost-per-gpu-hour 2.5] [--notify-cmd 'mail -s "{status}" me'] -- MODEL=phase2 MAX_STEPS=1000 [train flags]
    python -m autoresearch_b200.tools.launch status   --out results/run1
    python -m autoresearch_b200.tools.launch teardown --out results/run1

Role of hpc/deploy.sh, hpc/monitor.sh and hpc/teardown.sh, without their cloud-marketplace part (instance search,
ssh, rsync): the job is a local ``torch.distributed.run`` of ``python -m autoresearch_b200 train``.  What is
kept: a state file (``.deploy_state`` there, ``run_state.json`` here) that ``status`` / ``teardown`` read; the log
scraper and crash detection (tools/monitor.py); a safety watchdog with a wall-clock budget; salvage of log,
metrics and checkpoints into the result folder on every kind of exit; a cost report; a notification hook.
``teardown`` signals exactly the process group recorded in the state file.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import signal
import subprocess
import sys
import threading
import time
from pathlib import Path

from . import monitor


def _state_path(out: Path) -> Path:
    return out / "run_state.json"


def _salvage(out: Path, ckpt_dir: Path) -> list:
    """Copy what a finished or dying run leaves behind into the result folder."""
    kept = []
    if ckpt_dir.is_dir():
        dst = out / "checkpoints"
        for f in sorted(ckpt_dir.rglob("*")):
            if f.is_file():
                rel = f.relative_to(ckpt_dir)
                (dst / rel).parent.mkdir(parents=True, exist_ok=True)
                if not (dst / rel).exists() or (dst / rel).stat().st_mtime < f.stat().st_mtime:
                    shutil.copy2(f, dst / rel)
                kept.append(str(rel))
    return kept


def _report(out: Path, state: dict, status: str, cost_rate: float) -> dict:
    log = out / "train.log"
    parsed = monitor.parse(open(log, errors="replace")) if log.exists() else {"steps": [], "evals": [], "crashes": []}
    hours = (time.time() - state["started"]) / 3600.0
    rep = {"status": status, "hours": round(hours, 3), "gpus": state["gpus"],
           "gpu_hours": round(hours * state["gpus"], 3),
           "cost": round(hours * state["gpus"] * cost_rate, 2) if cost_rate else None,
           "last_step": parsed["steps"][-1] if parsed["steps"] else None,
           "val_bpb": [e["val_bpb"] for e in parsed["evals"]][-5:], "crash_markers": parsed["crashes"][:5]}
    (out / "report.json").write_text(json.dumps(rep, indent=1))
    return rep


def start(a, extra) -> int:
    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    env = dict(os.environ)
    flags = []
    for tok in extra:                      # NAME=value pairs become environment variables, the rest train flags
        if "=" in tok and tok.split("=", 1)[0].isidentifier() and not tok.startswith("-"):
            k, v = tok.split("=", 1)
            env[k] = v
        else:
            flags.append(tok)
    ckpt_dir = Path(env.setdefault("CHECKPOINT_DIR", str(out / "live_checkpoints")))
    env.setdefault("METRICS_JSONL", str(out / "metrics.jsonl"))
    if a.gpus > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(a.port), "-m", "autoresearch_b200", "train"] + flags
    else:
        cmd = [sys.executable, "-m", "autoresearch_b200", "train"] + flags
    log = open(out / "train.log", "ab", buffering=0)
    proc = subprocess.Popen(cmd, env=env, stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
    state = {"pid": proc.pid, "pgid": os.getpgid(proc.pid), "started": time.time(), "gpus": a.gpus, "cmd": cmd,
             "checkpoint_dir": str(ckpt_dir), "budget_hours": a.budget_hours}
    _state_path(out).write_text(json.dumps(state, indent=1))
    print(f"started pid {proc.pid} (process group {state['pgid']}); log {out / 'train.log'}", flush=True)
    status = {"v": "finished"}
    stop = threading.Event()

    def watchdog():
        while not stop.wait(a.poll_seconds):
            with open(out / "train.log", errors="replace") as f:
                p = monitor.parse(f)
            if p["crashes"]:
                status["v"] = "crashed"
            elif a.budget_hours and time.time() - state["started"] > a.budget_hours * 3600:
                status["v"] = "over budget"
            else:
                continue
            try:
                os.killpg(state["pgid"], signal.SIGTERM)
            except ProcessLookupError:
                pass
            return

    th = threading.Thread(target=watchdog, daemon=True)
    th.start()

    def on_signal(signum, _frame):
        status["v"] = f"interrupted by signal {signum}"
        try:
            os.killpg(state["pgid"], signal.SIGTERM)
        except ProcessLookupError:
            pass

    signal.signal(signal.SIGINT, on_signal)
    signal.signal(signal.SIGTERM, on_signal)
    try:
        rc = proc.wait()
    finally:
        stop.set()
        kept = _salvage(out, ckpt_dir)        # the EXIT trap of hpc/deploy.sh: always runs
        if status["v"] == "finished" and proc.returncode not in (0, None):
            status["v"] = f"exit code {proc.returncode}"
        rep = _report(out, state, status["v"], a.cost_per_gpu_hour)
        state["ended"] = time.time()
        state["status"] = status["v"]
        _state_path(out).write_text(json.dumps(state, indent=1))
        print(json.dumps(rep), flush=True)
        print(f"salvaged {len(kept)} checkpoint file(s) into {out / 'checkpoints'}", flush=True)
        if a.notify_cmd:
            msg = a.notify_cmd.format(status=status["v"], out=str(out))
            subprocess.run(msg, shell=True, input=json.dumps(rep).encode(), timeout=60, check=False)
    return 0 if status["v"] == "finished" and rc == 0 else 1


def status_cmd(a) -> int:
    out = Path(a.out)
    state = json.loads(_state_path(out).read_text())
    alive = False
    if "ended" not in state:
        try:
            os.kill(state["pid"], 0)
            alive = True
        except OSError:
            alive = False
    with open(out / "train.log", errors="replace") as f:
        print(monitor.summary(monitor.parse(f)))
    print("running" if alive else f"not running ({state.get('status', 'state unknown')})")
    return 0


def teardown(a) -> int:
    out = Path(a.out)
    state = json.loads(_state_path(out).read_text())
    if "ended" not in state:
        try:
            os.killpg(int(state["pgid"]), signal.SIGTERM)     # exactly the recorded process group
            for _ in range(50):
                time.sleep(0.2)
                os.kill(int(state["pid"]), 0)
            os.killpg(int(state["pgid"]), signal.SIGKILL)
        except (ProcessLookupError, OSError):
            pass
    kept = _salvage(out, Path(state["checkpoint_dir"]))
    rep = _report(out, state, state.get("status", "torn down"), a.cost_per_gpu_hour)
    print(json.dumps(rep))
    print(f"salvaged {len(kept)} checkpoint file(s)")
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    extra = []
    if "--" in argv:
        i = argv.index("--")
        argv, extra = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("action", choices=["start", "status", "teardown"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--port", type=int, default=29500)
    ap.add_argument("--budget-hours", type=float, default=0.0)
    ap.add_argument("--cost-per-gpu-hour", type=float, default=0.0)
    ap.add_argument("--notify-cmd", default="")
    ap.add_argument("--poll-seconds", type=float, default=30.0)
    a = ap.parse_args(argv)
    if a.action == "start":
        return start(a, extra)
    if a.action == "status":
        return status_cmd(a)
    return teardown(a)


if __name__ == "__main__":
    sys.exit(main())
