"""Tensor parallel (TP=2) on GPUs: the peer-memory collectives and the NCCL arm against each other
and against the single-GPU run."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = r"""
import json, os, sys, torch
import torch.distributed as dist
sys.path.insert(0, os.environ["ARB_ROOT"])
from autoresearch_b200.config import TrainConfig, ParallelConfig, model_preset
from autoresearch_b200.ops import kernels as K
world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
torch.cuda.set_device(local)
cfg = model_preset("small")
t = TrainConfig(device_batch_size=4, total_batch_size=4 * cfg.seq_len, max_steps=20, cooldown_steps=5,
                synthetic_data=True, synthetic_kind="zipf", impl="sm100", cooldown_trigger_file="",
                parallel=ParallelConfig(tp=world, comm=os.environ["ARB_COMM"]))
if world > 1:
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=__import__("datetime").timedelta(seconds=90))
    from autoresearch_b200.parallel.tp import TPTrainer
    tr = TPTrainer(cfg, t, tp=world, device=f"cuda:{local}", quiet=True)
    losses = [tr.global_loss(tr.train_step()) for _ in range(6)]
    mode = tr.backend.tp.mode
else:
    from autoresearch_b200.trainer import Trainer
    tr = Trainer(cfg, t, device="cuda:0", quiet=True)
    losses = [float(tr.train_step()) for _ in range(6)]
    mode = "single"
torch.cuda.synchronize(); K.check_err_flag()
if int(os.environ.get("RANK", "0")) == 0:
    print("RESULT " + json.dumps({"losses": losses, "mode": mode}))
if world > 1:
    dist.destroy_process_group()
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_fused_and_library_follow_single_gpu():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    import tempfile
    path = os.path.join(tempfile.mkdtemp(prefix="arb_tp_"), "worker.py")
    with open(path, "w") as f:
        f.write(WORKER)

    def run(n, comm, port):
        env = dict(os.environ, ARB_ROOT=root, ARB_COMM=comm, NCCL_NVLS_ENABLE="0")
        cmd = ([sys.executable, path] if n == 1 else
               [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                "--master-addr", "127.0.0.1", "--master-port", str(port), path])
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
        return json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])

    one = run(1, "fused", 0)
    fused = run(2, "fused", 29641)
    lib = run(2, "nccl", 29642)
    os.remove(path)
    assert fused["mode"] == "fused" and lib["mode"] == "library"
    for a, b, c in zip(one["losses"], fused["losses"], lib["losses"]):
        assert abs(a - b) < 1e-2 * abs(a) and abs(b - c) < 1e-2 * abs(b), (one, fused, lib)
