"""Data-parallel training on 2 GPUs: the peer-memory path and the NCCL path must both follow
the single-GPU run (same global batch, same seed)."""
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
from autoresearch_b200.trainer import Trainer
from autoresearch_b200.ops import kernels as K
world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
torch.cuda.set_device(local)
if world > 1:
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=__import__("datetime").timedelta(seconds=90))
cfg = model_preset("small")
t = TrainConfig(device_batch_size=4, total_batch_size=8 * cfg.seq_len, max_steps=20, cooldown_steps=5,
                synthetic_data=True, synthetic_kind="zipf", impl="sm100", cooldown_trigger_file="",
                parallel=ParallelConfig(dp=world, comm=os.environ["ARB_COMM"]))
tr = Trainer(cfg, t, device=f"cuda:{local}", quiet=True)
losses = []
for _ in range(8):
    l = tr.train_step()
    losses.append(tr.mean_loss_across_ranks(l))
torch.cuda.synchronize(); K.check_err_flag()
if int(os.environ.get("RANK", "0")) == 0:
    print("RESULT " + json.dumps({"losses": losses, "comm": tr.comm.name, "pending_pulls": len(K.pending_pulls)}))
if world > 1:
    dist.destroy_process_group()
"""


def _run(nproc, comm, port):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, ARB_ROOT=root, ARB_COMM=comm, NCCL_NVLS_ENABLE="0")
    import tempfile
    path = os.path.join(tempfile.mkdtemp(prefix="arb_dp_"), "worker.py")
    with open(path, "w") as f:
        f.write(WORKER)
    if nproc == 1:
        cmd = [sys.executable, path]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), path]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    os.remove(path)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[7:])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_dp2_matches_single_gpu():
    one = _run(1, "fused", 29611)
    fused = _run(2, "fused", 29612)
    lib = _run(2, "nccl", 29613)
    assert fused["comm"] == "fused" and lib["comm"] == "library"
    # after a step the dense weights owned by the other rank wait for the GEMMs that will pull them
    assert fused["pending_pulls"] > 0 and lib["pending_pulls"] == 0
    for a, b, c in zip(one["losses"], fused["losses"], lib["losses"]):
        # every decomposition sees the identical global batch: only the bf16 summation order differs
        assert abs(a - b) < 1e-2 * abs(a), (one, fused)
        assert abs(a - c) < 1e-2 * abs(a), (one, lib)
    assert fused["losses"][-1] < fused["losses"][0]
