"""Pipeline parallelism on GPUs with the sm_100a kernels: two stages as two processes (NCCL point-to-point, 1F1B,
receives posted one pass ahead), two stages inside one process (peer copies), and two stages x two data-parallel
replicas with the fused gradient exchange, all against the single-GPU run on the same global batch."""
import json
import os
import subprocess
import sys
import tempfile

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
mode = os.environ["ARB_MODE"]
torch.cuda.set_device(local)
cfg = model_preset("small")
t = TrainConfig(device_batch_size=2, total_batch_size=8 * cfg.seq_len, max_steps=20, cooldown_steps=5,
                synthetic_data=True, synthetic_kind="zipf", impl="sm100", cooldown_trigger_file="",
                parallel=ParallelConfig(comm="fused"))
extra = {}
if mode == "single":
    from autoresearch_b200.trainer import Trainer
    tr = Trainer(cfg, t, device="cuda:0", quiet=True)
    losses = [float(tr.train_step()) for _ in range(6)]
elif mode == "inproc":
    from autoresearch_b200.parallel.pipeline_inproc import InProcPipelineTrainer
    tr = InProcPipelineTrainer(cfg, t, ["cuda:0", "cuda:1"], quiet=True)
    losses = [float(tr.train_step()) for _ in range(6)]
    for d in (0, 1):
        torch.cuda.synchronize(d); K.check_err_flag(torch.device("cuda", d))
    extra["bytes"] = tr.comm_bytes
else:
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=__import__("datetime").timedelta(seconds=90))
    from autoresearch_b200.parallel.pipeline import PipelineTrainer
    tr = PipelineTrainer(cfg, t, pp=2, device=f"cuda:{local}", quiet=True)
    losses = [tr.global_loss(tr.train_step()) for _ in range(6)]
    extra["bytes"] = tr.comm_bytes
    extra["comm"] = tr.comm.name
    extra["accum"] = tr.accum
torch.cuda.synchronize(); K.check_err_flag()
if int(os.environ.get("RANK", "0")) == 0:
    print("RESULT " + json.dumps(dict(losses=losses, **extra)))
if dist.is_initialized():
    dist.destroy_process_group()
"""


def _run(mode, nproc, port):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(tempfile.mkdtemp(prefix="arb_pp_"), "worker.py")
    with open(path, "w") as f:
        f.write(WORKER)
    env = dict(os.environ, ARB_ROOT=root, ARB_MODE=mode, NCCL_NVLS_ENABLE="0")
    cmd = ([sys.executable, path] if nproc == 1 else
           [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
            "--master-addr", "127.0.0.1", "--master-port", str(port), path])
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    os.remove(path)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_stage_pipelines_follow_the_single_gpu_run():
    one = _run("single", 1, 0)
    procs = _run("procs", 2, 29671)
    inproc = _run("inproc", 1, 0)
    assert procs["bytes"] > 0 and inproc["bytes"] > 0 and procs["accum"] == 4
    for a, b, c in zip(one["losses"], procs["losses"], inproc["losses"]):
        assert abs(a - b) < 1e-2 * abs(a) and abs(a - c) < 1e-2 * abs(a), (one, procs, inproc)
    assert one["losses"][-1] < one["losses"][0]


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_pipeline_with_fused_data_parallel_exchange():
    one = _run("single", 1, 0)
    pd = _run("procs", 4, 29672)
    assert pd["comm"] == "fused" and pd["accum"] == 2
    for a, b in zip(one["losses"], pd["losses"]):
        assert abs(a - b) < 1e-2 * abs(a), (one, pd)
