"""MoE kernels: router, dispatch/combine, batched expert GEMMs, against the dense-equivalent
PyTorch MoE; expert parallelism over 2 GPUs against the single-GPU result."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("cf", [0.0, 2.0, 0.75])
def test_moe_block_matches_reference(cf):
    from autoresearch_b200.models.moe import MoEFn
    from autoresearch_b200.ops import kernels as K, reference as R
    torch.manual_seed(0)
    N, D, E, M, k = 512, 256, 4, 512, 2
    mk = lambda *s, sc=1.0: (torch.randn(*s, device="cuda") * sc).to(torch.bfloat16).requires_grad_(True)
    xn, resid = mk(N, D), mk(N, D)
    wr, wfc, wpr = mk(E, D, sc=0.2), mk(E, M, D, sc=0.05), mk(E, D, M, sc=0.05)
    out, aux = MoEFn.apply(xn, resid, wr, wfc, wpr, k, 0.01, cf, None, 0)
    g = torch.randn(N, D, device="cuda").to(torch.bfloat16)
    (out.float() * g.float()).sum().add(aux * 3.0).backward()
    K.check_err_flag()
    ref_in = [t.detach().float().requires_grad_(True) for t in (xn, resid, wr, wfc, wpr)]
    y, raux = R.moe_mlp(ref_in[0], ref_in[2], ref_in[3], ref_in[4], k, 0.01, cf)
    rout = ref_in[1] + y
    (rout * g.float()).sum().add(raux * 3.0).backward()
    assert _rel(out, rout) < 2e-2
    assert abs(aux.item() - raux.item()) < 1e-4
    for name, a, b in zip(("xn", "resid", "router", "fc", "proj"), (xn, resid, wr, wfc, wpr), ref_in):
        assert _rel(a.grad, b.grad) < 6e-2, (name, _rel(a.grad, b.grad))


def test_moe_model_trains():
    from autoresearch_b200.config import TrainConfig, model_preset
    from autoresearch_b200.ops import kernels as K
    from autoresearch_b200.trainer import Trainer
    cfg = model_preset("small_moe")
    t = TrainConfig(device_batch_size=4, total_batch_size=8 * cfg.seq_len, max_steps=30, cooldown_steps=10,
                    synthetic_data=True, impl="sm100", cooldown_trigger_file="")
    tr = Trainer(cfg, t, device="cuda", quiet=True)
    losses = [float(tr.train_step()) for _ in range(25)]
    K.check_err_flag()
    assert losses[-1] < losses[0] - 0.2, losses


WORKER = r"""
import json, os, sys, torch
import torch.distributed as dist
sys.path.insert(0, os.environ["ARB_ROOT"])
import dataclasses
from autoresearch_b200.config import TrainConfig, ParallelConfig, model_preset
from autoresearch_b200.trainer import Trainer
from autoresearch_b200.ops import kernels as K
world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
torch.cuda.set_device(local)
if world > 1:
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=__import__("datetime").timedelta(seconds=90))
cfg = model_preset("small_moe")
cfg = dataclasses.replace(cfg, moe=dataclasses.replace(cfg.moe, capacity_factor=4.0, aux_coeff=0.0))
t = TrainConfig(device_batch_size=4, total_batch_size=8 * cfg.seq_len, max_steps=20, cooldown_steps=5,
                synthetic_data=True, synthetic_kind="zipf", impl="sm100", cooldown_trigger_file="",
                parallel=ParallelConfig(dp=world, ep=world, comm=os.environ.get("ARB_COMM", "fused")))
tr = Trainer(cfg, t, device=f"cuda:{local}", quiet=True)
losses = [tr.mean_loss_across_ranks(tr.train_step()) for _ in range(6)]
torch.cuda.synchronize(); K.check_err_flag()
ck = {}
if world > 1:
    # checkpoint under expert parallelism: one file with the experts of every rank under their global ids
    tr.tcfg.checkpoint_dir = os.environ["ARB_CKPT"]
    tr.save(step=None)
    from autoresearch_b200.ckpt.safetensors_io import load_file
    sd = load_file(os.path.join(os.environ["ARB_CKPT"], "model.safetensors"))
    E, El = cfg.moe.n_experts, tr.model.blocks[0].expert_fc.shape[0]
    rank = dist.get_rank()
    mine = all(torch.equal(sd[f"h.0.moe.expert.{rank * El + e}.fc.weight"], tr.model.blocks[0].expert_fc[e].detach().cpu())
               for e in range(El))
    ok = torch.tensor([int(mine)], device="cuda"); dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    ck = {"experts_in_file": sum(1 for k in sd if k.startswith("h.0.moe.expert.") and k.endswith(".fc.weight")),
          "every_rank_found_its_experts": bool(ok.item())}
    # and back: a fresh expert-parallel trainer loads its slice of the file
    t2 = dataclasses.replace(t, init_weights_path=os.path.join(os.environ["ARB_CKPT"], "model.safetensors"))
    tr2 = Trainer(cfg, t2, device=f"cuda:{local}", quiet=True)
    same = torch.equal(tr2.model.blocks[1].expert_proj.detach(), tr.model.blocks[1].expert_proj.detach())
    ok2 = torch.tensor([int(same)], device="cuda"); dist.all_reduce(ok2, op=dist.ReduceOp.MIN)
    ck["reload_matches"] = bool(ok2.item())
if int(os.environ.get("RANK", "0")) == 0:
    print("RESULT " + json.dumps({"losses": losses, "ep": tr.ep, "experts_local": tr.model.blocks[0].expert_fc.shape[0], "ckpt": ck,
                                  "exchange": getattr(tr.backend.ep, "mode", None) if world > 1 else None}))
if world > 1:
    dist.destroy_process_group()
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_two_gpus_matches_single_gpu():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    import tempfile
    path = os.path.join(tempfile.mkdtemp(prefix="arb_ep_"), "worker.py")
    with open(path, "w") as f:
        f.write(WORKER)
    ckdir = tempfile.mkdtemp(prefix="arb_ep_ckpt_")
    env = dict(os.environ, ARB_ROOT=root, NCCL_NVLS_ENABLE="0", ARB_DISABLE_MULTIMEM="1", ARB_CKPT=ckdir)

    def run(n, port, comm="fused"):
        cmd = ([sys.executable, path] if n == 1 else
               [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                "--master-addr", "127.0.0.1", "--master-port", str(port), path])
        r = subprocess.run(cmd, env=dict(env, ARB_COMM=comm), capture_output=True, text=True, timeout=240)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
        return json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])

    one, two, lib = run(1, 0), run(2, 29631), run(2, 29632, "nccl")
    assert two["exchange"] == "fused" and lib["exchange"] == "library"      # the library all-to-all arm
    for a, b in zip(one["losses"], lib["losses"]):
        assert abs(a - b) < 1e-2 * abs(a), (one, lib)
    os.remove(path)
    import shutil
    shutil.rmtree(ckdir, ignore_errors=True)
    assert one["ep"] == 1 and two["ep"] == 2 and two["experts_local"] == 2
    assert two["ckpt"] == {"experts_in_file": 4, "every_rank_found_its_experts": True, "reload_matches": True}, two["ckpt"]
    for a, b in zip(one["losses"], two["losses"]):
        assert abs(a - b) < 1e-2 * abs(a), (one, two)


def test_slot_positions_match_token_order_prefix_sum():
    """pos[s] counts the earlier slots of the same expert; counts[e] the slots per expert."""
    from autoresearch_b200.ops import kernels as K
    torch.manual_seed(5)
    for S, E in ((1, 4), (1000, 8), (5000, 3), (70001, 32)):
        idx = torch.randint(0, E, (S,), device="cuda", dtype=torch.int32)
        pos = torch.empty(S, dtype=torch.int32, device="cuda")
        counts = torch.empty(E, dtype=torch.int32, device="cuda")
        scratch = torch.empty(((S + 1023) // 1024) * E, dtype=torch.int32, device="cuda")
        K._check(K.lib().arb_moe_slot_positions(idx.data_ptr(), S, E, scratch.data_ptr(), pos.data_ptr(), counts.data_ptr(),
                                                K._stream()), "moe_slot_positions")
        onehot = torch.nn.functional.one_hot(idx.long(), E)
        ref = (onehot.cumsum(0) - 1).gather(1, idx.long().view(-1, 1)).squeeze(1)
        assert torch.equal(pos.long(), ref)
        assert torch.equal(counts.long(), onehot.sum(0))
