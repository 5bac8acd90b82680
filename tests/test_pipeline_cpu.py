"""Pipeline parallelism on CPU ranks (gloo): schedule shape, layer split, and loss parity of a
2-stage 1F1B run with the single-process run."""
import json
import os
import subprocess
import sys

from autoresearch_b200.parallel.pipeline import one_f_one_b, split_layers


def test_layer_split_gives_remainder_to_early_stages():
    assert split_layers(30, 4) == [(0, 8), (8, 16), (16, 23), (23, 30)]
    assert split_layers(30, 8)[0] == (0, 4) and split_layers(30, 8)[-1] == (27, 30)
    assert split_layers(2, 2) == [(0, 1), (1, 2)]


def test_1f1b_schedule_properties():
    for P in (2, 3, 4):
        for M in (1, 2, 4, 8):
            for s in range(P):
                sch = one_f_one_b(s, P, M)
                assert [i for k, i in sch if k == "F"] == list(range(M))
                assert [i for k, i in sch if k == "B"] == list(range(M))
                for k, i in sch:       # a micro-batch is never back-propagated before its forward
                    if k == "B":
                        assert sch.index(("F", i)) < sch.index(("B", i))
                live = peak = 0
                for k, _ in sch:
                    live += 1 if k == "F" else -1
                    peak = max(peak, live)
                assert peak <= min(P - s, M)     # activations in flight are bounded by the depth


WORKER = r"""
import os, sys, json, torch, torch.distributed as dist
sys.path.insert(0, os.environ["ARB_ROOT"])
from autoresearch_b200.config import TrainConfig, model_preset
from autoresearch_b200.parallel.pipeline import PipelineTrainer
dist.init_process_group("gloo")
cfg = model_preset("tiny", n_layer=3)
t = TrainConfig(device_batch_size=2, total_batch_size=8 * 128, max_steps=10, cooldown_steps=3, synthetic_data=True,
                synthetic_kind="zipf", impl="oracle", cooldown_trigger_file="")
t.init_scheme = "normal"
tr = PipelineTrainer(cfg, t, pp=dist.get_world_size(), device="cpu", quiet=True)
ls = [tr.loss_on_all_ranks(tr.train_step()) for _ in range(4)]
if dist.get_rank() == 0:
    print("RESULT " + json.dumps({"losses": ls, "accum": tr.accum, "bytes": tr.comm_bytes}))
dist.destroy_process_group()
"""


import pytest


@pytest.mark.parametrize("stages", [2, 3])
def test_pipeline_matches_single_process(tmp_path, stages):
    """Two stages (every exchange between the same pair) and three (a middle stage talks to both neighbours)."""
    import torch
    from autoresearch_b200.config import TrainConfig, model_preset
    from autoresearch_b200.models.init import init_weights
    from autoresearch_b200.trainer import Trainer
    cfg = model_preset("tiny", n_layer=3)
    t = TrainConfig(device_batch_size=2, total_batch_size=8 * 128, max_steps=10, cooldown_steps=3, synthetic_data=True,
                    synthetic_kind="zipf", impl="oracle", cooldown_trigger_file="")
    one = Trainer(cfg, t, device="cpu", quiet=True)
    init_weights(one.model, seed=t.seed, scheme="normal")
    for gi, st in one.opt.state.items():
        st["master"].copy_(one.layout.group_view(one.layout.flat_param, one.layout.groups[gi]).float())
    ref = [float(one.train_step()) for _ in range(4)]
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={stages}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29654 + stages), str(script)],
                       env=dict(os.environ, ARB_ROOT=root), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["accum"] == 4 and res["bytes"] > 0
    for a, b in zip(ref, res["losses"]):
        assert abs(a - b) < 2e-3, (ref, res)


def test_merged_schedule_respects_stage_order_and_dependencies():
    from autoresearch_b200.parallel.pipeline_inproc import merged_schedule
    for P in (1, 2, 3, 4):
        for M in (1, 2, 5, 8):
            order = merged_schedule(P, M)
            assert len(order) == 2 * P * M
            seen = set()
            for s, k, i in order:
                if k == "F" and s > 0:
                    assert (s - 1, "F", i) in seen
                if k == "B":
                    assert (s, "F", i) in seen
                    if s < P - 1:
                        assert (s + 1, "B", i) in seen
                seen.add((s, k, i))
            for s in range(P):
                assert [(k, i) for ss, k, i in order if ss == s] == one_f_one_b(s, P, M)


def test_in_process_pipeline_matches_single_stage_and_resumes(tmp_path):
    """The one-process pipeline driver on two (CPU) 'devices': same losses as the plain trainer, per-stage
    checkpoints under stage_{i}/, and an exact resume."""
    import torch
    from autoresearch_b200.config import TrainConfig, model_preset
    from autoresearch_b200.models.init import init_weights
    from autoresearch_b200.parallel.pipeline_inproc import InProcPipelineTrainer
    from autoresearch_b200.trainer import Trainer
    cfg = model_preset("tiny")

    def tc(**kw):
        t = TrainConfig(device_batch_size=2, total_batch_size=8 * 128, max_steps=10, cooldown_steps=3, synthetic_data=True,
                        synthetic_kind="zipf", impl="oracle", cooldown_trigger_file="", **kw)
        t.init_scheme = "normal"
        return t

    one = Trainer(cfg, tc(), device="cpu", quiet=True)
    init_weights(one.model, seed=42, scheme="normal")
    for gi, st in one.opt.state.items():
        st["master"].copy_(one.layout.group_view(one.layout.flat_param, one.layout.groups[gi]).float())
    ref = [float(one.train_step()) for _ in range(5)]
    one.prefetch.close()
    pp = InProcPipelineTrainer(cfg, tc(checkpoint_dir=str(tmp_path)), ["cpu", "cpu"], quiet=True)
    assert pp.accum == 4 and pp.world == 2
    got = [float(pp.train_step()) for _ in range(3)]
    pp.save()
    pp.prefetch.close()
    assert (tmp_path / "stage_0" / "model.safetensors").exists() and (tmp_path / "stage_1" / "optim_state.safetensors").exists()
    again = InProcPipelineTrainer(cfg, tc(checkpoint_dir=str(tmp_path), resume=True), ["cpu", "cpu"], quiet=True)
    assert again.step == 3
    got += [float(again.train_step()) for _ in range(2)]
    again.prefetch.close()
    assert pp.comm_bytes > 0
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-3, (ref, got)
