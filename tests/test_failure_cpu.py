"""Failure detection, all on the host: silent ranks are found by the heartbeat watchdog, a rank
that dies between steps ends its peers' next collective with an error instead of a hang, a loss
blow-up stops the run, and a cooldown trigger file ends an open-ended run with a checkpoint."""
import json
import os
import subprocess
import sys
import time

import pytest

from autoresearch_b200.parallel.heartbeat import DictStore, Heartbeat, RankFailure


def test_watchdog_flags_silent_rank_with_fake_clock():
    store = DictStore()
    now = [0.0]
    hbs = [Heartbeat(store, r, 3, interval_s=1, timeout_s=5, clock=lambda: now[0]) for r in range(3)]
    for _ in range(3):
        for h in hbs:
            h.beat()
        for h in hbs:
            h.observe()
        now[0] += 1
    assert all(h.dead_ranks() == [] for h in hbs)
    hbs[2].pause()                                   # rank 2's messages are dropped from now on
    for _ in range(8):
        for h in hbs:
            h.beat()
        for h in hbs:
            h.observe()
        now[0] += 1
    assert hbs[0].dead_ranks() == [2] and hbs[1].dead_ranks() == [2]
    with pytest.raises(RankFailure) as e:
        hbs[0].check()
    assert e.value.ranks == [2]
    hbs[2].resume()
    for h in hbs:
        h.beat()
    for h in hbs:
        h.observe()
    assert hbs[0].dead_ranks() == []


def test_watchdog_thread_detects_real_silence():
    store = DictStore()
    a = Heartbeat(store, 0, 2, interval_s=0.05, timeout_s=0.3).start()
    b = Heartbeat(store, 1, 2, interval_s=0.05, timeout_s=0.3).start()
    time.sleep(0.3)
    assert a.dead_ranks() == [] and b.dead_ranks() == []
    b.stop()                                          # rank 1 exits
    deadline = time.time() + 5
    while time.time() < deadline and not a.dead_ranks():
        time.sleep(0.05)
    assert a.dead_ranks() == [1]
    a.stop()


WORKER = r"""
import os, sys, time, datetime, torch, torch.distributed as dist
rank = int(os.environ["RANK"])
dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=8))
t = torch.ones(4)
dist.all_reduce(t)                                    # step 1: everyone is here
if rank == 1:
    os._exit(0)                                       # leaves between steps, nothing in flight
try:
    dist.all_reduce(t)                                # step 2: the peer is gone
    print("RESULT hung-or-passed")
except Exception as e:
    print("RESULT error " + type(e).__name__)
"""


def test_peer_exit_between_steps_surfaces_as_error_not_hang(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29671")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    out0, _ = procs[0].communicate(timeout=120)
    procs[1].wait(timeout=120)
    assert "RESULT error" in out0, out0


def test_nan_batch_stops_the_run(capsys):
    import torch
    from autoresearch_b200.config import TrainConfig, model_preset
    from autoresearch_b200.trainer import Trainer
    cfg = model_preset("tiny")
    t = TrainConfig(device_batch_size=2, total_batch_size=256, max_steps=50, cooldown_steps=5, synthetic_data=True,
                    impl="oracle", cooldown_trigger_file="", log_interval=1)
    tr = Trainer(cfg, t, device="cpu")
    with torch.no_grad():
        tr.model.lm_head.fill_(float("nan"))          # host-side injection into the loss path
    tr.run()
    out = capsys.readouterr().out
    assert "blew up" in out and tr.step < 5


def test_trigger_file_starts_cooldown_and_run_ends(tmp_path, capsys):
    from autoresearch_b200.config import TrainConfig, model_preset
    from autoresearch_b200.trainer import Trainer
    trig = tmp_path / "cooldown"
    cfg = model_preset("tiny")
    t = TrainConfig(device_batch_size=2, total_batch_size=256, max_steps=None, cooldown_steps=3, synthetic_data=True,
                    impl="oracle", cooldown_trigger_file=str(trig), log_interval=1)
    tr = Trainer(cfg, t, device="cpu", quiet=True)
    for _ in range(4):
        tr.train_step()
    assert tr.wsd.cooldown_start is None and not tr.wsd.finished(tr.step)
    trig.write_text("")
    tr.train_step()
    assert tr.wsd.cooldown_start == 4
    while not tr.wsd.finished(tr.step):
        tr.train_step()
    assert tr.step == 7
