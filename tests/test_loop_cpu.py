"""The shared step loop: input prefetch ring, data-position bookkeeping, agreement on the end of the data,
the device error word, and exact resume on TKNS shards."""
import threading
import time

import numpy as np
import pytest
import torch

from autoresearch_b200.config import TrainConfig, model_preset
from autoresearch_b200.data.prefetch import PinnedPrefetcher
from autoresearch_b200.data.shards import ShardLoader, write_shard
from autoresearch_b200.data.synthetic import ZipfStream
from autoresearch_b200.loop import DeviceFault
from autoresearch_b200.trainer import Trainer


class _CountingLoader:
    """Batch n is filled with the value n; ends after `limit` batches."""

    def __init__(self, B, T, limit=None):
        self.B, self.T, self.n, self.limit = B, T, 0, limit

    def next_batch(self, ids, tgt):
        if self.limit is not None and self.n >= self.limit:
            return None
        ids.fill_(self.n)
        tgt.fill_(self.n + 1000)
        self.n += 1
        return ids, tgt

    def state_dict(self):
        return {"n": self.n}

    def load_state_dict(self, d):
        self.n = int(d["n"])


class _GatedEvent:
    """Stands in for the CUDA event of a host->device copy that has not finished yet."""

    def __init__(self):
        self.done = threading.Event()

    def synchronize(self):
        self.done.wait(5.0)


def test_prefetcher_keeps_order_and_never_rewrites_a_slot_before_its_copy_is_done():
    B, T, depth = 2, 8, 3
    pf = PinnedPrefetcher(_CountingLoader(B, T), B, T, depth=depth)
    held = []
    seen = []
    for step in range(12):
        slot, ids, tgt = pf.next()
        seen.append(int(ids[0, 0]))
        assert int(tgt[0, 0]) == seen[-1] + 1000
        ev = _GatedEvent()
        held.append((slot, ids, seen[-1], ev))
        pf.release(slot, ev)
        if len(held) == depth - 1:
            # the "copy" of the oldest slot is still in flight: the producer must not have touched it
            time.sleep(0.05)
            s0, ids0, v0, ev0 = held.pop(0)
            assert int(ids0[0, 0]) == v0 and int(ids0[-1, -1]) == v0
            ev0.done.set()
    assert seen == list(range(12))
    for _, _, _, ev in held:
        ev.done.set()
    pf.close()


def test_prefetcher_position_is_that_of_the_last_batch_taken():
    B, T = 1, 4
    pf = PinnedPrefetcher(_CountingLoader(B, T), B, T, depth=4)
    assert pf.wait_for(3)
    for _ in range(2):
        slot, _, _ = pf.next()
        pf.release(slot)
    assert pf.state_dict() == {"n": 2}               # although the producer is further ahead
    pf.load_state_dict({"n": 7})
    slot, ids, _ = pf.next()
    assert int(ids[0, 0]) == 7
    pf.close()


def test_prefetcher_reports_the_end_before_a_partial_step():
    B, T = 1, 4
    pf = PinnedPrefetcher(_CountingLoader(B, T, limit=5), B, T, depth=5)
    assert pf.wait_for(4)
    for _ in range(4):
        slot, _, _ = pf.next()
        pf.release(slot)
    assert not pf.wait_for(4)                         # one batch left: not a whole step of four
    pf.close()


def test_micro_steps_see_the_loader_sequence_with_four_accumulation_steps():
    """accum = 4 with two device buffers: every micro-step's device ids equal the stream's, in order."""
    cfg = model_preset("tiny")
    t = TrainConfig(device_batch_size=1, total_batch_size=4 * cfg.seq_len, max_steps=3, cooldown_steps=1,
                    synthetic_data=True, synthetic_kind="zipf", impl="oracle", cooldown_trigger_file="")
    tr = Trainer(cfg, t, device="cpu", quiet=True)
    assert tr.accum == 4
    ref = ZipfStream(1, cfg.seq_len, cfg.vocab, seed=t.seed)
    seen = []
    orig = tr.model.forward

    def spy(ids, tgt, **kw):
        seen.append((ids.clone(), tgt.clone()))
        return orig(ids, tgt, **kw)

    tr.model.forward = spy
    for _ in range(2):
        tr.train_step()
    assert len(seen) == 8
    for ids, tgt in seen:
        ri, rt = ref.next_batch()
        assert torch.equal(ids, ri) and torch.equal(tgt, rt)
    tr.prefetch.close()


def test_a_kernel_fault_stops_the_run_before_logging(capsys):
    cfg = model_preset("tiny")
    t = TrainConfig(device_batch_size=2, total_batch_size=2 * cfg.seq_len, max_steps=6, cooldown_steps=2,
                    synthetic_data=True, synthetic_kind="zipf", impl="oracle", cooldown_trigger_file="")
    tr = Trainer(cfg, t, device="cpu")
    tr._kernel_error = lambda: "peer barrier wait timed out" if tr.step == 3 else None
    with pytest.raises(DeviceFault) as e:
        tr.run()
    assert "rank 0" in str(e.value) and "step 2" in str(e.value) and "peer barrier" in str(e.value)
    out = capsys.readouterr().out
    assert "step     1 |" in out and "step     2 |" not in out


def _write_shards(d, n_shards, rows, T, vocab):
    rng = np.random.default_rng(0)
    for i in range(n_shards):
        write_shard(d / f"shard_{i:05d}.bin", rng.integers(1, vocab, size=(rows, T + 1), dtype=np.uint16), vocab)


def test_shard_loader_position_round_trip(tmp_path):
    T = 16
    _write_shards(tmp_path, 4, 5, T, 200)
    a = ShardLoader(tmp_path, 2, T, split="train", seed=3)
    for _ in range(9):                                 # crosses shard and epoch boundaries (15 train rows)
        a.next_batch()
    st = a.state_dict()
    b = ShardLoader(tmp_path, 2, T, split="train", seed=3)
    b.load_state_dict(st)
    for _ in range(5):
        xa, xb = a.next_batch(), b.next_batch()
        assert torch.equal(xa[0], xb[0]) and torch.equal(xa[1], xb[1])


def test_trainer_resume_on_shards_continues_the_data_stream(tmp_path):
    cfg = model_preset("tiny")
    data = tmp_path / "data"
    data.mkdir()
    _write_shards(data, 3, 6, cfg.seq_len, cfg.vocab)

    def mk(resume, ck):
        t = TrainConfig(device_batch_size=2, total_batch_size=4 * cfg.seq_len, max_steps=8, cooldown_steps=2,
                        data_dir=str(data), impl="oracle", cooldown_trigger_file="", checkpoint_dir=str(ck), resume=resume)
        return Trainer(cfg, t, device="cpu", quiet=True)

    one = mk(False, tmp_path / "a")
    ref = [float(one.train_step()) for _ in range(6)]
    one.prefetch.close()
    two = mk(False, tmp_path / "b")
    first = [float(two.train_step()) for _ in range(3)]
    two.save(step=None)
    two.prefetch.close()
    three = mk(True, tmp_path / "b")
    assert three.step == 3
    rest = [float(three.train_step()) for _ in range(3)]
    three.prefetch.close()
    assert first + rest == pytest.approx(ref, abs=1e-6)
