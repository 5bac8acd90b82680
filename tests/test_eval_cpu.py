"""Bits-per-byte evaluation and the shard-driven training run (eval lines, final checkpoint)."""
import json
import math
import re

import numpy as np
import torch

from autoresearch_b200.config import TrainConfig, model_preset
from autoresearch_b200.data.shards import write_shard
from autoresearch_b200.eval.bpb import eval_bpb, load_token_bytes


class _FixedLoader:
    def __init__(self, batches, B, T):
        self.batches, self.B, self.T = list(batches), B, T

    def next_batch(self):
        return self.batches.pop(0) if self.batches else None


class _FakeModel(torch.nn.Module):
    def __init__(self, per_tok):
        super().__init__()
        self.per_tok = per_tok

    def forward(self, ids, tgt):
        return None, self.per_tok


def test_bpb_formula_masks_zero_byte_tokens():
    tb = torch.tensor([0, 1, 2, 4], dtype=torch.int32)
    ids = torch.zeros(1, 4, dtype=torch.int32)
    tgt = torch.tensor([[1, 0, 2, 3]], dtype=torch.int32)
    nats = torch.tensor([0.5, 9.0, 1.0, 2.0])               # the 9.0 belongs to a 0-byte (special) target
    got = eval_bpb(_FakeModel(nats), _FixedLoader([(ids, tgt)], 1, 4), tb, max_batches=1)
    assert abs(got - (0.5 + 1.0 + 2.0) / (math.log(2) * (1 + 2 + 4))) < 1e-9


def test_token_bytes_loader_checks_length(tmp_path):
    p = tmp_path / "token_bytes.json"
    p.write_text(json.dumps([1, 2, 3]))
    assert load_token_bytes(tmp_path, 3).tolist() == [1, 2, 3]
    import pytest
    with pytest.raises(ValueError):
        load_token_bytes(p, 4)


def test_shard_training_run_logs_eval_and_writes_checkpoint(tmp_path, capsys):
    from autoresearch_b200.trainer import Trainer
    cfg = model_preset("tiny")
    rng = np.random.default_rng(0)
    data = tmp_path / "shards"
    data.mkdir()
    for i in range(3):
        write_shard(data / f"shard_{i:05d}.bin", rng.integers(0, cfg.vocab, size=(16, cfg.seq_len + 1)).astype(np.uint16), cfg.vocab)
    tokd = tmp_path / "tok"
    tokd.mkdir()
    (tokd / "token_bytes.json").write_text(json.dumps([0] * 4 + [3] * (cfg.vocab - 4)))
    t = TrainConfig(device_batch_size=2, total_batch_size=2 * cfg.seq_len, max_steps=5, cooldown_steps=2,
                    data_dir=str(data), tokenizer_dir=str(tokd), checkpoint_dir=str(tmp_path / "ck"), eval_interval=2,
                    checkpoint_interval=0, impl="oracle", cooldown_trigger_file="", log_interval=1)
    Trainer(cfg, t, device="cpu").run()
    out = capsys.readouterr().out
    assert re.search(r"\[eval\] step 2 \| val_bpb \d+\.\d{4}", out)
    assert re.search(r"\[eval\] final \| val_bpb \d+\.\d{4}", out)
    assert "[checkpoint] saved" in out and (tmp_path / "ck" / "model.safetensors").exists()
    assert (tmp_path / "ck" / "trainer_state.json").exists() and (tmp_path / "ck" / "optim_state.safetensors").exists()
    bpb = float(re.search(r"final \| val_bpb (\d+\.\d+)", out).group(1))
    assert 1.5 < bpb < 4.0                                   # ~ln(256)/ln2/3 bits per byte at chance level
