"""Device memory plan: sizes from the configuration, one reservation, no growth while training, refusal at start-up."""
import pytest
import torch

from autoresearch_b200.config import TrainConfig, model_preset
from autoresearch_b200.utils import memplan


def test_plan_of_the_headline_configs_is_in_the_expected_range():
    p = memplan.plan(model_preset("phase2"), 4)
    assert 100e9 < p.total_bytes < 125e9                      # ~3 GiB per layer kept for the backward pass
    names = [n for n, _ in p.step]
    assert any("packed qkv" in n for n in names) and any("logits chunk" in n for n in names)
    assert "MB" in p.report()
    # eight-way data parallel, two sequences per micro-step: half the activations, an eighth of the optimizer state
    p8 = memplan.plan(model_preset("phase2"), 2, dp=8, fused_dp=True)
    assert p8.total_bytes < 0.55 * p.total_bytes
    opt1 = dict(p.persistent)["optimizer state (3 x fp32, owner shard)"]
    opt8 = dict(p8.persistent)["optimizer state (3 x fp32, owner shard)"]
    assert abs(opt8 * 8 - opt1) < 128
    # tensor parallel halves the wide activations but not the gathered ones
    w1 = memplan.plan(model_preset("wide"), 1)
    w2 = memplan.plan(model_preset("wide"), 1, tp=2)
    assert 0.5 * w1.total_bytes < w2.total_bytes < 0.85 * w1.total_bytes


@pytest.mark.gpu
def test_training_stays_inside_the_reserved_plan():
    from autoresearch_b200.trainer import Trainer
    cfg = model_preset("small")
    t = TrainConfig(device_batch_size=8, total_batch_size=16 * cfg.seq_len, max_steps=10, cooldown_steps=2,
                    synthetic_data=True, synthetic_kind="zipf", impl="sm100", cooldown_trigger_file="")
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    tr = Trainer(cfg, t, device="cuda", quiet=True)
    assert tr.mem_reserved["reserved_mb"] > 0
    tr.train_step()
    torch.cuda.synchronize()
    reserved1 = torch.cuda.memory_reserved()
    for _ in range(3):
        tr.train_step()
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - base
    assert peak <= tr.mem_plan.total_bytes, (peak, tr.mem_plan.report())
    assert peak >= 0.5 * tr.mem_plan.total_bytes, (peak, tr.mem_plan.report())     # the plan is not a wild over-estimate
    # steps after the first take nothing more from the driver (small-pool segments aside)
    assert torch.cuda.memory_reserved() - reserved1 <= 32 << 20
    tr.prefetch.close()


@pytest.mark.gpu
def test_a_configuration_that_cannot_fit_is_refused_before_step_zero():
    from autoresearch_b200.trainer import Trainer
    cfg = model_preset("phase1")
    t = TrainConfig(device_batch_size=1024, total_batch_size=1024 * cfg.seq_len, max_steps=10, cooldown_steps=2,
                    synthetic_data=True, synthetic_kind="zipf", impl="sm100", cooldown_trigger_file="")
    with pytest.raises(MemoryError) as e:
        Trainer(cfg, t, device="cuda", quiet=True)
    assert "BATCH_SIZE" in str(e.value)
