"""Schedules: values restated from the reference's optimizer unit tests
(brain/src/optim.rs:1010-1075) and from the WSD mapping (brain/src/train.rs:692-700)."""
import math

from autoresearch_b200.config import ScheduleConfig, derive_accumulation
from autoresearch_b200.optim import schedule as S


def test_linear_multiplier_points():
    c = ScheduleConfig(warmdown_ratio=0.75, final_lr_frac=0.05, schedule="linear")
    assert S.lr_multiplier(0.0, c) == 1.0
    assert S.lr_multiplier(0.1, c) == 1.0
    assert abs(S.lr_multiplier(0.25, c) - 1.0) < 1e-12
    mid = S.lr_multiplier(0.625, c)          # c = 0.5 -> 0.5 + 0.5*0.05
    assert abs(mid - 0.525) < 1e-12
    assert abs(S.lr_multiplier(1.0, c) - 0.05) < 1e-12


def test_cosine_multiplier_points():
    c = ScheduleConfig(warmdown_ratio=0.75, final_lr_frac=0.05, schedule="cosine")
    assert S.lr_multiplier(0.2, c) == 1.0
    mid = S.lr_multiplier(0.625, c)
    assert abs(mid - (0.5 + 0.5 * 0.05)) < 1e-12
    assert abs(S.lr_multiplier(1.0, c) - 0.05) < 1e-12


def test_wsd_is_peak_then_linear_to_final():
    c = ScheduleConfig(warmdown_ratio=0.75, final_lr_frac=0.02)
    w = S.WSDState(max_steps=1000, cooldown_steps=300, warmdown_ratio=c.warmdown_ratio)
    mults = []
    for step in range(1000):
        w.update(step)
        mults.append(S.lr_multiplier(w.progress(step), c))
    assert all(m == 1.0 for m in mults[:700])
    assert abs(mults[850] - (0.5 + 0.5 * 0.02)) < 1e-9
    assert mults[999] > 0.02 and mults[999] < 0.03
    assert w.finished(1000) and not w.finished(999)


def test_trigger_starts_cooldown_and_run_ends_after_it():
    w = S.WSDState(max_steps=None, cooldown_steps=10, warmdown_ratio=0.5)
    for step in range(5):
        w.update(step)
        assert w.progress(step) == 0.0 and not w.finished(step)
    w.update(5, triggered=True)
    assert w.cooldown_start == 5
    assert abs(w.progress(5) - 0.5) < 1e-12 and abs(w.progress(10) - 0.75) < 1e-12
    assert w.finished(15) and not w.finished(14)


def test_momentum_weight_decay_and_dscale():
    c = ScheduleConfig()
    assert abs(S.muon_momentum(0, c) - 0.85) < 1e-12
    assert abs(S.muon_momentum(150, c) - 0.925) < 1e-12
    assert abs(S.muon_momentum(200, c) - 0.95) < 1e-12 and abs(S.muon_momentum(10**6, c) - 0.95) < 1e-12
    assert abs(S.muon_weight_decay(0.0, c) - 0.2) < 1e-12 and S.muon_weight_decay(1.0, c) == 0.0
    assert abs(S.dmodel_lr_scale(768) - 1.0) < 1e-12
    assert abs(S.dmodel_lr_scale(1024) - (1024 / 768) ** -0.5) < 1e-12


def test_warmup_in_steps():
    assert S.warmup_multiplier(1, 0) == 1.0
    assert S.warmup_multiplier(5, 10) == 0.5 and S.warmup_multiplier(20, 10) == 1.0


def test_env_recipe_scaling():
    c = ScheduleConfig.from_env({"PEAK_LR": "0.02", "WEIGHT_DECAY": "0.3", "FINAL_LR_FRAC": "0.02"})
    assert abs(c.embedding_lr - 0.45) < 1e-12 and abs(c.unembedding_lr - 0.0025) < 1e-12
    assert abs(c.scalar_lr - 0.25) < 1e-12 and c.weight_decay == 0.3


def test_accumulation_derivation():
    assert derive_accumulation(524288, 4, 32768, 1) == (4, 4)
    assert derive_accumulation(524288, 4, 32768, 2) == (4, 2)
    assert derive_accumulation(524288, 4, 32768, 4) == (4, 1)
    assert derive_accumulation(524288, 4, 32768, 8) == (2, 1)
    assert derive_accumulation(524288, 64, 2048, 8) == (32, 1)
    import pytest
    with pytest.raises(ValueError):
        derive_accumulation(524288, 4, 32768, 3)
    with pytest.raises(ValueError):
        derive_accumulation(1000, 4, 32768, 1)
