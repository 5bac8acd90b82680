"""Learning-rate, momentum and weight-decay schedules.

Warm-up -> constant -> cooldown ("WSD").  The reference drives every schedule from a
synthetic ``progress`` value that is 0 during the stable phase and ramps from
``1 - warmdown_ratio`` to 1 over ``cooldown_steps`` (brain/src/train.rs:692-700); the
multiplier functions are brain/src/optim.rs:139-182.  With that mapping the learning rate
is: peak until ``cooldown_start``, then linear (or cosine) to ``final_lr_frac * peak`` over
``cooldown_steps``; ``warmdown_ratio`` only shapes the Muon weight decay.

Warm-up is counted in steps here (``warmup_steps``); the reference's ratio-based warm-up
multiplies by ``progress / warmup_ratio`` which is 0 for the whole stable phase, so any
non-zero ratio froze training there.  The default (0 steps) is identical to the reference.
"""
from __future__ import annotations

import math
from typing import Optional

from ..config import ScheduleConfig


def wsd_progress(step: int, cooldown_start: Optional[int], cooldown_steps: int,
                 warmdown_ratio: float) -> float:
    if cooldown_start is None:
        return 0.0
    frac = min(max(step - cooldown_start, 0) / float(max(cooldown_steps, 1)), 1.0)
    return (1.0 - warmdown_ratio) + warmdown_ratio * frac


def lr_multiplier(progress: float, cfg: ScheduleConfig) -> float:
    """1 while progress < 1 - warmdown; then c = (1 - progress)/warmdown and
    linear: c + (1-c)*final ; cosine: m + (1-m)*final with m = (1 + cos(pi*(1-c)))/2."""
    wd = cfg.warmdown_ratio
    if wd <= 0.0 or progress < 1.0 - wd:
        return 1.0
    c = min(max((1.0 - progress) / wd, 0.0), 1.0)
    if cfg.schedule == "cosine":
        m = 0.5 * (1.0 + math.cos(math.pi * (1.0 - c)))
        return m + (1.0 - m) * cfg.final_lr_frac
    return c + (1.0 - c) * cfg.final_lr_frac


def warmup_multiplier(step: int, warmup_steps: int) -> float:
    """`step` is 1-indexed (the step about to be taken)."""
    if warmup_steps <= 0:
        return 1.0
    return min(step / float(warmup_steps), 1.0)


def muon_momentum(step: int, cfg: ScheduleConfig) -> float:
    """0.85 -> 0.95 over the first 200 steps (brain/src/optim.rs:175-178)."""
    f = min(step / float(cfg.muon_momentum_warmup_steps), 1.0)
    return cfg.muon_momentum_start + (cfg.muon_momentum_end - cfg.muon_momentum_start) * f


def muon_weight_decay(progress: float, cfg: ScheduleConfig) -> float:
    """wd * (1 - progress) (brain/src/optim.rs:180-182)."""
    return cfg.weight_decay * (1.0 - progress)


def dmodel_lr_scale(d_model: int) -> float:
    """(D/768)^-0.5 applied to the AdamW learning rates of wte, lm_head, VE and routers
    (brain/src/optim.rs:139-141)."""
    return (d_model / 768.0) ** -0.5


class WSDState:
    """Tracks when the cooldown starts: automatically at ``max_steps - cooldown_steps`` or
    when a trigger fires (the reference watches a file, brain/src/train.rs:880-899)."""

    def __init__(self, max_steps: Optional[int], cooldown_steps: int, warmdown_ratio: float,
                 warmup_steps: int = 0):
        self.max_steps = max_steps
        self.cooldown_steps = cooldown_steps
        self.warmdown_ratio = warmdown_ratio
        self.warmup_steps = warmup_steps
        self.cooldown_start: Optional[int] = None

    def update(self, step: int, triggered: bool = False) -> None:
        if self.cooldown_start is not None:
            return
        if triggered:
            self.cooldown_start = step
        elif self.max_steps is not None and step >= max(self.max_steps - self.cooldown_steps, 0):
            self.cooldown_start = max(self.max_steps - self.cooldown_steps, 0)

    def progress(self, step: int) -> float:
        return wsd_progress(step, self.cooldown_start, self.cooldown_steps, self.warmdown_ratio)

    def finished(self, step: int) -> bool:
        if self.max_steps is not None and step >= self.max_steps:
            return True
        return (self.cooldown_start is not None
                and step >= self.cooldown_start + self.cooldown_steps)

    def state_dict(self):
        return {"cooldown_start": self.cooldown_start}

    def load_state_dict(self, d):
        self.cooldown_start = d.get("cooldown_start")
