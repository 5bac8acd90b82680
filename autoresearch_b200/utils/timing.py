"""CUDA-event phase timing (device time, read only on log steps) and MFU accounting.

The reference records four events per step and reads them only when it logs
(brain/src/train.rs:867-870,969-975,1042-1052); MFU = flops_per_token * tokens / dt / peak
(brain/src/train.rs:152-188,708).
"""
from __future__ import annotations

import os as _os
import time

import torch


class PhaseTimer:
    def __init__(self, enabled: bool):
        self.enabled = enabled and torch.cuda.is_available()
        if self.enabled:
            self.ev = {k: torch.cuda.Event(enable_timing=True)
                       for k in ("start", "bwd_end", "opt_end", "end")}
        self.wall = {}

    def mark(self, name: str):
        if self.enabled:
            self.ev[name].record()
        self.wall[name] = time.perf_counter()

    def read_ms(self):
        """(fwd_bwd_ms, opt_ms, total_ms): one host<->device sync."""
        if self.enabled:
            self.ev["end"].synchronize()
            return (self.ev["start"].elapsed_time(self.ev["bwd_end"]),
                    self.ev["bwd_end"].elapsed_time(self.ev["opt_end"]),
                    self.ev["start"].elapsed_time(self.ev["end"]))
        w = self.wall
        return ((w["bwd_end"] - w["start"]) * 1e3, (w["opt_end"] - w["bwd_end"]) * 1e3,
                (w["end"] - w["start"]) * 1e3)


B200_NOMINAL_BF16_FLOPS = 2.25e15   # dense bf16 tensor peak of one B200 (the reference hard-codes its H100's 990e12)


def resolve_peak_flops(explicit: "float | None" = None) -> float:
    """MFU denominator per GPU: the configured value (TrainConfig.peak_flops), else the environment variable
    ARB_PEAK_TFLOPS, else the nominal dense bf16 peak of a B200.  A benchmark that wants MFU against a measured
    matmul rate passes that rate in."""
    if explicit:
        return float(explicit)
    env = _os.environ.get("ARB_PEAK_TFLOPS", "")
    try:
        if env and float(env) > 0:
            return float(env) * 1e12
    except ValueError:
        pass
    return B200_NOMINAL_BF16_FLOPS


def vram_mb() -> float:
    if torch.cuda.is_available():
        free, total = torch.cuda.mem_get_info()
        return (total - free) / (1024.0 * 1024.0)
    return 0.0


# ---- NVTX ranges (opt-in: ARB_NVTX=1) ----------------------------------------------------------------
# Phase and layer ranges for timeline tools (role of the phase events of brain/src/train.rs:867-870, which this
# package keeps as PhaseTimer; the reference has no NVTX).  Off by default: a range push/pop costs host time in the
# launch path.
import contextlib as _contextlib

NVTX = _os.environ.get("ARB_NVTX", "0") == "1"


@_contextlib.contextmanager
def nvtx_range(name: str):
    if NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield
