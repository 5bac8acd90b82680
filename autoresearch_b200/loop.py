"""What every training driver shares: input staging, the step loop, device-timed phases, MFU,
log lines, the JSONL metrics file, proxy / final evaluation, periodic checkpoints, peer
liveness and the check of the kernels' error word.

The reference has three drivers with three copies of this loop (brain/src/train.rs:707-1180 single
GPU, :1191-1603 in-process pipeline, :1620-2029 NCCL pipeline); its pipeline copies log wall-clock
time only, have no evaluation and no resume.  Here the data-parallel ``Trainer``, the tensor-
parallel ``TPTrainer`` and the pipeline ``PipelineTrainer`` derive from one ``TrainerBase`` and
differ only in ``train_step`` and in how a loss / a checkpoint is assembled across ranks.

Log formats (scraped by the monitoring tools; brain/src/train.rs:1036-1051,1059,1152,1170-1177):
``step N | loss .. | lr .. | dt ..s | tok/s .. | mfu ..% | vram ..MB | steps_left ..``,
``timing | fwd+bwd ..ms  opt ..ms  gpu ..ms  wall_gap ..ms``, ``[eval] step N | val_bpb ..``,
``[checkpoint] saved ..`` and the ``---`` trailer.
"""
from __future__ import annotations

import json
import math
import os
import time
from typing import Optional

import torch
import torch.distributed as dist

from .config import ModelConfig, TrainConfig
from .data.prefetch import PinnedPrefetcher
from .eval.bpb import PROXY_EVAL_BATCHES
from .optim.schedule import lr_multiplier
from .utils.timing import PhaseTimer, nvtx_range, resolve_peak_flops, vram_mb


class DeviceFault(RuntimeError):
    """A kernel of this package reported a failure through the device error word (a bounded wait that
    ran out: tensor-core pipeline, attention pipeline, peer barrier, MoE dispatch)."""


class TrainerBase:
    # ---- filled by the subclass before _init_common --------------------------------------------
    mcfg: ModelConfig
    tcfg: TrainConfig
    device: torch.device
    quiet: bool = False
    rank: int = 0            # global rank
    world: int = 1           # GPUs of the job (MFU denominator)
    data_rank: int = 0       # coordinates of this rank's data stream
    data_world: int = 1
    micro_batch: int = 1
    accum: int = 1
    log_rank: int = 0        # the rank that prints and writes the metrics file
    impl: str = "oracle"

    # -------------------------------------------------------------------------------------------
    def _init_common(self) -> None:
        t, m = self.tcfg, self.mcfg
        on_gpu = self.device.type == "cuda"
        self.step = 0
        self.loss_ema = 0.0
        self.ema_steps = 0
        self.total_train_s = 0.0
        self.steady_steps = 0
        self.peak_flops = resolve_peak_flops(getattr(t, "peak_flops", None))
        self.flops_per_token = m.flops_per_token()
        self.timer = PhaseTimer(on_gpu)
        self.token_bytes = None
        self.train_loader = self._make_loader("train")
        B, T = self.micro_batch, m.seq_len
        # pinned host ring filled by a background thread + A/B device buffers
        # (brain/src/train.rs:31-97,348-409,915-931)
        self.prefetch = PinnedPrefetcher(self.train_loader, B, T, depth=min(self.accum, 8) + 1, pin=on_gpu)
        self._d = [(torch.empty(B, T, dtype=torch.int32, device=self.device),
                    torch.empty(B, T, dtype=torch.int32, device=self.device)) for _ in range(2)]
        self._loss_acc = torch.zeros((), dtype=torch.float32, device=self.device)
        self.h2d_bytes_per_step = 2 * B * T * 4 * self.accum
        self.metrics_f = open(t.metrics_jsonl, "a") if (t.metrics_jsonl and self.rank == self.log_rank) else None
        self._dist = dist.is_available() and dist.is_initialized()
        # A finite data source can end on one rank first (round-robin shards): the ranks agree, on the host,
        # whether a whole step's batches exist before any of them launches a micro-step.
        self._host_group = None
        if self._dist and dist.get_world_size() > 1 and not t.synthetic_data:
            self._host_group = dist.new_group(backend="gloo")
        self.hb = None
        if self._dist and dist.get_world_size() > 1 and t.heartbeat_timeout_s > 0:
            from .parallel.heartbeat import Heartbeat
            store = dist.distributed_c10d._get_default_store()
            self.hb = Heartbeat(store, dist.get_rank(), dist.get_world_size(),
                                interval_s=max(t.heartbeat_timeout_s / 10.0, 0.05),
                                timeout_s=t.heartbeat_timeout_s).start()

    # ---- device memory ---------------------------------------------------------------------------
    def plan_memory(self, **kw) -> None:
        """Computes this rank's memory plan, reserves the step-time part in one allocation (a configuration that
        cannot fit is refused here, before step 0) and prints the reference's start-up line
        ``Allocated N MB GPU memory (B=..)`` (brain/src/train.rs:721)."""
        from .utils import memplan
        self.mem_plan = memplan.plan(self.mcfg, self.micro_batch, **kw)
        self.mem_reserved = {"reserved_mb": 0.0}
        if self.device.type == "cuda" and self.impl == "sm100" and os.environ.get("ARB_NO_RESERVE", "0") != "1":
            self.mem_reserved = memplan.reserve(self.mem_plan.step_bytes, self.device)
        self._say(f"Allocated {self.mem_plan.total_bytes / memplan.MB:.1f} MB GPU memory (B={self.micro_batch})")
        if os.environ.get("ARB_MEMPLAN_VERBOSE", "0") == "1":
            self._say(self.mem_plan.report())

    # ---- small helpers ---------------------------------------------------------------------------
    def _say(self, msg: str) -> None:
        if not self.quiet and self.rank == self.log_rank:
            print(msg, flush=True)

    @property
    def tokens_per_step(self) -> int:
        return self.micro_batch * self.mcfg.seq_len * self.accum * self.data_world

    def _make_loader(self, split: str):
        from .data.shards import ShardLoader, StdinRowStream
        from .data.synthetic import LcgStream, ZipfStream
        t, m = self.tcfg, self.mcfg
        B, T = self.micro_batch, m.seq_len
        if t.synthetic_data:
            if t.synthetic_kind == "zipf":
                return ZipfStream(B, T, m.vocab, seed=t.seed + (0 if split == "train" else 7919),
                                  rank=self.data_rank, world=self.data_world)
            s = LcgStream(B, T, m.vocab)
            s.pos = (self.data_rank * B) % s.buf.shape[0]
            return s
        if t.stream_input and split == "train":
            if self.data_world > 1:
                raise RuntimeError("--stream-input is one stream: use shards with data parallelism")
            return StdinRowStream(B, T)
        return ShardLoader(t.data_dir, B, T, split=split, num_train_shards=t.num_train_shards,
                           seed=t.seed, rank=self.data_rank, world=self.data_world)

    # ---- input staging ---------------------------------------------------------------------------
    def step_data_ready(self) -> bool:
        """True when every rank has the batches of a whole optimizer step; no kernel has been launched
        for the step when this returns False."""
        ok = self.prefetch.wait_for(self.accum)
        if self._host_group is not None:
            flag = torch.tensor([1 if ok else 0], dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self._host_group)
            ok = bool(flag.item())
        return ok

    def _stage_batch(self, micro: int):
        """Next batch: pinned slot -> device buffer `micro & 1` (async).  The slot goes back to the
        producer together with the event that marks the end of its copies."""
        got = self.prefetch.next()
        if got is None:
            return None
        slot, h_ids, h_tgt = got
        d_ids, d_tgt = self._d[micro & 1]
        d_ids.copy_(h_ids, non_blocking=True)
        d_tgt.copy_(h_tgt, non_blocking=True)
        ev = None
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
        self.prefetch.release(slot, ev)
        return d_ids, d_tgt

    # ---- failure detection -------------------------------------------------------------------------
    def _kernel_error(self) -> Optional[str]:
        """What the kernels of this package have written to the device error word since the last read (None:
        nothing).  One 4-byte device->host read."""
        if self.device.type != "cuda" or self.impl != "sm100":
            return None
        from .ops import kernels as K
        try:
            K.check_err_flag(self.device)
        except K.KernelError as e:
            return str(e)
        return None

    def check_device_errors(self, phase: str) -> None:
        """Called where the loop has just synchronised with the device: a kernel whose bounded wait ran out has
        produced garbage, so the run stops here, naming rank and phase, before the step is logged, evaluated or
        written to a checkpoint."""
        msg = self._kernel_error()
        if msg:
            self.prefetch.close()
            raise DeviceFault(f"rank {self.rank}, {phase}: {msg}")

    def _pre_step(self) -> None:
        if self.hb is not None:
            self.hb.check()          # a silent peer ends the run here, before any collective waits for it

    def _cooldown_triggered(self) -> bool:
        f = self.tcfg.cooldown_trigger_file
        return bool(f) and self.wsd.cooldown_start is None and os.path.exists(f)

    # ---- hooks -------------------------------------------------------------------------------------
    def train_step(self):
        raise NotImplementedError

    def global_loss(self, loss: torch.Tensor) -> float:
        """The step's mean loss as seen by the whole job (a collective when world > 1)."""
        return float(loss.item())

    def banner(self):
        return []

    def can_evaluate(self) -> bool:
        return True

    def evaluate(self, max_batches: Optional[int]) -> float:
        raise NotImplementedError

    def save(self, step: Optional[int]) -> Optional[str]:
        raise NotImplementedError

    def _max_over_ranks(self, v: float) -> float:
        if self._dist and dist.get_world_size() > 1:
            tm = torch.tensor([v], device=self.device, dtype=torch.float32)
            dist.all_reduce(tm, op=dist.ReduceOp.MAX)
            return float(tm.item())
        return v

    # ---- the loop ----------------------------------------------------------------------------------
    def run(self) -> None:
        t, m = self.tcfg, self.mcfg
        tokens_per_step = self.tokens_per_step
        for line in self.banner():
            self._say(line)
        t_total0 = time.perf_counter()
        max_diag = t.diagnostic_steps
        real_data = not t.synthetic_data and max_diag is None
        while True:
            if max_diag is not None and self.step >= max_diag:
                break
            if self.wsd.finished(self.step):
                break
            w0 = time.perf_counter()
            loss = self.train_step()
            if loss is None:
                self._say("data source exhausted")
                break
            step = self.step - 1
            is_eval = (t.eval_interval > 0 and step > 0 and step % t.eval_interval == 0 and real_data
                       and self.can_evaluate())
            if step % t.log_interval == 0 or step <= 10 or is_eval:
                fb_ms, opt_ms, gpu_ms = self.timer.read_ms()          # the only host<->device sync of a log step
                self.check_device_errors(f"step {step}")
                dt = time.perf_counter() - w0
                lv = self.global_loss(loss)
                if not math.isnan(lv):
                    self.loss_ema = 0.9 * self.loss_ema + 0.1 * lv
                    self.ema_steps += 1
                debiased = self.loss_ema / (1.0 - 0.9 ** max(self.ema_steps, 1))
                gpu_ms = self._max_over_ranks(gpu_ms)
                step_s = max(gpu_ms / 1e3, 1e-9)
                tok_s = tokens_per_step / step_s
                mfu = 100.0 * self.flops_per_token * tokens_per_step / step_s / (self.peak_flops * self.world)
                lrm = lr_multiplier(self.wsd.progress(step), t.schedule_cfg)
                left = (t.max_steps - self.step) if t.max_steps else -1
                vram = vram_mb()
                self._say(f"step {step:>5} | loss {debiased:.4f} | lr {lrm:.3f} | dt {step_s:.3f}s | "
                          f"tok/s {int(tok_s)} | mfu {mfu:.1f}% | vram {vram:.0f}MB | steps_left {left}")
                self._say(f"timing | fwd+bwd {fb_ms:.1f}ms  opt {opt_ms:.1f}ms  gpu {gpu_ms:.1f}ms  "
                          f"wall_gap {max(dt * 1e3 - gpu_ms, 0.0):.1f}ms")
                if step > 10:
                    self.total_train_s += step_s
                    self.steady_steps += 1
                if self.metrics_f:
                    self.metrics_f.write(json.dumps(dict(
                        step=step, loss=lv, loss_ema=debiased, lr_mult=lrm, dt_device_max_s=step_s,
                        tok_s=tok_s, mfu=mfu, fwd_bwd_ms=fb_ms, opt_ms=opt_ms, vram_mb=vram,
                        comm_bytes=int(getattr(self, "comm_bytes", 0)))) + "\n")
                    self.metrics_f.flush()
                if lv > 100 or math.isnan(lv):
                    self._say(f"loss {lv} blew up at step {step}; stopping")
                    break
            if is_eval:
                bpb = self.evaluate(PROXY_EVAL_BATCHES)
                self._say(f"[eval] step {step} | val_bpb {bpb:.4f}")
            if (t.checkpoint_interval > 0 and step > 0 and step % t.checkpoint_interval == 0
                    and t.checkpoint_dir and real_data):
                self.save(step=None)
        total_s = time.perf_counter() - t_total0
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self.check_device_errors("end of training")
        if real_data and t.checkpoint_dir:
            p = self.save(step=None)
            self._say(f"[checkpoint] saved {p}")
            if self.can_evaluate():
                bpb = self.evaluate(None)
                self._say(f"[eval] final | val_bpb {bpb:.4f}")
        steady = self.steady_steps
        mfu = (100.0 * self.flops_per_token * tokens_per_step * steady
               / max(self.total_train_s, 1e-9) / (self.peak_flops * self.world)) if steady else 0.0
        self._say("---")
        self._say(f"training_seconds: {self.total_train_s:.1f}")
        self._say(f"total_seconds:    {total_s:.1f}")
        self._say(f"mfu_percent:      {mfu:.2f}")
        self._say(f"total_tokens_M:   {tokens_per_step * self.step / 1e6:.1f}")
        self._say(f"num_steps:        {self.step}")
        self._say(f"num_params_M:     {m.num_params()['total'] / 1e6:.1f}")
        self._say(f"depth:            {m.n_layer}")
        self.prefetch.close()


__all__ = ["TrainerBase", "DeviceFault", "nvtx_range"]
