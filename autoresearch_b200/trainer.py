"""Training driver: step loop, gradient accumulation to a fixed tokens/step budget, WSD
schedule, device-timed phases, logging, proxy / final bits-per-byte evaluation,
checkpoints, diagnostics.

Structure and log formats follow the reference driver (brain/src/train.rs:707-1180):
``step N | loss .. | lr .. | dt ..s | tok/s .. | mfu ..% | vram ..MB | steps_left ..``,
``timing | fwd+bwd ..ms  opt ..ms  gpu ..ms  wall_gap ..ms``, ``[eval] step N | val_bpb ..``
and the ``---`` trailer block.  Differences: data parallelism (the reference has none),
device-side bpb reduction, exact resume, a JSONL metrics file.
"""
from __future__ import annotations

import json
import math
import os
import time
from pathlib import Path
from typing import Optional

import torch
import torch.distributed as dist

from .ckpt import checkpoint as ckpt
from .config import ModelConfig, TrainConfig, derive_accumulation
from .data.shards import ShardLoader, StdinRowStream
from .data.synthetic import LcgStream, ZipfStream
from .eval.bpb import PROXY_EVAL_BATCHES, eval_bpb, load_token_bytes
from .models.gpt import GPT
from .models.init import init_weights
from .ops.backend import get_backend
from .optim.muon_adamw import MuonAdamW
from .optim.schedule import WSDState, lr_multiplier, warmup_multiplier
from .parallel.dp import LibraryComm, LocalComm
from .parallel.layout import ParamLayout
from .utils.timing import PhaseTimer, measured_peak_flops, nvtx_range, vram_mb


def _log(msg: str, rank: int = 0):
    if rank == 0:
        print(msg, flush=True)


class Trainer:
    """One data-parallel replica group training a full (non-pipelined) model."""

    def __init__(self, mcfg: ModelConfig, tcfg: TrainConfig, device: Optional[str] = None,
                 group=None, quiet: bool = False):
        self.mcfg, self.tcfg = mcfg, tcfg
        self.dist = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank(group) if self.dist else 0
        self.world = dist.get_world_size(group) if self.dist else 1
        self.group = group
        self.quiet = quiet
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        on_gpu = self.device.type == "cuda"
        impl = tcfg.impl
        if impl == "auto":
            impl = "sm100" if (on_gpu and torch.cuda.get_device_capability(self.device)[0] == 10) else "oracle"
        self.impl = impl
        self.dtype = torch.bfloat16 if on_gpu and impl != "oracle" else torch.float32
        self.backend = get_backend(impl, mcfg)
        self.ep = self.world if (tcfg.parallel.ep > 1 and mcfg.moe is not None and self.world > 1) else 1
        self.model = GPT(mcfg, self.backend, dtype=self.dtype, device=self.device, ep=self.ep,
                         ep_rank=self.rank if self.ep > 1 else 0)
        if tcfg.load_checkpoint:
            st = ckpt.load_weights(self.model, tcfg.load_checkpoint, strict=True)
            self._say(f"Loaded checkpoint {tcfg.load_checkpoint}: {st}")
        elif tcfg.init_weights_path:
            st = ckpt.load_weights(self.model, tcfg.init_weights_path, strict=False)
            self._say(f"Loaded initial weights {tcfg.init_weights_path}: {st}")
        else:
            init_weights(self.model, seed=tcfg.seed)
        self.micro_batch, self.accum = derive_accumulation(
            tcfg.total_batch_size, tcfg.device_batch_size, mcfg.seq_len, self.world)
        # ---- flat storage, communicator, optimizer ---------------------------------------
        self.comm = self._make_comm()
        alloc = getattr(self.comm, "allocator", None)
        groups = self.model.named_matrix_groups()
        expert_groups = [g for g in groups if g[2] == "muon_expert"] if self.ep > 1 else []
        dense_groups = [g for g in groups if g not in expert_groups]
        self.layout = ParamLayout(dense_groups, self.world, self.rank, allocator=alloc)
        if hasattr(self.comm, "attach"):
            self.comm.attach(self.layout)
        kernels = getattr(self.backend, "optim_kernels", None)
        self.opt = MuonAdamW(self.layout, tcfg.schedule_cfg, mcfg.d_model,
                             kernels=kernels() if callable(kernels) else None)
        # expert-parallel experts are unique to their rank: no reduction, a rank-local optimizer
        self.expert_layout = self.expert_opt = None
        if expert_groups:
            self.expert_layout = ParamLayout(expert_groups, 1, 0)
            self.expert_opt = MuonAdamW(self.expert_layout, tcfg.schedule_cfg, mcfg.d_model,
                                        kernels=kernels() if callable(kernels) else None)
            from .parallel.ep import EPContext
            self.backend.ep = EPContext(self.group if self.group is not None else dist.group.WORLD, self.device,
                                        mcfg.moe.n_experts, mcfg.d_model, self.micro_batch * mcfg.seq_len,
                                        mcfg.moe.top_k, mcfg.moe.capacity_factor)
        self.wsd = WSDState(tcfg.max_steps, tcfg.cooldown_steps, tcfg.schedule_cfg.warmdown_ratio,
                            warmup_steps=int(round(tcfg.schedule_cfg.warmup_ratio * (tcfg.max_steps or 0))))
        self.step = 0
        self.loss_ema = 0.0
        self.ema_steps = 0
        self.peak_flops = measured_peak_flops()
        self.flops_per_token = mcfg.flops_per_token()
        self.train_loader = self._make_loader("train")
        self.token_bytes = None
        self.timer = PhaseTimer(on_gpu)
        # pinned staging + A/B device buffers (brain/src/train.rs:31-97,915-931)
        B, T = self.micro_batch, mcfg.seq_len
        pin = on_gpu
        self._h = [(torch.empty(B, T, dtype=torch.int32, pin_memory=pin),
                    torch.empty(B, T, dtype=torch.int32, pin_memory=pin)) for _ in range(2)]
        self._d = [(torch.empty(B, T, dtype=torch.int32, device=self.device),
                    torch.empty(B, T, dtype=torch.int32, device=self.device)) for _ in range(2)]
        self._loss_acc = torch.zeros((), dtype=torch.float32, device=self.device)
        self.metrics_f = open(tcfg.metrics_jsonl, "a") if (tcfg.metrics_jsonl and self.rank == 0) else None
        self.total_train_s = 0.0
        self.steady_steps = 0
        self.h2d_bytes_per_step = 2 * B * T * 4 * self.accum
        self.hb = None
        if self.dist and self.world > 1 and tcfg.heartbeat_timeout_s > 0:
            from .parallel.heartbeat import Heartbeat
            store = dist.distributed_c10d._get_default_store()
            self.hb = Heartbeat(store, dist.get_rank(), dist.get_world_size(),
                                interval_s=max(tcfg.heartbeat_timeout_s / 10.0, 0.05),
                                timeout_s=tcfg.heartbeat_timeout_s).start()
        if tcfg.resume and tcfg.checkpoint_dir:
            self._resume()

    # ------------------------------------------------------------------
    def _say(self, msg):
        if not self.quiet:
            _log(msg, self.rank)

    def _make_comm(self):
        if self.world == 1:
            return LocalComm()
        # the peer-memory path hands gradients to the sm_100a optimizer kernels and parameters to the sm_100a GEMMs;
        # every other backend (fp32 oracle, library baseline) uses the library collectives
        if (self.tcfg.parallel.comm == "fused" and self.device.type == "cuda"
                and type(self.backend).__name__ == "Sm100Backend"):
            from .parallel.fused_dp import FusedComm
            return FusedComm(self.group, self.device)
        bucket = torch.bfloat16 if self.device.type == "cuda" else None
        return LibraryComm(self.group, bucket_dtype=bucket)

    def _make_loader(self, split: str):
        t, m = self.tcfg, self.mcfg
        B, T = self.micro_batch, m.seq_len
        if t.synthetic_data:
            if t.synthetic_kind == "zipf":
                return ZipfStream(B, T, m.vocab, seed=t.seed + (0 if split == "train" else 7919),
                                  rank=self.rank, world=self.world)
            s = LcgStream(B, T, m.vocab)
            s.pos = (self.rank * B) % s.buf.shape[0]
            return s
        if t.stream_input and split == "train":
            if self.world > 1 and self.rank != 0:
                raise RuntimeError("--stream-input feeds rank 0 only; use shards with data parallelism")
            return StdinRowStream(B, T)
        return ShardLoader(t.data_dir, B, T, split=split, num_train_shards=t.num_train_shards,
                           seed=t.seed, rank=self.rank, world=self.world)

    def _resume(self):
        d = Path(self.tcfg.checkpoint_dir)
        p = d / "model.safetensors"
        if not p.exists():
            return
        ckpt.load_weights(self.model, str(p), strict=True)
        for gi, st in self.opt.state.items():
            st["master"].copy_(self.layout.group_view(self.layout.flat_param, self.layout.groups[gi]).float())
        import glob
        from .ckpt.safetensors_io import load_file
        for f in sorted(glob.glob(str(d / "optim_state*.safetensors"))):
            self.opt.load_state_dict(load_file(f))
        sp = d / "trainer_state.json"
        if sp.exists():
            st = json.loads(sp.read_text())
            self.step = int(st["step"])
            self.loss_ema, self.ema_steps = st["loss_ema"], st["ema_steps"]
            self.wsd.load_state_dict(st["wsd"])
            if hasattr(self.train_loader, "load_state_dict") and st.get("data"):
                self.train_loader.load_state_dict(st["data"])
        self._say(f"Resumed from {d} at step {self.step}")

    # ------------------------------------------------------------------
    def _stage_batch(self, slot: int):
        h_ids, h_tgt = self._h[slot]
        got = self.train_loader.next_batch(h_ids, h_tgt)
        if got is None:
            return None
        d_ids, d_tgt = self._d[slot]
        d_ids.copy_(h_ids, non_blocking=True)
        d_tgt.copy_(h_tgt, non_blocking=True)
        return d_ids, d_tgt

    def train_step(self) -> Optional[float]:
        """One optimizer step (accum micro-steps).  Returns the mean loss as a device
        scalar tensor (no host sync) or None when the data source is exhausted."""
        m, t = self.mcfg, self.tcfg
        if self.hb is not None:
            self.hb.check()          # a silent peer ends the run here, before any collective waits for it
        self.timer.mark("start")
        self.wsd.update(self.step, triggered=self._cooldown_triggered())
        self.layout.zero_grad()
        if self.expert_layout is not None:
            self.expert_layout.zero_grad()
        self._loss_acc.zero_()
        tokens_micro = self.micro_batch * m.seq_len
        grad_scale = 1.0 / (tokens_micro * self.accum * self.world)
        for micro in range(self.accum):
            batch = self._stage_batch(micro & 1)
            if batch is None:
                return None
            ids, tgt = batch
            with nvtx_range(f"forward micro {micro}"):
                scaled, per_tok = self.model(ids, tgt, grad_scale=grad_scale)
            with nvtx_range(f"backward micro {micro}"):
                scaled.backward()
            self.layout.accumulate_autograd_grads()
            if self.expert_layout is not None:
                self.expert_layout.accumulate_autograd_grads()
            self._loss_acc += per_tok.sum() / (tokens_micro * self.accum)
        self.timer.mark("bwd_end")
        if t.diagnostic_steps is not None:
            self._print_grad_norms()
            self.timer.mark("opt_end")
            self.timer.mark("end")
            self.step += 1
            return self._loss_acc
        with nvtx_range("gradient exchange"):
            self.comm.reduce_scatter_grads(self.layout)
        progress = self.wsd.progress(self.step)
        wm = warmup_multiplier(self.step + 1, self.wsd.warmup_steps)
        gs = self.comm.grad_source(self.layout) if hasattr(self.comm, "grad_source") else None
        with nvtx_range("optimizer"):
            self.opt.step(self.step + 1, progress, wm, grad_source=gs)
            if self.expert_opt is not None:
                self.expert_opt.step(self.step + 1, progress, wm)
        with nvtx_range("parameter exchange"):
            self.comm.all_gather_params(self.layout)
        self.timer.mark("opt_end")
        self.timer.mark("end")
        self.step += 1
        return self._loss_acc

    def _cooldown_triggered(self) -> bool:
        f = self.tcfg.cooldown_trigger_file
        return bool(f) and self.wsd.cooldown_start is None and os.path.exists(f)

    def _print_grad_norms(self):
        for a in self.layout.atoms:
            for u in a.units:
                g = self.layout.flat_grad[u.offset:u.offset + u.numel]
                self._say(f"[diag] step {self.step} {u.name} grad_norm {g.float().norm().item():.6e}")

    # ------------------------------------------------------------------
    def mean_loss_across_ranks(self, loss: torch.Tensor) -> float:
        if self.world > 1:
            l = loss.detach().clone()
            dist.all_reduce(l, group=self.group)
            return float(l.item()) / self.world
        return float(loss.item())

    def run(self):
        t, m = self.tcfg, self.mcfg
        tokens_per_step = self.micro_batch * m.seq_len * self.accum * self.world
        self._say(f"Model: {m.name} {m.num_params()['total'] / 1e6:.1f}M params, impl={self.impl}, "
                  f"dtype={str(self.dtype).split('.')[-1]}, world={self.world} ({self.comm.name})")
        self._say(f"Batch: {self.micro_batch} x {m.seq_len} x accum {self.accum} x dp {self.world} = "
                  f"{tokens_per_step} tokens/step")
        self._say(self.layout.describe())
        t_total0 = time.perf_counter()
        max_diag = t.diagnostic_steps
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
            is_eval = (t.eval_interval > 0 and step > 0 and step % t.eval_interval == 0
                       and not t.synthetic_data and max_diag is None)
            if step % t.log_interval == 0 or step <= 10 or is_eval:
                fb_ms, opt_ms, gpu_ms = self.timer.read_ms()
                dt = time.perf_counter() - w0
                lv = self.mean_loss_across_ranks(loss)
                if not math.isnan(lv):
                    self.loss_ema = 0.9 * self.loss_ema + 0.1 * lv
                    self.ema_steps += 1
                debiased = self.loss_ema / (1.0 - 0.9 ** max(self.ema_steps, 1))
                if self.world > 1:
                    tm = torch.tensor([gpu_ms], device=self.device)
                    dist.all_reduce(tm, op=dist.ReduceOp.MAX, group=self.group)
                    gpu_ms = float(tm.item())
                step_s = max(gpu_ms / 1e3, 1e-9)
                tok_s = tokens_per_step / step_s
                mfu = 100.0 * self.flops_per_token * tokens_per_step / step_s / (self.peak_flops * self.world)
                lrm = lr_multiplier(self.wsd.progress(step), t.schedule_cfg)
                left = (t.max_steps - self.step) if t.max_steps else -1
                self._say(f"step {step:>5} | loss {debiased:.4f} | lr {lrm:.3f} | dt {step_s:.3f}s | "
                          f"tok/s {int(tok_s)} | mfu {mfu:.1f}% | vram {vram_mb():.0f}MB | steps_left {left}")
                self._say(f"timing | fwd+bwd {fb_ms:.1f}ms  opt {opt_ms:.1f}ms  gpu {gpu_ms:.1f}ms  "
                          f"wall_gap {max(dt * 1e3 - gpu_ms, 0.0):.1f}ms")
                if step > 10:
                    self.total_train_s += step_s
                    self.steady_steps += 1
                if self.metrics_f:
                    self.metrics_f.write(json.dumps(dict(
                        step=step, loss=lv, loss_ema=debiased, lr_mult=lrm, dt_device_max_s=step_s,
                        tok_s=tok_s, mfu=mfu, fwd_bwd_ms=fb_ms, opt_ms=opt_ms, vram_mb=vram_mb())) + "\n")
                    self.metrics_f.flush()
                if lv > 100 or math.isnan(lv):
                    self._say(f"loss {lv} blew up at step {step}; stopping")
                    break
            if is_eval:
                bpb = self.evaluate(PROXY_EVAL_BATCHES)
                self._say(f"[eval] step {step} | val_bpb {bpb:.4f}")
            if (t.checkpoint_interval > 0 and step > 0 and step % t.checkpoint_interval == 0
                    and t.checkpoint_dir and not t.synthetic_data and max_diag is None):
                self.save(step=None)
        total_s = time.perf_counter() - t_total0
        if max_diag is None and t.checkpoint_dir and not t.synthetic_data:
            p = self.save(step=None)
            self._say(f"[checkpoint] saved {p}")
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

    # ------------------------------------------------------------------
    def evaluate(self, max_batches: Optional[int]) -> float:
        if self.token_bytes is None:
            self.token_bytes = load_token_bytes(self.tcfg.tokenizer_dir, self.mcfg.vocab, self.device)
        loader = self._make_loader("val")
        return eval_bpb(self.model, loader, self.token_bytes, max_batches, self.device,
                        group=self.group if self.world > 1 else None)

    def save(self, step: Optional[int]) -> Optional[str]:
        if hasattr(self.comm, "flush"):
            self.comm.flush()     # weights whose pull is still pending are read below
        state = dict(step=self.step, loss_ema=self.loss_ema, ema_steps=self.ema_steps,
                     wsd=self.wsd.state_dict(), world=self.world,
                     data=(self.train_loader.state_dict() if hasattr(self.train_loader, "state_dict") else None))
        d = Path(self.tcfg.checkpoint_dir)
        d.mkdir(parents=True, exist_ok=True)
        from .ckpt.safetensors_io import save_file
        name = "optim_state.safetensors" if self.world == 1 else f"optim_state.rank{self.rank}.safetensors"
        save_file(self.opt.state_dict(), str(d / name))
        path = None
        gather = None
        if self.ep > 1:
            def gather(t):      # [E_local, ...] of every rank -> [E, ...]; ranks hold consecutive expert ids
                out = torch.empty((t.shape[0] * self.world,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
                dist.all_gather_into_tensor(out, t.detach().contiguous(), group=self.group)
                return out
        if self.rank == 0:
            path = ckpt.save_checkpoint(self.model, str(d), step=step, trainer_state=state, expert_gather=gather)
        elif gather is not None:
            ckpt.model_to_engine_tensors(self.model, expert_gather=gather, materialise=False)
        if self.world > 1:
            dist.barrier(group=self.group)
        return path
