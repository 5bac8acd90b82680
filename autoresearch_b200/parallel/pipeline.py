"""Pipeline parallelism, one process per stage, with a 1F1B schedule over point-to-point sends (NCCL on
GPUs, gloo on CPU ranks).

What is kept from the reference's multi-process driver (brain/src/train.rs:1620-2029): one rank per
stage; layers split ``L // n`` with the remainder on the early stages; stage 0 owns the token
embedding, the last stage owns the LM head and the loss; every stage keeps and updates only its own
slice of ``resid_lambdas`` / ``x0_lambdas``; ``x`` and ``x0`` travel forward together; every rank
writes its checkpoint to ``rank_{r}/`` (brain/src/train.rs:1998-2002).

What is different: the reference runs one micro-batch through all stages strictly in sequence
(bubble (n-1)/n) with blocking sends and logs wall-clock time only; here micro-batches are
interleaved one-forward-one-backward.  Transfers never block the host (a wait is a dependency
of the compute stream on the transfer), sends are left in flight until the end of the step,
and whenever a pass's output and the next pass's input travel between the same two stages
(every pass of the steady state) the send and the receive are issued as ONE grouped NCCL
operation.  That grouping is what keeps two neighbours from each sitting in a send the other
has not posted a receive for; for the same reason receives are not posted a whole pass early:
a receive kernel that spins for the length of a pass occupies a hardware queue which the
compute stream, or the send its peer is waiting for, may share.  The gradient of ``x0`` is accumulated along the chain (each boundary carries d_x and d_x0
back) instead of every stage sending its partial sum to stage 0.  Pipeline stages can be combined
with data parallelism (rank = dp_index * n_stages + stage), whose gradient exchange is the same
fused peer-memory path as in the plain data-parallel trainer.  Loop, logging, timing, evaluation,
checkpoint cadence and resume are the shared ones of ``TrainerBase``.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ckpt import checkpoint as ckpt
from ..config import ModelConfig, TrainConfig, derive_accumulation
from ..models.gpt import GPT
from ..models.init import init_weights
from ..ops.backend import get_backend
from ..optim.muon_adamw import MuonAdamW
from ..loop import TrainerBase
from ..optim.schedule import WSDState, warmup_multiplier
from .dp import LibraryComm, LocalComm
from .layout import ParamLayout


def split_layers(n_layer: int, n_stages: int) -> List[Tuple[int, int]]:
    """[lo, hi) per stage; remainder layers go to the early stages."""
    base, rem = divmod(n_layer, n_stages)
    out, lo = [], 0
    for s in range(n_stages):
        hi = lo + base + (1 if s < rem else 0)
        out.append((lo, hi))
        lo = hi
    return out


def one_f_one_b(stage: int, n_stages: int, n_micro: int) -> List[Tuple[str, int]]:
    """The order of forward ('F', i) and backward ('B', i) passes of one stage."""
    warm = min(n_stages - 1 - stage, n_micro)
    sched: List[Tuple[str, int]] = []
    f = b = 0
    for _ in range(warm):
        sched.append(("F", f)); f += 1
    for _ in range(n_micro - warm):
        sched.append(("F", f)); f += 1
        sched.append(("B", b)); b += 1
    for _ in range(warm):
        sched.append(("B", b)); b += 1
    return sched


class PipelineTrainer(TrainerBase):
    def __init__(self, mcfg: ModelConfig, tcfg: TrainConfig, pp: int, device: str = "cpu", quiet: bool = False):
        if not dist.is_initialized():
            raise RuntimeError("pipeline training needs an initialised process group (torchrun)")
        self.mcfg, self.tcfg, self.pp = mcfg, tcfg, pp
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        if self.world % pp:
            raise ValueError(f"world size {self.world} is not a multiple of {pp} pipeline stages")
        self.dp = self.world // pp
        self.stage = self.rank % pp
        self.dp_idx = self.rank // pp
        self.data_rank, self.data_world = self.dp_idx, self.dp
        self.log_rank = self.world - 1            # the loss lives on the last stage (the reference logs there too)
        self.device = torch.device(device)
        self.quiet = quiet
        on_gpu = self.device.type == "cuda"
        impl = tcfg.impl
        if impl == "auto":
            impl = "sm100" if (on_gpu and torch.cuda.get_device_capability(self.device)[0] == 10) else "oracle"
        self.impl = impl
        self.dtype = torch.bfloat16 if on_gpu and impl != "oracle" else torch.float32
        self.backend = get_backend(impl, mcfg)
        # process groups (collective creation: every rank calls all): one DP group per stage
        self.dp_group = None
        for s in range(pp):
            g = dist.new_group([d * pp + s for d in range(self.dp)])
            if s == self.stage:
                self.dp_group = g
        lo, hi = split_layers(mcfg.n_layer, pp)[self.stage]
        self.first, self.last = self.stage == 0, self.stage == pp - 1
        self.model = GPT(mcfg, self.backend, dtype=self.dtype, device=self.device, layer_range=(lo, hi),
                         has_embedding=self.first, has_head=self.last)
        self._init_stage_weights()
        self.micro_batch, self.accum = derive_accumulation(tcfg.total_batch_size, tcfg.device_batch_size,
                                                           mcfg.seq_len, self.dp)
        fused = tcfg.parallel.comm == "fused" and on_gpu and impl == "sm100"
        if self.dp == 1:
            self.comm = LocalComm()
        elif fused:
            from .fused_dp import FusedComm
            self.comm = FusedComm(self.dp_group, self.device)
        else:
            self.comm = LibraryComm(self.dp_group, torch.bfloat16 if on_gpu else None)
        self.layout = ParamLayout(self.model.named_matrix_groups(), self.dp, self.dp_idx,
                                  allocator=getattr(self.comm, "allocator", None))
        if hasattr(self.comm, "attach"):
            self.comm.attach(self.layout)
        kernels = getattr(self.backend, "optim_kernels", None)
        self.opt = MuonAdamW(self.layout, tcfg.schedule_cfg, mcfg.d_model, kernels=kernels() if callable(kernels) else None)
        self.wsd = WSDState(tcfg.max_steps, tcfg.cooldown_steps, tcfg.schedule_cfg.warmdown_ratio,
                            int(round(tcfg.schedule_cfg.warmup_ratio * (tcfg.max_steps or 0))))
        self.sched = one_f_one_b(self.stage, pp, self.accum)
        self.comm_bytes = 0
        self._init_common()
        # every micro-batch of a step is staged up front (a stage needs batch i again for its backward)
        B, T = self.micro_batch, mcfg.seq_len
        self._d = [(torch.empty(B, T, dtype=torch.int32, device=self.device),
                    torch.empty(B, T, dtype=torch.int32, device=self.device)) for _ in range(self.accum)]
        # a stage keeps the forward tensors of up to (pp - stage) micro-batches in flight
        in_flight = min(pp - self.stage, self.accum)
        self.plan_memory(dp=self.dp, n_layer_local=(hi - lo) * in_flight, has_embedding=self.first, has_head=self.last,
                         fused_dp=fused and self.dp > 1, act_bytes=2 if self.dtype == torch.bfloat16 else 4,
                         ce_chunk=max(mcfg.ce_chunk, getattr(self.backend, "big_ce_chunk", 0)))
        if tcfg.resume and tcfg.checkpoint_dir:
            self._resume()

    def _init_stage_weights(self):
        """Initialise the full model once per rank with the shared seed and keep this stage's
        slice, so that a pipelined run starts from the same weights as a single-process run."""
        t = self.tcfg
        if t.load_checkpoint:
            ckpt.load_weights(self.model, t.load_checkpoint, strict=True)
            return
        full = GPT(self.mcfg, get_backend("oracle", self.mcfg), dtype=torch.float32, device="cpu")
        if t.init_weights_path:
            ckpt.load_weights(full, t.init_weights_path, strict=False)
        else:
            init_weights(full, seed=t.seed, scheme=getattr(t, "init_scheme", "reference"))
        src = dict(full.named_parameters())
        lo = self.model.layer_lo
        with torch.no_grad():
            for n, p in self.model.named_parameters():
                if n in ("resid_lambdas", "x0_lambdas"):
                    p.copy_(src[n][lo:self.model.layer_hi])
                elif n.startswith("blocks."):
                    parts = n.split(".")
                    parts[1] = str(int(parts[1]) + lo)
                    p.copy_(src[".".join(parts)])
                else:
                    p.copy_(src[n])
        del full

    # ---- transfers ----------------------------------------------------------------------------------
    def _peer(self, stage: int) -> int:
        return self.dp_idx * self.pp + stage

    def _exchange(self, send, recv_from, act_shape):
        """One grouped point-to-point operation: `send` = (tensors, stage) or None, `recv_from` = stage or None (two
        tensors of `act_shape` are received).  Returns (received tensors, requests, tensors kept alive)."""
        ops, bufs, keep = [], [], []
        if send is not None:
            for t in send[0]:
                t = t.contiguous()
                keep.append(t)
                self.comm_bytes += t.numel() * t.element_size()
                ops.append(dist.P2POp(dist.isend, t, self._peer(send[1])))
        if recv_from is not None:
            for _ in range(2):
                b = torch.empty(act_shape, dtype=self.dtype, device=self.device)
                bufs.append(b)
                ops.append(dist.P2POp(dist.irecv, b, self._peer(recv_from)))
        reqs = dist.batch_isend_irecv(ops) if ops else []
        return bufs, reqs, keep

    def _needs(self, op):
        """The stage a pass receives its inputs from (None: it has them)."""
        kind, _ = op
        if kind == "F":
            return None if self.first else self.stage - 1
        return None if self.last else self.stage + 1

    def train_step(self):
        m = self.mcfg
        self._pre_step()
        if not self.step_data_ready():
            return None
        self.timer.mark("start")
        self.wsd.update(self.step, triggered=self._cooldown_triggered())
        self.layout.zero_grad()
        B, T, D = self.micro_batch, m.seq_len, m.d_model
        act_shape = (B * T, D)
        tokens_micro = B * T
        grad_scale = 1.0 / (tokens_micro * self.accum * self.dp)
        batches = [self._stage_batch(i) for i in range(self.accum)]
        saved = {}
        in_flight = []            # requests (and their tensors) of sends that nobody has waited for yet
        self._loss_acc.zero_()
        out_send = None           # (tensors, stage): what the previous pass produced for a neighbour
        for kind, i in self.sched:
            src = self._needs((kind, i))
            got = []
            if out_send is not None and src is not None and out_send[1] == src:
                got, reqs, keep = self._exchange(out_send, src, act_shape)         # one grouped send + receive
                out_send = None
            else:
                if out_send is not None:
                    _, r0, k0 = self._exchange(out_send, None, act_shape)
                    in_flight.append((r0, k0))
                    out_send = None
                reqs, keep = [], []
                if src is not None:
                    got, reqs, keep = self._exchange(None, src, act_shape)
            for r in reqs:
                r.wait()                                                             # the compute stream waits, not the host
            ids, tgt = batches[i]
            if kind == "F":
                if self.first:
                    x_in = x0_in = None
                else:
                    x_in, x0_in = got
                    x_in.requires_grad_(True); x0_in.requires_grad_(True)
                out = self.model(ids, tgt, grad_scale=grad_scale, x_in=x_in, x0_in=x0_in)
                if self.last:
                    scaled, per_tok = out
                    self._loss_acc += per_tok.sum() / (tokens_micro * self.accum)
                    saved[i] = (x_in, x0_in, scaled, None)
                else:
                    x_out, x0_out = out
                    out_send = ([x_out.detach(), x0_out.detach()], self.stage + 1)
                    saved[i] = (x_in, x0_in, x_out, x0_out)
            else:
                x_in, x0_in, y, x0_out = saved.pop(i)
                if self.last:
                    y.backward()
                    d_x0_down = None
                else:
                    d_x, d_x0_down = got
                    if self.first:
                        # x0_out is the embedding output itself: both gradients enter the graph
                        torch.autograd.backward([y, x0_out], [d_x, d_x0_down])
                    else:
                        torch.autograd.backward([y], [d_x])
                self.layout.accumulate_autograd_grads()
                if not self.first:
                    g0 = x0_in.grad if x0_in.grad is not None else torch.zeros_like(x0_in)
                    if d_x0_down is not None:
                        g0 = g0 + d_x0_down
                    out_send = ([x_in.grad, g0], self.stage - 1)
        if out_send is not None:
            _, r0, k0 = self._exchange(out_send, None, act_shape)
            in_flight.append((r0, k0))
        for reqs, _keep in in_flight:
            for r in reqs:
                r.wait()
        self.timer.mark("bwd_end")
        self.comm.reduce_scatter_grads(self.layout)
        progress = self.wsd.progress(self.step)
        gs = self.comm.grad_source(self.layout) if hasattr(self.comm, "grad_source") else None
        self.opt.step(self.step + 1, progress, warmup_multiplier(self.step + 1, self.wsd.warmup_steps), grad_source=gs)
        self.comm.all_gather_params(self.layout)
        self.timer.mark("opt_end")
        self.timer.mark("end")
        self.step += 1
        return self._loss_acc

    def _stage_batch(self, micro: int):
        got = self.prefetch.next()
        slot, h_ids, h_tgt = got
        d_ids, d_tgt = self._d[micro]
        d_ids.copy_(h_ids, non_blocking=True)
        d_tgt.copy_(h_tgt, non_blocking=True)
        ev = None
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
        self.prefetch.release(slot, ev)
        return d_ids, d_tgt

    def global_loss(self, loss: torch.Tensor) -> float:
        """The loss lives on the last stage; share it (mean over DP replicas)."""
        v = loss.detach().clone() if self.last else torch.zeros((), dtype=torch.float32, device=self.device)
        dist.all_reduce(v)
        return float(v.item()) / self.dp

    loss_on_all_ranks = global_loss

    def banner(self):
        m = self.mcfg
        return [f"Model: {m.name} {m.num_params()['total'] / 1e6:.1f}M params, impl={self.impl}, "
                f"dtype={str(self.dtype).split('.')[-1]}, world={self.world}",
                f"Pipeline: {self.pp} stages x dp {self.dp} ({self.comm.name}); stage layers "
                f"{split_layers(m.n_layer, self.pp)}; {self.accum} micro-batches of {self.micro_batch} sequences (1F1B) = "
                f"{self.tokens_per_step} tokens/step"]

    # ---- evaluation: a forward-only pass down the pipeline; the last stage scores ---------------------
    def evaluate(self, max_batches: Optional[int]) -> float:
        from ..eval.bpb import eval_bpb, load_token_bytes
        if self.token_bytes is None:
            self.token_bytes = load_token_bytes(self.tcfg.tokenizer_dir, self.mcfg.vocab, self.device)
        act_shape = (self.micro_batch * self.mcfg.seq_len, self.mcfg.d_model)

        def forward(ids, tgt):
            x_in = x0_in = None
            if not self.first:
                got, reqs, _ = self._exchange(None, self.stage - 1, act_shape)
                for r in reqs:
                    r.wait()
                x_in, x0_in = got
            out = self.model(ids, tgt, x_in=x_in, x0_in=x0_in)
            if self.last:
                return out[1], tgt
            _, reqs, _keep = self._exchange(([out[0], out[1]], self.stage + 1), None, act_shape)
            for r in reqs:
                r.wait()
            return torch.zeros(0, device=self.device), tgt.reshape(-1)[:0]

        return eval_bpb(self.model, self._make_loader("val"), self.token_bytes, max_batches, self.device,
                        group=dist.group.WORLD, forward=forward)

    # ---- checkpoints: every rank its own directory ------------------------------------------------------
    def _dir(self) -> Path:
        return Path(self.tcfg.checkpoint_dir) / f"rank_{self.rank}"

    def save(self, step: Optional[int] = None) -> Optional[str]:
        if hasattr(self.comm, "flush"):
            self.comm.flush()
        state = dict(step=self.step, loss_ema=self.loss_ema, ema_steps=self.ema_steps, wsd=self.wsd.state_dict(),
                     pp=self.pp, dp=self.dp, stage=self.stage, data=self.prefetch.state_dict())
        path = ckpt.save_checkpoint(self.model, self.tcfg.checkpoint_dir, step=step, optimizer=self.opt,
                                    trainer_state=state, subdir=f"rank_{self.rank}")
        dist.barrier()
        # the logging rank reports its own file; every rank has written one
        return path

    def _resume(self):
        from ..ckpt.safetensors_io import load_file
        d = self._dir()
        p = d / "model.safetensors"
        if not p.exists():
            return
        ckpt.load_weights(self.model, str(p), strict=True)
        for gi, st in self.opt.state.items():
            st["master"].copy_(self.layout.group_view(self.layout.flat_param, self.layout.groups[gi]).float())
        if (d / "optim_state.safetensors").exists():
            self.opt.load_state_dict(load_file(str(d / "optim_state.safetensors")))
            for gi, st in self.opt.state.items():           # exact parameters from the fp32 masters
                self.layout.group_view(self.layout.flat_param, self.layout.groups[gi]).copy_(st["master"])
            self.comm.all_gather_params(self.layout)
        sp = d / "trainer_state.json"
        if sp.exists():
            st = json.loads(sp.read_text())
            self.step = int(st["step"])
            self.loss_ema, self.ema_steps = st.get("loss_ema", 0.0), st.get("ema_steps", 0)
            self.wsd.load_state_dict(st["wsd"])
            if st.get("data") and hasattr(self.train_loader, "load_state_dict"):
                self.prefetch.load_state_dict(st["data"])
        self._say(f"Resumed from {d} at step {self.step}")
