"""Pipeline parallelism with a 1F1B schedule over point-to-point sends (NCCL on GPUs, gloo on
CPU ranks).

What is kept from the reference (brain/src/train.rs:1620-2029, brain/src/pipeline.rs:45-259):
one rank per stage; layers split ``L // n`` with the remainder on the early stages; stage 0 owns
the token embedding, the last stage owns the LM head and the loss; every stage keeps and
updates only its own slice of ``resid_lambdas`` / ``x0_lambdas``; ``x`` and ``x0`` travel forward
together; checkpoints go to ``stage_{i}/`` sub-directories.

What is different: the reference runs one micro-batch through all stages strictly in sequence
(bubble (n-1)/n) with blocking sends; here micro-batches are interleaved one-forward-one-backward
and transfers are posted asynchronously so they overlap compute.  The gradient of ``x0`` is
accumulated along the chain (each boundary carries d_x and d_x0 back) instead of every stage
sending its partial sum to stage 0.  Pipeline stages can be combined with data parallelism:
rank = dp_index * n_stages + stage.
"""
from __future__ import annotations

import time
from typing import List, Tuple

import torch
import torch.distributed as dist

from ..ckpt import checkpoint as ckpt
from ..config import ModelConfig, TrainConfig, derive_accumulation
from ..models.gpt import GPT
from ..models.init import init_weights
from ..ops.backend import get_backend
from ..optim.muon_adamw import MuonAdamW
from ..optim.schedule import WSDState, lr_multiplier, warmup_multiplier
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


class PipelineTrainer:
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
        self.device = torch.device(device)
        self.quiet = quiet
        on_gpu = self.device.type == "cuda"
        impl = tcfg.impl
        if impl == "auto":
            impl = "sm100" if (on_gpu and torch.cuda.get_device_capability(self.device)[0] == 10) else "oracle"
        self.dtype = torch.bfloat16 if on_gpu and impl != "oracle" else torch.float32
        self.backend = get_backend(impl, mcfg)
        # process groups: one DP group per stage (collective creation: every rank calls all)
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
        self.comm = LocalComm() if self.dp == 1 else LibraryComm(self.dp_group,
                                                                 torch.bfloat16 if on_gpu else None)
        self.layout = ParamLayout(self.model.named_matrix_groups(), self.dp, self.dp_idx)
        kernels = getattr(self.backend, "optim_kernels", None)
        self.opt = MuonAdamW(self.layout, tcfg.schedule_cfg, mcfg.d_model, kernels=kernels() if callable(kernels) else None)
        self.wsd = WSDState(tcfg.max_steps, tcfg.cooldown_steps, tcfg.schedule_cfg.warmdown_ratio,
                            int(round(tcfg.schedule_cfg.warmup_ratio * (tcfg.max_steps or 0))))
        self.step = 0
        from ..trainer import Trainer
        self.loader = Trainer._make_loader(self._loader_shim(), "train")
        self.sched = one_f_one_b(self.stage, pp, self.accum)
        self.comm_bytes = 0

    # the single-GPU trainer's loader factory only needs these attributes
    def _loader_shim(self):
        class S: pass
        s = S()
        s.tcfg, s.mcfg, s.micro_batch = self.tcfg, self.mcfg, self.micro_batch
        s.rank, s.world = self.dp_idx, self.dp
        return s

    def _init_stage_weights(self):
        """Initialise the full model once per rank with the shared seed and keep this stage's
        slice, so that a pipelined run starts from the same weights as a single-process run."""
        t = self.tcfg
        if t.load_checkpoint:
            ckpt.load_weights(self.model, t.load_checkpoint, strict=True)
            return
        full = GPT(self.mcfg, get_backend("oracle", self.mcfg), dtype=torch.float32, device="cpu")
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

    # ------------------------------------------------------------------
    def _send(self, tensors, dst_stage) -> list:
        dst = self.dp_idx * self.pp + dst_stage
        hs = []
        for t in tensors:
            t = t.contiguous()
            self.comm_bytes += t.numel() * t.element_size()
            hs.append((dist.isend(t, dst), t))
        return hs

    def _recv(self, shapes, src_stage) -> list:
        src = self.dp_idx * self.pp + src_stage
        out = []
        for shp in shapes:
            buf = torch.empty(shp, dtype=self.dtype, device=self.device)
            out.append((dist.irecv(buf, src), buf))
        return out

    def train_step(self):
        m = self.mcfg
        self.wsd.update(self.step)
        self.layout.zero_grad()
        B, T, D = self.micro_batch, m.seq_len, m.d_model
        act_shape = (B * T, D)
        tokens_micro = B * T
        grad_scale = 1.0 / (tokens_micro * self.accum * self.dp)
        batches = [self.loader.next_batch() for _ in range(self.accum)]
        if any(b is None for b in batches):
            return None
        batches = [(i.to(self.device), t.to(self.device)) for i, t in batches]
        saved = {}
        pending = []
        loss_acc = torch.zeros((), dtype=torch.float32, device=self.device)
        for kind, i in self.sched:
            ids, tgt = batches[i]
            if kind == "F":
                if self.first:
                    x_in = x0_in = None
                else:
                    (hx, x_in), (h0, x0_in) = self._recv([act_shape, act_shape], self.stage - 1)
                    hx.wait(); h0.wait()
                    x_in.requires_grad_(True); x0_in.requires_grad_(True)
                out = self.model(ids, tgt, grad_scale=grad_scale, x_in=x_in, x0_in=x0_in)
                if self.last:
                    scaled, per_tok = out
                    loss_acc += per_tok.sum() / (tokens_micro * self.accum)
                    saved[i] = (x_in, x0_in, scaled, None)
                else:
                    x_out, x0_out = out
                    pending += self._send([x_out.detach(), x0_out.detach()], self.stage + 1)
                    saved[i] = (x_in, x0_in, x_out, x0_out)
            else:
                x_in, x0_in, y, x0_out = saved.pop(i)
                if self.last:
                    y.backward()
                    d_x0_down = None
                else:
                    (hx, d_x), (h0, d_x0_down) = self._recv([act_shape, act_shape], self.stage + 1)
                    hx.wait(); h0.wait()
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
                    pending += self._send([x_in.grad, g0], self.stage - 1)
        for h, _keep in pending:
            h.wait()
        self.comm.reduce_scatter_grads(self.layout)
        progress = self.wsd.progress(self.step)
        self.opt.step(self.step + 1, progress, warmup_multiplier(self.step + 1, self.wsd.warmup_steps))
        self.comm.all_gather_params(self.layout)
        self.step += 1
        return loss_acc

    def loss_on_all_ranks(self, loss: torch.Tensor) -> float:
        """The loss lives on the last stage; share it (mean over DP replicas)."""
        v = loss.detach().clone() if self.last else torch.zeros((), dtype=torch.float32, device=self.device)
        dist.all_reduce(v)
        return float(v.item()) / self.dp

    def run(self):
        t = self.tcfg
        tokens = self.micro_batch * self.mcfg.seq_len * self.accum * self.dp
        if self.rank == 0 and not self.quiet:
            print(f"Pipeline: {self.pp} stages x dp {self.dp}; stage layers {split_layers(self.mcfg.n_layer, self.pp)}; "
                  f"{self.accum} micro-batches of {self.micro_batch} sequences (1F1B)", flush=True)
        ema, n = 0.0, 0
        while not self.wsd.finished(self.step):
            t0 = time.perf_counter()
            loss = self.train_step()
            if loss is None:
                break
            if self.device.type == "cuda":
                torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            step = self.step - 1
            if step % t.log_interval == 0 or step <= 10:
                lv = self.loss_on_all_ranks(loss)
                ema = 0.9 * ema + 0.1 * lv; n += 1
                if self.rank == self.world - 1 and not self.quiet:
                    lrm = lr_multiplier(self.wsd.progress(step), t.schedule_cfg)
                    left = (t.max_steps - self.step) if t.max_steps else -1
                    print(f"step {step:>5} | loss {ema / (1 - 0.9 ** n):.4f} | lr {lrm:.3f} | dt {dt:.3f}s | "
                          f"tok/s {int(tokens / dt)} | mfu 0.0% | vram 0MB | steps_left {left}", flush=True)
        if t.checkpoint_dir and not t.synthetic_data and self.dp_idx == 0:
            p = ckpt.save_checkpoint(self.model, t.checkpoint_dir, subdir=f"stage_{self.stage}")
            print(f"[checkpoint] saved {p}", flush=True)
        dist.barrier()
