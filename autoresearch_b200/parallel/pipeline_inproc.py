"""Pipeline parallelism inside ONE process that drives every GPU of the pipeline.

The reference's first multi-GPU mode (brain/src/pipeline.rs:45-259, brain/src/train.rs:1191-1603):
one context, stream, staged buffer set and GEMM runner per GPU, all-pairs peer access, activations
(x, x0), targets and gradients (d_x, d_x0) moved with peer copies, per-stage checkpoints under
``stage_{i}/``, no evaluation.  There the stages run strictly one after the other with full stream
synchronisations around every transfer.

Here the single host thread walks the merged one-forward-one-backward schedules of all stages and
only ENQUEUES work: every stage has its own device and stream, the peer copies are ordered by
events (the framework's device-to-device copy), nothing waits on the host, so stage s computes
micro-batch i while stage s+1 computes micro-batch i-1.  Each stage owns its slice of the model,
its flat parameter storage and its optimizer; the gradient of x0 is accumulated along the chain.
Loop, logging, timing and checkpoint cadence are the shared ones of ``TrainerBase``; evaluation is
a forward-only walk over the stages.  One process per GPU (``PipelineTrainer``) is the form that
combines with data parallelism; this one needs no launcher and no process group.
"""
from __future__ import annotations

import contextlib
import json
from pathlib import Path
from typing import List, Optional, Sequence, Tuple

import torch

from ..ckpt import checkpoint as ckpt
from ..config import ModelConfig, TrainConfig, derive_accumulation
from ..loop import TrainerBase
from ..models.gpt import GPT
from ..models.init import init_weights
from ..ops.backend import get_backend
from ..optim.muon_adamw import MuonAdamW
from ..optim.schedule import WSDState, warmup_multiplier
from .layout import ParamLayout
from .pipeline import one_f_one_b, split_layers


def merged_schedule(n_stages: int, n_micro: int) -> List[Tuple[int, str, int]]:
    """A single issue order (stage, 'F'|'B', micro-batch) that respects every stage's 1F1B order and the data
    dependencies between stages: F(i) of stage s after F(i) of s-1, B(i) of stage s after B(i) of s+1."""
    per = [one_f_one_b(s, n_stages, n_micro) for s in range(n_stages)]
    pos = [0] * n_stages
    done = set()
    out: List[Tuple[int, str, int]] = []
    total = sum(len(p) for p in per)
    while len(out) < total:
        progressed = False
        for s in range(n_stages):
            while pos[s] < len(per[s]):
                kind, i = per[s][pos[s]]
                dep = (s - 1, "F", i) if kind == "F" else (s + 1, "B", i)
                if 0 <= dep[0] < n_stages and dep not in done:
                    break
                out.append((s, kind, i))
                done.add((s, kind, i))
                pos[s] += 1
                progressed = True
        if not progressed:
            raise RuntimeError("pipeline schedule cannot make progress")
    return out


class InProcPipelineTrainer(TrainerBase):
    def __init__(self, mcfg: ModelConfig, tcfg: TrainConfig, devices: Sequence, quiet: bool = False):
        self.mcfg, self.tcfg = mcfg, tcfg
        self.devices = [torch.device(d) for d in devices]
        self.pp = len(self.devices)
        if self.pp < 1 or self.pp > mcfg.n_layer:
            raise ValueError(f"{self.pp} stages for {mcfg.n_layer} layers")
        self.rank, self.world = 0, self.pp
        self.data_rank, self.data_world = 0, 1
        self.device = self.devices[-1]             # loss, timing events and the error word live on the last stage
        self.quiet = quiet
        on_gpu = all(d.type == "cuda" for d in self.devices)
        impl = tcfg.impl
        if impl == "auto":
            impl = "sm100" if (on_gpu and torch.cuda.get_device_capability(self.devices[0])[0] == 10) else "oracle"
        self.impl = impl
        self.dtype = torch.bfloat16 if on_gpu and impl != "oracle" else torch.float32
        self.micro_batch, self.accum = derive_accumulation(tcfg.total_batch_size, tcfg.device_batch_size, mcfg.seq_len, 1)
        full = GPT(mcfg, get_backend("oracle", mcfg), dtype=torch.float32, device="cpu")
        if tcfg.load_checkpoint or tcfg.init_weights_path:
            ckpt.load_weights(full, tcfg.load_checkpoint or tcfg.init_weights_path, strict=bool(tcfg.load_checkpoint))
        else:
            init_weights(full, seed=tcfg.seed, scheme=getattr(tcfg, "init_scheme", "reference"))
        src = dict(full.named_parameters())
        self.backends, self.models, self.layouts, self.opts = [], [], [], []
        for s, (lo, hi) in enumerate(split_layers(mcfg.n_layer, self.pp)):
            dev = self.devices[s]
            with self._on(dev):
                be = get_backend(impl, mcfg)
                model = GPT(mcfg, be, dtype=self.dtype, device=dev, layer_range=(lo, hi),
                            has_embedding=(s == 0), has_head=(s == self.pp - 1))
                with torch.no_grad():
                    for n, p in model.named_parameters():
                        if n in ("resid_lambdas", "x0_lambdas"):
                            p.copy_(src[n][lo:hi])
                        elif n.startswith("blocks."):
                            parts = n.split(".")
                            parts[1] = str(int(parts[1]) + lo)
                            p.copy_(src[".".join(parts)])
                        else:
                            p.copy_(src[n])
                lay = ParamLayout(model.named_matrix_groups(), 1, 0)
                kernels = getattr(be, "optim_kernels", None)
                opt = MuonAdamW(lay, tcfg.schedule_cfg, mcfg.d_model, kernels=kernels() if callable(kernels) else None)
            self.backends.append(be); self.models.append(model); self.layouts.append(lay); self.opts.append(opt)
        del full, src
        self.model = self.models[-1]
        self.wsd = WSDState(tcfg.max_steps, tcfg.cooldown_steps, tcfg.schedule_cfg.warmdown_ratio,
                            int(round(tcfg.schedule_cfg.warmup_ratio * (tcfg.max_steps or 0))))
        self.sched = merged_schedule(self.pp, self.accum)
        self.comm_bytes = 0
        with self._on(self.device):
            self._init_common()
        B, T = self.micro_batch, mcfg.seq_len
        # the token ids of every micro-batch of a step, on every stage's device (value embeddings need them,
        # the last stage needs the targets); staged from the pinned ring to stage 0 and peer-copied onward
        self._ids = [[torch.empty(B, T, dtype=torch.int32, device=d) for _ in range(self.accum)] for d in self.devices]
        self._tgt = [torch.empty(B, T, dtype=torch.int32, device=self.device) for _ in range(self.accum)]
        if tcfg.resume and tcfg.checkpoint_dir:
            self._resume()

    @staticmethod
    def _on(dev):
        return torch.cuda.device(dev) if dev.type == "cuda" else contextlib.nullcontext()

    def _move(self, t: torch.Tensor, dev) -> torch.Tensor:
        """Peer copy to the next / previous stage (the copy is ordered after its producer and before its consumer by
        the framework's cross-device stream events; the host does not wait)."""
        self.comm_bytes += t.numel() * t.element_size()
        return t.to(dev, non_blocking=True) if t.device != dev else t

    def _stage_inputs(self) -> None:
        for i in range(self.accum):
            slot, h_ids, h_tgt = self.prefetch.next()
            d0 = self.devices[0]
            with self._on(d0):
                self._ids[0][i].copy_(h_ids, non_blocking=True)
                ev = None
                if d0.type == "cuda":
                    ev = torch.cuda.Event()
                    ev.record()
            with self._on(self.device):
                self._tgt[i].copy_(h_tgt, non_blocking=True)
                if self.device.type == "cuda":
                    ev2 = torch.cuda.Event()
                    ev2.record()
                    ev = _Both(ev, ev2) if ev is not None else ev2
            self.prefetch.release(slot, ev)
            for s in range(1, self.pp):
                self._ids[s][i].copy_(self._ids[0][i], non_blocking=True)

    def train_step(self):
        m = self.mcfg
        self._pre_step()
        if not self.step_data_ready():
            return None
        with self._on(self.device):
            self.timer.mark("start")
        self.wsd.update(self.step, triggered=self._cooldown_triggered())
        for s, lay in enumerate(self.layouts):
            with self._on(self.devices[s]):
                lay.zero_grad()
        self._stage_inputs()
        tokens_micro = self.micro_batch * m.seq_len
        grad_scale = 1.0 / (tokens_micro * self.accum)
        with self._on(self.device):
            self._loss_acc.zero_()
        saved = {}
        fwd_out = {}      # (stage, i) -> (x, x0) on the NEXT stage's device
        bwd_out = {}      # (stage, i) -> (d_x, d_x0) on the PREVIOUS stage's device
        last = self.pp - 1
        for s, kind, i in self.sched:
            dev = self.devices[s]
            with self._on(dev):
                if kind == "F":
                    if s == 0:
                        x_in = x0_in = None
                    else:
                        x_in, x0_in = fwd_out.pop((s - 1, i))
                        x_in.requires_grad_(True); x0_in.requires_grad_(True)
                    out = self.models[s](self._ids[s][i], self._tgt[i] if s == last else None, grad_scale=grad_scale,
                                         x_in=x_in, x0_in=x0_in)
                    if s == last:
                        scaled, per_tok = out
                        self._loss_acc += per_tok.sum() / (tokens_micro * self.accum)
                        saved[(s, i)] = (x_in, x0_in, scaled, None)
                    else:
                        x_out, x0_out = out
                        nd = self.devices[s + 1]
                        fwd_out[(s, i)] = (self._move(x_out.detach(), nd), self._move(x0_out.detach(), nd))
                        saved[(s, i)] = (x_in, x0_in, x_out, x0_out)
                else:
                    x_in, x0_in, y, x0_out = saved.pop((s, i))
                    if s == last:
                        y.backward()
                        d_x0_down = None
                    else:
                        d_x, d_x0_down = bwd_out.pop((s + 1, i))
                        if s == 0:
                            torch.autograd.backward([y, x0_out], [d_x, d_x0_down])
                        else:
                            torch.autograd.backward([y], [d_x])
                    self.layouts[s].accumulate_autograd_grads()
                    if s > 0:
                        g0 = x0_in.grad if x0_in.grad is not None else torch.zeros_like(x0_in)
                        if d_x0_down is not None:
                            g0 = g0 + d_x0_down
                        pd = self.devices[s - 1]
                        bwd_out[(s, i)] = (self._move(x_in.grad, pd), self._move(g0, pd))
        with self._on(self.device):
            self.timer.mark("bwd_end")
        progress = self.wsd.progress(self.step)
        wm = warmup_multiplier(self.step + 1, self.wsd.warmup_steps)
        for s, opt in enumerate(self.opts):
            with self._on(self.devices[s]):
                opt.step(self.step + 1, progress, wm)
        with self._on(self.device):
            self.timer.mark("opt_end")
            self.timer.mark("end")
        self.step += 1
        return self._loss_acc

    def _kernel_error(self) -> Optional[str]:
        if self.impl != "sm100":
            return None
        from ..ops import kernels as K
        for s, dev in enumerate(self.devices):
            try:
                with self._on(dev):
                    torch.cuda.synchronize(dev)
                    K.check_err_flag(dev)
            except K.KernelError as e:
                return f"stage {s}: {e}"
        return None

    def banner(self):
        m = self.mcfg
        return [f"Model: {m.name} {m.num_params()['total'] / 1e6:.1f}M params, impl={self.impl}, "
                f"dtype={str(self.dtype).split('.')[-1]}, {self.pp} GPUs in one process",
                f"Pipeline (in-process, peer copies): stage layers {split_layers(m.n_layer, self.pp)}; "
                f"{self.accum} micro-batches of {self.micro_batch} sequences (1F1B) = {self.tokens_per_step} tokens/step"]

    # ---- evaluation: forward-only walk over the stages -----------------------------------------------
    def evaluate(self, max_batches: Optional[int]) -> float:
        from ..eval.bpb import eval_bpb, load_token_bytes
        if self.token_bytes is None:
            self.token_bytes = load_token_bytes(self.tcfg.tokenizer_dir, self.mcfg.vocab, self.device)

        def forward(ids, tgt):
            x = x0 = None
            for s, model in enumerate(self.models):
                dev = self.devices[s]
                with self._on(dev):
                    ids_s = ids.to(dev, non_blocking=True)
                    if s == self.pp - 1:
                        return model(ids_s, tgt, x_in=x, x0_in=x0)[1], tgt
                    x, x0 = model(ids_s, None, x_in=x, x0_in=x0)
                    nd = self.devices[s + 1]
                    x, x0 = x.to(nd, non_blocking=True), x0.to(nd, non_blocking=True)

        for mdl in self.models[:-1]:
            mdl.eval()
        try:
            with self._on(self.device):
                return eval_bpb(self.model, self._make_loader("val"), self.token_bytes, max_batches, self.device,
                                forward=forward)
        finally:
            for mdl in self.models[:-1]:
                mdl.train()

    # ---- checkpoints: one directory per stage -----------------------------------------------------------
    def save(self, step: Optional[int] = None) -> Optional[str]:
        state = dict(step=self.step, loss_ema=self.loss_ema, ema_steps=self.ema_steps, wsd=self.wsd.state_dict(),
                     pp=self.pp, data=self.prefetch.state_dict())
        path = None
        for s in range(self.pp):
            with self._on(self.devices[s]):
                path = ckpt.save_checkpoint(self.models[s], self.tcfg.checkpoint_dir, step=step, optimizer=self.opts[s],
                                            trainer_state=state, subdir=f"stage_{s}")
        return str(Path(path).parent.parent) if path else None

    def _resume(self):
        from ..ckpt.safetensors_io import load_file
        root = Path(self.tcfg.checkpoint_dir)
        if not (root / "stage_0" / "model.safetensors").exists():
            return
        for s in range(self.pp):
            d = root / f"stage_{s}"
            with self._on(self.devices[s]):
                ckpt.load_weights(self.models[s], str(d / "model.safetensors"), strict=True)
                lay, opt = self.layouts[s], self.opts[s]
                for gi, st in opt.state.items():
                    st["master"].copy_(lay.group_view(lay.flat_param, lay.groups[gi]).float())
                if (d / "optim_state.safetensors").exists():
                    opt.load_state_dict(load_file(str(d / "optim_state.safetensors")))
                    for gi, st in opt.state.items():
                        lay.group_view(lay.flat_param, lay.groups[gi]).copy_(st["master"])
        sp = root / "stage_0" / "trainer_state.json"
        if sp.exists():
            st = json.loads(sp.read_text())
            self.step = int(st["step"])
            self.loss_ema, self.ema_steps = st.get("loss_ema", 0.0), st.get("ema_steps", 0)
            self.wsd.load_state_dict(st["wsd"])
            if st.get("data") and hasattr(self.train_loader, "load_state_dict"):
                self.prefetch.load_state_dict(st["data"])
        self._say(f"Resumed from {root} at step {self.step}")


class _Both:
    """Two copy-complete events of one pinned slot (its ids went to stage 0, its targets to the last stage)."""

    def __init__(self, a, b):
        self.a, self.b = a, b

    def synchronize(self):
        self.a.synchronize()
        self.b.synchronize()
