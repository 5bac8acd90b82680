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
from pathlib import Path
from typing import Optional

import torch
import torch.distributed as dist

from .ckpt import checkpoint as ckpt
from .config import ModelConfig, TrainConfig, derive_accumulation
from .eval.bpb import eval_bpb, load_token_bytes
from .loop import DeviceFault, TrainerBase
from .models.gpt import GPT
from .models.init import init_weights
from .ops.backend import get_backend
from .optim.muon_adamw import MuonAdamW
from .optim.schedule import WSDState, warmup_multiplier
from .parallel.dp import LibraryComm, LocalComm
from .parallel.layout import ParamLayout
from .utils.timing import nvtx_range


class Trainer(TrainerBase):
    """One data-parallel replica group training a full (non-pipelined) model."""

    def __init__(self, mcfg: ModelConfig, tcfg: TrainConfig, device: Optional[str] = None,
                 group=None, quiet: bool = False):
        self.mcfg, self.tcfg = mcfg, tcfg
        self.dist = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank(group) if self.dist else 0
        self.world = dist.get_world_size(group) if self.dist else 1
        self.group = group
        self.quiet = quiet
        self.data_rank, self.data_world = self.rank, self.world
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
        # gradient buckets by depth (only the peer-memory exchange overlaps with the backward pass)
        self.n_buckets = 1
        bucket_of = None
        if getattr(self.comm, "name", "") == "fused" and tcfg.parallel.dp_buckets > 1 and mcfg.n_layer >= 2:
            self.n_buckets = min(int(tcfg.parallel.dp_buckets), mcfg.n_layer)
            bucket_of = self._bucket_of
        self.layout = ParamLayout(dense_groups, self.world, self.rank, allocator=alloc, bucket_of=bucket_of,
                                  n_buckets=self.n_buckets)
        if hasattr(self.comm, "attach"):
            self.comm.attach(self.layout)
        if self.n_buckets > 1:
            L_, nb = mcfg.n_layer, self.n_buckets
            lowest = {}
            for l in range(L_):
                lowest[self._layer_bucket(l)] = min(l, lowest.get(self._layer_bucket(l), l))
            # the last bucket ends with the embeddings: it is exchanged after the backward pass, not from a hook
            self.model.grad_bucket_boundaries = {l: b for b, l in lowest.items() if b < nb - 1}
            self._side = torch.cuda.Stream(device=self.device)
        kernels = getattr(self.backend, "optim_kernels", None)
        self.opt = MuonAdamW(self.layout, tcfg.schedule_cfg, mcfg.d_model,
                             kernels=kernels() if callable(kernels) else None)
        # expert-parallel experts are unique to their rank: no reduction, a rank-local optimizer
        self.expert_layout = self.expert_opt = None
        if expert_groups:
            self.expert_layout = ParamLayout(expert_groups, 1, 0)
            self.expert_opt = MuonAdamW(self.expert_layout, tcfg.schedule_cfg, mcfg.d_model,
                                        kernels=kernels() if callable(kernels) else None)
            from .parallel.ep import EPContext, LibraryEPContext
            ctx_cls = EPContext if tcfg.parallel.comm == "fused" else LibraryEPContext
            self.backend.ep = ctx_cls(self.group if self.group is not None else dist.group.WORLD, self.device,
                                      mcfg.moe.n_experts, mcfg.d_model, self.micro_batch * mcfg.seq_len,
                                      mcfg.moe.top_k, mcfg.moe.capacity_factor)
        self.wsd = WSDState(tcfg.max_steps, tcfg.cooldown_steps, tcfg.schedule_cfg.warmdown_ratio,
                            warmup_steps=int(round(tcfg.schedule_cfg.warmup_ratio * (tcfg.max_steps or 0))))
        self._init_common()
        self.plan_memory(dp=self.world, ep=self.ep, fused_dp=(self.comm.name == "fused"),
                         act_bytes=2 if self.dtype == torch.bfloat16 else 4,
                         ce_chunk=max(mcfg.ce_chunk, getattr(self.backend, "big_ce_chunk", 0)))
        if tcfg.resume and tcfg.checkpoint_dir:
            self._resume()

    # ------------------------------------------------------------------
    def _layer_bucket(self, layer: int) -> int:
        """Upper layers finish their backward first: bucket 0 = the top third, ..., the last bucket = the bottom."""
        return (self.mcfg.n_layer - 1 - layer) * self.n_buckets // self.mcfg.n_layer

    def _bucket_of(self, name: str) -> int:
        parts = name.split(".")
        if parts[0] == "h" and len(parts) > 1 and parts[1].isdigit():
            return self._layer_bucket(int(parts[1]))
        return self.n_buckets - 1            # embeddings, head, per-layer scalar vectors

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
        files = sorted(glob.glob(str(d / "optim_state*.safetensors")))
        for f in files:
            self.opt.load_state_dict(load_file(f))
        if files:
            # the weight file holds bf16 roundings; the fp32 masters are the exact parameters: owners rewrite
            # their shards from them and everyone fetches the rest, as after an optimizer step
            for gi, st in self.opt.state.items():
                self.layout.group_view(self.layout.flat_param, self.layout.groups[gi]).copy_(st["master"])
            self.comm.all_gather_params(self.layout)
        sp = d / "trainer_state.json"
        if sp.exists():
            st = json.loads(sp.read_text())
            self.step = int(st["step"])
            self.loss_ema, self.ema_steps = st["loss_ema"], st["ema_steps"]
            self.wsd.load_state_dict(st["wsd"])
            if hasattr(self.train_loader, "load_state_dict") and st.get("data"):
                self.prefetch.load_state_dict(st["data"])
        self._say(f"Resumed from {d} at step {self.step}")

    # ------------------------------------------------------------------
    def train_step(self) -> Optional[float]:
        """One optimizer step (accum micro-steps).  Returns the mean loss as a device
        scalar tensor (no host sync) or None when the data source is exhausted."""
        m, t = self.mcfg, self.tcfg
        self._pre_step()
        if not self.step_data_ready():
            return None
        self.timer.mark("start")
        self.wsd.update(self.step, triggered=self._cooldown_triggered())
        self.layout.zero_grad()
        if self.expert_layout is not None:
            self.expert_layout.zero_grad()
        self._loss_acc.zero_()
        tokens_micro = self.micro_batch * m.seq_len
        grad_scale = 1.0 / (tokens_micro * self.accum * self.world)
        overlap = self.n_buckets > 1 and t.diagnostic_steps is None
        progress = self.wsd.progress(self.step)
        wm = warmup_multiplier(self.step + 1, self.wsd.warmup_steps)

        def run_optimizer(bucket, src):
            self.opt.step(self.step + 1, progress, wm, grad_source=src, bucket=bucket)

        def bucket_ready(bucket):             # fires inside the last micro-step's backward pass
            with nvtx_range(f"gradient exchange, bucket {bucket}"):
                self.comm.exchange_bucket(self.layout, bucket, run_optimizer, self._side)

        for micro in range(self.accum):
            ids, tgt = self._stage_batch(micro)
            self.model.grad_bucket_cb = bucket_ready if (overlap and micro == self.accum - 1) else None
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
        if overlap:
            self.model.grad_bucket_cb = None
            bucket_ready(self.n_buckets - 1)                 # the bottom layers, embeddings and scalars
            if self.expert_opt is not None:
                self.expert_opt.step(self.step + 1, progress, wm)
            torch.cuda.current_stream(self.device).wait_stream(self._side)
            self.comm.activate_staged()
        else:
            with nvtx_range("gradient exchange"):
                self.comm.reduce_scatter_grads(self.layout)
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

    def _print_grad_norms(self):
        for a in self.layout.atoms:
            for u in a.units:
                g = self.layout.flat_grad[u.offset:u.offset + u.numel]
                self._say(f"[diag] step {self.step} {u.name} grad_norm {g.float().norm().item():.6e}")

    # ------------------------------------------------------------------
    def global_loss(self, loss: torch.Tensor) -> float:
        if self.world > 1:
            l = loss.detach().clone()
            dist.all_reduce(l, group=self.group)
            return float(l.item()) / self.world
        return float(loss.item())

    mean_loss_across_ranks = global_loss

    def banner(self):
        m = self.mcfg
        return [f"Model: {m.name} {m.num_params()['total'] / 1e6:.1f}M params, impl={self.impl}, "
                f"dtype={str(self.dtype).split('.')[-1]}, world={self.world} ({self.comm.name})",
                f"Batch: {self.micro_batch} x {m.seq_len} x accum {self.accum} x dp {self.world} = "
                f"{self.tokens_per_step} tokens/step",
                self.layout.describe()]

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
                     data=self.prefetch.state_dict())
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
