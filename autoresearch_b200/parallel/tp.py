"""Tensor parallelism with sequence-sharded activations (Megatron-style TP+SP), for the wide
configuration (TP=2 x DP=4 on 8 GPUs).

The reference has no tensor parallelism.  Per layer and TP rank:

    x_shard [N/tp, D] --resid-scale-norm--> xn_shard --ALL-GATHER--> xn [N, D]
    qkv = xn Wqkv_local^T (H/tp heads) -> RoPE/QK-norm/VE -> attention -> a [N, D/tp]
    partial = a Wo_local^T [N, D] --REDUCE-SCATTER--> + x_shard --norm--> xn_shard
    ... same pattern for the MLP (Wfc column-parallel, Wdn row-parallel).

Embedding, final norm, LM head and the loss run on the local token shard with replicated
weights.  Two communication arms:

* ``library`` – torch.distributed all_gather / reduce_scatter (NCCL or gloo): the baseline.
* ``fused``   – peer memory, tied into the tcgen05 GEMMs (``FusedTPContext.gemm_rs`` /
  ``ag_gemm``): GEMM -> reduce-scatter runs the GEMM once per destination rank with that rank's
  staging slab as its output, so every finished 256 x 256 tile leaves the epilogue as TMA stores
  over NVLink while the tensor cores work on the next tile, and a local kernel sums the slabs;
  all-gather -> GEMM pulls the peers' row blocks (NVLink loads) on a side stream while the GEMM
  already multiplies the local rows, and multiplies the pulled rows when they have arrived.  The
  pulled rows are kept in local memory because each of them is read by every column tile of the
  GEMM; reading them from the peer inside the GEMM would cross NVLink once per column tile.
"""
from __future__ import annotations

import ctypes as C
import json
from pathlib import Path
from typing import List, Optional

import torch
import torch.distributed as dist

from ..config import ModelConfig, TrainConfig, derive_accumulation
from ..models.gpt import GPT
from ..models.init import init_weights
from ..ops.backend import get_backend
from ..optim.muon_adamw import MuonAdamW
from ..loop import TrainerBase
from ..optim.schedule import WSDState, warmup_multiplier
from .dp import LibraryComm, LocalComm
from .layout import ParamLayout


class _AllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return tp.all_gather_rows(x)

    @staticmethod
    def backward(ctx, g):
        return ctx.tp.reduce_scatter_rows(g.contiguous()), None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return tp.reduce_scatter_rows(x)

    @staticmethod
    def backward(ctx, g):
        return ctx.tp.all_gather_rows(g.contiguous()), None


class TPContext:
    """Library arm (works on gloo CPU ranks and NCCL)."""

    mode = "library"

    def __init__(self, group, rank: int, size: int):
        self.group, self.rank, self.size = group, rank, size
        self.bytes = 0

    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty((x.shape[0] * self.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        self.bytes += out.numel() * out.element_size()
        if dist.get_backend(self.group) == "gloo":
            parts = list(out.chunk(self.size, 0))
            dist.all_gather(parts, x.contiguous(), group=self.group)
        else:
            dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def reduce_scatter_rows(self, x: torch.Tensor) -> torch.Tensor:
        n = x.shape[0] // self.size
        self.bytes += x.numel() * x.element_size()
        if dist.get_backend(self.group) == "gloo":
            y = x.clone()
            dist.all_reduce(y, group=self.group)
            return y[self.rank * n:(self.rank + 1) * n].contiguous()
        out = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group)
        return out

    def all_gather(self, x):
        return _AllGather.apply(x, self)

    def reduce_scatter(self, x):
        return _ReduceScatter.apply(x, self)


class FusedTPContext(TPContext):
    """Peer-memory arm (CUDA only): see the module docstring."""

    mode = "fused"

    def __init__(self, group, rank, size, device, max_rows: int, d_model: int):
        super().__init__(group, rank, size)
        from ..ops import kernels as K
        from .symm import SymmBuffer
        self.K = K
        self.device = torch.device(device)
        self.D = d_model
        self.max_rows = max_rows
        self.n_max = max_rows // size
        # Both staging areas are double buffered: a rank writes half k%2 of a peer during operation k and the
        # peer reads it after barrier k; the same half is written again only in operation k+2, i.e. after the
        # writer has passed barrier k+1, which the reader enters only after its reads of operation k.
        self.ag = SymmBuffer(2 * self.n_max * d_model, torch.bfloat16, self.device, group)       # [2][n, D] my shard
        self.rs = SymmBuffer(2 * max_rows * d_model, torch.bfloat16, self.device, group)         # [2][src][n, D]
        self.flags = SymmBuffer(64, torch.int32, self.device, group)
        for b in (self.ag, self.rs, self.flags):
            b.rendezvous()
        dist.barrier(group=group)
        self._flag_ptrs = (C.c_void_p * size)(*self.flags.peer_ptrs)
        self.epoch = 0
        self.n_ag = self.n_rs = 0
        self.side = torch.cuda.Stream(device=self.device)

    def barrier(self):
        self.epoch += 1
        self.K._check(self.K.lib().arb_peer_barrier(self._flag_ptrs, self.size, self.rank, self.epoch,
                                                    self.K.err_flag(self.device).data_ptr(), self.K._stream()), "peer_barrier")

    # ---- all-gather ---------------------------------------------------------------------------
    def _publish_and_pull(self, x, out):
        """Copy the local shard into this rank's staging half, then, on the side stream, pull every peer's shard
        into its rows of `out`.  Returns the event that marks the arrival of the pulled rows."""
        K = self.K
        n, D = x.shape
        half = self.n_ag & 1
        self.n_ag += 1
        off = half * self.n_max * self.D
        self.ag.tensor[off: off + n * D].view(n, D).copy_(x)
        self.barrier()                                          # every shard of this operation is published
        self.bytes += n * (self.size - 1) * D * 2
        main = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(self.side):
            self.side.wait_event(ready)
            # the pull kernel addresses the peers' staging halves as shards of one virtual [size*n, D] tensor
            ptrs = (C.c_void_p * self.size)(*[p + off * 2 - r * n * D * 2 for r, p in enumerate(self.ag.peer_ptrs)])
            K._check(K.lib().arb_all_gather_pull(ptrs, self.size, self.rank, out.data_ptr(), n * D * 2, self.side.cuda_stream),
                     "tp_all_gather_pull")
            arrived = torch.cuda.Event()
            arrived.record(self.side)
        out.record_stream(self.side)
        return arrived

    def all_gather_rows(self, x):
        n, D = x.shape
        if x.dtype != torch.bfloat16 or n > self.n_max or D != self.D:
            return super().all_gather_rows(x)
        out = torch.empty(n * self.size, D, dtype=x.dtype, device=x.device)
        arrived = self._publish_and_pull(x, out)
        out[self.rank * n:(self.rank + 1) * n].copy_(x)
        torch.cuda.current_stream(self.device).wait_event(arrived)
        return out

    def ag_gemm(self, x, w, trans_b=True, epi=None, aux=None):
        """(all-gather of the row shards x) @ op(w): returns the product [size*n, cols] and the gathered
        operand (the backward needs it).  The local rows are multiplied while the peers' rows travel."""
        K = self.K
        n, D = x.shape
        if x.dtype != torch.bfloat16 or n > self.n_max or D != self.D:
            xf = super().all_gather_rows(x)
            return K.gemm(xf, w, trans_b=trans_b, epi=epi if epi is not None else K.EPI_STORE_BF16, aux=aux), xf
        epi = K.EPI_STORE_BF16 if epi is None else epi
        N = n * self.size
        cols = w.shape[0] if trans_b else w.shape[1]
        xf = torch.empty(N, D, dtype=x.dtype, device=x.device)
        y = torch.empty(N, cols, dtype=torch.bfloat16, device=x.device)
        arrived = self._publish_and_pull(x, xf)
        lo, hi = self.rank * n, (self.rank + 1) * n
        xf[lo:hi].copy_(x)
        K.gemm(x, w, trans_b=trans_b, out=y[lo:hi], epi=epi, aux=None if aux is None else aux[lo:hi])
        torch.cuda.current_stream(self.device).wait_event(arrived)
        for a, b in ((0, lo), (hi, N)):                         # the row blocks of the other ranks
            if b > a:
                K.gemm(xf[a:b], w, trans_b=trans_b, out=y[a:b], epi=epi, aux=None if aux is None else aux[a:b])
        return y, xf

    # ---- reduce-scatter -----------------------------------------------------------------------
    def _reduce_slabs(self, half, n, D):
        """Sum of the `size` source slabs of staging half `half` -> [n, D] bf16 (local reads only)."""
        K = self.K
        base = self.rs.tensor.data_ptr() + half * self.max_rows * self.D * 2
        ptrs = (C.c_void_p * self.size)(*[base + s * self.n_max * self.D * 2 for s in range(self.size)])
        out = torch.empty(n, D, dtype=torch.bfloat16, device=self.device)
        K._check(K.lib().arb_sum_slabs_bf16(ptrs, self.size, n * D, out.data_ptr(), K._stream()), "tp_reduce_slabs")
        return out

    def _slab(self, dst_rank, half, n, D):
        """Rank `dst_rank`'s staging slab for rows sent by this rank, as an [n, D] tensor."""
        off = (half * self.max_rows + self.rank * self.n_max) * self.D
        if dst_rank == self.rank:
            return self.rs.tensor[off: off + n * D].view(n, D)
        return self.rs.peer_tensor(dst_rank, (n, D), torch.bfloat16, off)

    def reduce_scatter_rows(self, x):
        N, D = x.shape
        if x.dtype != torch.bfloat16 or N > self.max_rows or D != self.D or N % self.size:
            return super().reduce_scatter_rows(x)
        n = N // self.size
        half = self.n_rs & 1
        self.n_rs += 1
        self.bytes += (N - n) * D * 2
        # one kernel of this package stores every row block into its owner's slab (peer stores over NVLink)
        x = x.contiguous()
        K = self.K
        order = [(self.rank + 1 + i) % self.size for i in range(self.size)]
        off = (half * self.max_rows + self.rank * self.n_max) * self.D * 2
        src = (C.c_void_p * self.size)(*[x.data_ptr() + r * n * D * 2 for r in order])
        dst = (C.c_void_p * self.size)(*[self.rs.peer_ptrs[r] + off for r in order])
        nb = (C.c_longlong * self.size)(*[n * D * 2] * self.size)
        K._check(K.lib().arb_pull_ranges(src, dst, nb, self.size, K._stream()), "tp_push_rows")
        self.barrier()
        return self._reduce_slabs(half, n, D)

    def gemm_rs(self, a, w, trans_b=True):
        """Row block `rank` of sum over ranks of (a @ op(w)).  The GEMM runs once per destination rank with that
        rank's staging slab as its output: the tiles leave the epilogue as TMA stores over NVLink."""
        K = self.K
        N = a.shape[0]
        D = w.shape[0] if trans_b else w.shape[1]
        if a.dtype != torch.bfloat16 or N > self.max_rows or D != self.D or N % self.size:
            return super().reduce_scatter_rows(K.gemm(a, w, trans_b=trans_b))
        n = N // self.size
        half = self.n_rs & 1
        self.n_rs += 1
        self.bytes += (N - n) * D * 2
        for i in range(self.size):                              # peers first: their tiles have the longer way
            r = (self.rank + 1 + i) % self.size
            K.gemm(a[r * n:(r + 1) * n], w, trans_b=trans_b, out=self._slab(r, half, n, D))
        self.barrier()                                          # all slabs of this operation have arrived
        return self._reduce_slabs(half, n, D)


def shard_full_model_into(full: GPT, model: GPT, tp_rank: int, tp: int) -> None:
    """Copy rank `tp_rank`'s slices of a full model's weights into a TP-sharded model."""
    cfg = full.cfg
    D = cfg.d_model
    Dl = D // tp
    sl = slice(tp_rank * Dl, (tp_rank + 1) * Dl)
    with torch.no_grad():
        for name in ("wte", "lm_head", "resid_lambdas", "x0_lambdas"):
            getattr(model, name).copy_(getattr(full, name))
        for fb, mb in zip(full.blocks, model.blocks):
            q, k, v = fb.wqkv[:D], fb.wqkv[D:2 * D], fb.wqkv[2 * D:]
            mb.wqkv.copy_(torch.cat([q[sl], k[sl], v[sl]], 0))
            mb.wo.copy_(fb.wo[:, sl])
            if fb.wfc is not None:
                M = fb.wfc.shape[0] // tp
                mb.wfc.copy_(fb.wfc[tp_rank * M:(tp_rank + 1) * M])
                mb.wdn.copy_(fb.wdn[:, tp_rank * M:(tp_rank + 1) * M])
            if fb.ve is not None:
                mb.ve.copy_(fb.ve[:, sl])
                H = fb.ve_gate.shape[0] // tp
                mb.ve_gate.copy_(fb.ve_gate[tp_rank * H:(tp_rank + 1) * H])


def gather_full_model(model: GPT, tp_group, tp_rank: int, tp: int) -> Optional[GPT]:
    """Inverse of shard_full_model_into: every rank of the TP group sends its slices (collective), rank 0 of the
    group returns a full fp32 CPU model, the others None.  Used to write the standard single-file checkpoint."""
    cfg = model.cfg

    def gather(t: torch.Tensor) -> List[torch.Tensor]:
        parts = [torch.empty_like(t) for _ in range(tp)]
        dist.all_gather(parts, t.detach().contiguous(), group=tp_group)
        return [p.float().cpu() for p in parts]

    full = GPT(cfg, get_backend("oracle", cfg), dtype=torch.float32, device="cpu") if tp_rank == 0 else None
    with torch.no_grad():
        if full is not None:
            for name in ("wte", "lm_head", "resid_lambdas", "x0_lambdas"):
                getattr(full, name).copy_(getattr(model, name).detach().float().cpu())
        for i, mb in enumerate(model.blocks):
            fb = full.blocks[i] if full is not None else None
            Dl = cfg.d_model // tp
            qkv = gather(mb.wqkv)
            wo = gather(mb.wo)
            if fb is not None:
                fb.wqkv.copy_(torch.cat([torch.cat([p[j * Dl:(j + 1) * Dl] for p in qkv], 0) for j in range(3)], 0))
                fb.wo.copy_(torch.cat(wo, 1))
            if mb.wfc is not None:
                fc, dn = gather(mb.wfc), gather(mb.wdn)
                if fb is not None:
                    fb.wfc.copy_(torch.cat(fc, 0))
                    fb.wdn.copy_(torch.cat(dn, 1))
            if mb.ve is not None:
                ve, gate = gather(mb.ve), gather(mb.ve_gate)
                if fb is not None:
                    fb.ve.copy_(torch.cat(ve, 1))
                    fb.ve_gate.copy_(torch.cat(gate, 0))
    return full


REPLICATED_KINDS = ("adamw_emb", "adamw_head", "adamw_lr", "adamw_l0", "adamw_router")


class TPTrainer(TrainerBase):
    """world = tp x dp; rank = dp_index * tp + tp_rank.  A TP group shares one micro-batch.  The step loop, logging,
    timing, evaluation and checkpoint cadence are the shared ones of ``TrainerBase``."""

    def __init__(self, mcfg: ModelConfig, tcfg: TrainConfig, tp: int, device: str = "cpu", quiet: bool = False):
        if not dist.is_initialized():
            raise RuntimeError("tensor parallelism needs an initialised process group (torchrun)")
        if mcfg.moe is not None:
            raise ValueError("tensor parallelism is implemented for the dense model")
        self.mcfg, self.tcfg, self.tp = mcfg, tcfg, tp
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        if self.world % tp or mcfg.n_head % tp:
            raise ValueError("world size and head count must be multiples of tp")
        self.dp = self.world // tp
        self.tp_rank, self.dp_idx = self.rank % tp, self.rank // tp
        self.data_rank, self.data_world = self.dp_idx, self.dp
        self.device = torch.device(device)
        self.quiet = quiet
        on_gpu = self.device.type == "cuda"
        impl = tcfg.impl
        if impl == "auto":
            impl = "sm100" if (on_gpu and torch.cuda.get_device_capability(self.device)[0] == 10) else "oracle"
        self.impl = impl
        self.dtype = torch.bfloat16 if on_gpu and impl != "oracle" else torch.float32
        self.tp_group = self.dp_group = None
        for d in range(self.dp):
            g = dist.new_group([d * tp + t for t in range(tp)])
            if d == self.dp_idx:
                self.tp_group = g
        for t in range(tp):
            g = dist.new_group([d * tp + t for d in range(self.dp)])
            if t == self.tp_rank:
                self.dp_group = g
        self.micro_batch, self.accum = derive_accumulation(tcfg.total_batch_size, tcfg.device_batch_size,
                                                           mcfg.seq_len, self.dp)
        n_tokens = self.micro_batch * mcfg.seq_len
        if n_tokens % tp:
            raise ValueError("tokens per micro-batch must divide over tp")
        self.backend = get_backend(impl, mcfg)
        fused = tcfg.parallel.comm == "fused" and on_gpu and impl == "sm100"
        if fused:
            self.backend.tp = FusedTPContext(self.tp_group, self.tp_rank, tp, self.device, n_tokens, mcfg.d_model)
        else:
            self.backend.tp = TPContext(self.tp_group, self.tp_rank, tp)
        self.model = GPT(mcfg, self.backend, dtype=self.dtype, device=self.device, tp=tp)
        full = GPT(mcfg, get_backend("oracle", mcfg), dtype=torch.float32, device="cpu")
        if tcfg.load_checkpoint or tcfg.init_weights_path:
            from ..ckpt import checkpoint as ckpt
            ckpt.load_weights(full, tcfg.load_checkpoint or tcfg.init_weights_path, strict=bool(tcfg.load_checkpoint))
        else:
            init_weights(full, seed=tcfg.seed, scheme=getattr(tcfg, "init_scheme", "reference"))
        shard_full_model_into(full, self.model, self.tp_rank, tp)
        del full
        groups = self.model.named_matrix_groups()
        rep = [g for g in groups if g[2] in REPLICATED_KINDS]
        shd = [g for g in groups if g[2] not in REPLICATED_KINDS]
        # replicated parameters: gradients summed over ALL ranks; sharded ones over the DP group of this TP index.
        # With the peer-memory arm both exchanges are the fused data-parallel path (reduce-scatter inside the
        # optimizer kernels, all-gather inside the consuming GEMMs), each over its own group.
        self.comm_rep = self._make_dp_comm(None, self.world, fused)
        self.lay_rep = ParamLayout(rep, self.world, self.rank, allocator=getattr(self.comm_rep, "allocator", None))
        if hasattr(self.comm_rep, "attach"):
            self.comm_rep.attach(self.lay_rep)
        self.comm_shd = self._make_dp_comm(self.dp_group, self.dp, fused)
        self.lay_shd = ParamLayout(shd, self.dp, self.dp_idx, allocator=getattr(self.comm_shd, "allocator", None))
        if hasattr(self.comm_shd, "attach"):
            self.comm_shd.attach(self.lay_shd)
        kernels = getattr(self.backend, "optim_kernels", None)
        kk = kernels() if callable(kernels) else None
        self.opt_rep = MuonAdamW(self.lay_rep, tcfg.schedule_cfg, mcfg.d_model, kernels=kk)
        self.opt_shd = MuonAdamW(self.lay_shd, tcfg.schedule_cfg, mcfg.d_model, kernels=kk)
        self.wsd = WSDState(tcfg.max_steps, tcfg.cooldown_steps, tcfg.schedule_cfg.warmdown_ratio,
                            int(round(tcfg.schedule_cfg.warmup_ratio * (tcfg.max_steps or 0))))
        self._init_common()
        self.plan_memory(dp=self.dp, tp=tp, fused_dp=fused and self.dp > 1,
                         act_bytes=2 if self.dtype == torch.bfloat16 else 4,
                         ce_chunk=max(mcfg.ce_chunk, getattr(self.backend, "big_ce_chunk", 0)))
        if tcfg.resume and tcfg.checkpoint_dir:
            self._resume()

    def _make_dp_comm(self, group, size: int, fused: bool):
        if size == 1:
            return LocalComm()
        if fused:
            from .fused_dp import FusedComm
            return FusedComm(group, self.device)
        return LibraryComm(group, torch.bfloat16 if self.device.type == "cuda" else None)

    @property
    def comm_name(self) -> str:
        return f"tp-{self.backend.tp.mode}+dp-{self.comm_shd.name if self.dp > 1 else self.comm_rep.name}"

    @property
    def comm_bytes(self) -> int:
        return int(self.backend.tp.bytes)

    def train_step(self):
        m = self.mcfg
        self._pre_step()
        if not self.step_data_ready():
            return None
        self.timer.mark("start")
        self.wsd.update(self.step, triggered=self._cooldown_triggered())
        self.lay_rep.zero_grad(); self.lay_shd.zero_grad()
        n_tokens = self.micro_batch * m.seq_len
        grad_scale = 1.0 / (n_tokens * self.accum * self.dp)
        self._loss_acc.zero_()
        for micro in range(self.accum):
            ids, tgt = self._stage_batch(micro)
            scaled, per_tok = self.model(ids, tgt, grad_scale=grad_scale)
            scaled.backward()
            self.lay_rep.accumulate_autograd_grads(); self.lay_shd.accumulate_autograd_grads()
            self._loss_acc += per_tok.sum() / (n_tokens * self.accum)
        self.timer.mark("bwd_end")
        self.comm_rep.reduce_scatter_grads(self.lay_rep)
        self.comm_shd.reduce_scatter_grads(self.lay_shd)
        progress = self.wsd.progress(self.step)
        wm = warmup_multiplier(self.step + 1, self.wsd.warmup_steps)
        src = lambda c, lay: c.grad_source(lay) if hasattr(c, "grad_source") else None
        self.opt_rep.step(self.step + 1, progress, wm, grad_source=src(self.comm_rep, self.lay_rep))
        self.opt_shd.step(self.step + 1, progress, wm, grad_source=src(self.comm_shd, self.lay_shd))
        self.comm_rep.all_gather_params(self.lay_rep)
        self.comm_shd.all_gather_params(self.lay_shd)
        self.timer.mark("opt_end")
        self.timer.mark("end")
        self.step += 1
        return self._loss_acc

    # ---- evaluation: every rank scores its token shard of its replica's batch -----------------------
    def evaluate(self, max_batches: Optional[int]) -> float:
        from ..eval.bpb import eval_bpb, load_token_bytes
        if self.token_bytes is None:
            self.token_bytes = load_token_bytes(self.tcfg.tokenizer_dir, self.mcfg.vocab, self.device)
        n = (self.micro_batch * self.mcfg.seq_len) // self.tp
        shard = slice(self.tp_rank * n, (self.tp_rank + 1) * n)

        def forward(ids, tgt):
            _, per_tok = self.model(ids, tgt)
            return per_tok, tgt.reshape(-1)[shard]

        return eval_bpb(self.model, self._make_loader("val"), self.token_bytes, max_batches, self.device,
                        group=dist.group.WORLD, forward=forward)

    # ---- checkpoints --------------------------------------------------------------------------------
    def _flush(self):
        for c in (self.comm_rep, self.comm_shd):
            if hasattr(c, "flush"):
                c.flush()

    def save(self, step: Optional[int] = None) -> Optional[str]:
        """One standard checkpoint file (full, unsharded tensors), written by rank 0: the TP group of the first
        DP replica gathers its shards (collective within that group).  Optimizer state is written per rank."""
        from ..ckpt import checkpoint as ckpt
        from ..ckpt.safetensors_io import save_file
        self._flush()
        d = Path(self.tcfg.checkpoint_dir)
        d.mkdir(parents=True, exist_ok=True)
        osd = dict(self.opt_rep.state_dict())
        osd.update(self.opt_shd.state_dict())
        save_file(osd, str(d / f"optim_state.rank{self.rank}.safetensors"))
        path = None
        if self.dp_idx == 0:
            full = gather_full_model(self.model, self.tp_group, self.tp_rank, self.tp)
            if full is not None:
                state = dict(step=self.step, loss_ema=self.loss_ema, ema_steps=self.ema_steps, wsd=self.wsd.state_dict(),
                             tp=self.tp, dp=self.dp, world=self.world, data=self.prefetch.state_dict())
                path = ckpt.save_checkpoint(full, str(d), step=step, trainer_state=state)
        dist.barrier()
        return path

    def _resume(self):
        from ..ckpt import checkpoint as ckpt
        from ..ckpt.safetensors_io import load_file
        d = Path(self.tcfg.checkpoint_dir)
        p = d / "model.safetensors"
        if not p.exists():
            return
        full = GPT(self.mcfg, get_backend("oracle", self.mcfg), dtype=torch.float32, device="cpu")
        ckpt.load_weights(full, str(p), strict=True)
        shard_full_model_into(full, self.model, self.tp_rank, self.tp)
        del full
        for opt, lay in ((self.opt_rep, self.lay_rep), (self.opt_shd, self.lay_shd)):
            for gi, st in opt.state.items():
                st["master"].copy_(lay.group_view(lay.flat_param, lay.groups[gi]).float())
        f = d / f"optim_state.rank{self.rank}.safetensors"
        sp = d / "trainer_state.json"
        if sp.exists():
            st = json.loads(sp.read_text())
            if f.exists() and (st.get("tp"), st.get("world")) == (self.tp, self.world):
                sd = load_file(str(f))
                for opt, lay, comm in ((self.opt_rep, self.lay_rep, self.comm_rep), (self.opt_shd, self.lay_shd, self.comm_shd)):
                    opt.load_state_dict(sd)
                    for gi, ost in opt.state.items():       # exact parameters from the fp32 masters
                        lay.group_view(lay.flat_param, lay.groups[gi]).copy_(ost["master"])
                    comm.all_gather_params(lay)
            self.step = int(st["step"])
            self.loss_ema, self.ema_steps = st.get("loss_ema", 0.0), st.get("ema_steps", 0)
            self.wsd.load_state_dict(st["wsd"])
            if st.get("data") and hasattr(self.train_loader, "load_state_dict"):
                self.prefetch.load_state_dict(st["data"])
        self._say(f"Resumed from {d} at step {self.step}")

    def global_loss(self, loss: torch.Tensor) -> float:
        """Each rank holds the loss of its token shard (already divided by the full micro-batch
        token count): sum over the TP group, mean over DP replicas."""
        v = loss.detach().clone()
        dist.all_reduce(v)
        return float(v.item()) / self.dp

    def banner(self):
        m = self.mcfg
        return [f"Model: {m.name} {m.num_params()['total'] / 1e6:.1f}M params, impl={self.impl}, "
                f"dtype={str(self.dtype).split('.')[-1]}, world={self.world}",
                f"Tensor parallel: tp {self.tp} x dp {self.dp} ({self.comm_name}); "
                f"{self.micro_batch} x {m.seq_len} x accum {self.accum} per TP group = {self.tokens_per_step} tokens/step"]
