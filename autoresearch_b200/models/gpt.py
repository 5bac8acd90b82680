"""GPT with parameter-free RMSNorm, RoPE + QK-norm, ReLU^2 MLP (or top-k MoE), value
embeddings with a sigmoid gate, learned residual / x0-skip scalars, SSSSL sliding-window
attention and a soft-capped LM head.

The sequence of operations per layer follows the reference engine's forward pass
(brain/src/forward.rs:359-739; readable form original/train.py:267-290).  The module is
written against an ops backend (`autoresearch_b200.ops.backend`) so the same graph runs
on the pure-PyTorch oracle, the library baseline, or the sm_100a kernels.

A model can be built for a contiguous slice of layers (pipeline stage): stage 0 owns the
token embedding, the last stage owns the LM head and the loss, every stage holds the
slices of `resid_lambdas` / `x0_lambdas` of its own layers (brain/src/train.rs:1652-1669).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from ..utils.timing import nvtx_range
from ..config import ModelConfig
from ..ops import reference as R


class Block(nn.Module):
    def __init__(self, cfg: ModelConfig, layer: int, dtype, device, tp: int = 1, ep: int = 1):
        super().__init__()
        D, M = cfg.d_model, cfg.mlp_dim
        self.layer = layer
        self.cfg = cfg
        self.tp = tp
        kw = dict(dtype=dtype, device=device)
        # wq, wk, wv are three row blocks of one packed matrix: the QKV GEMM reads it as a
        # single [3D, D] operand and Muon treats each [D, D] block as its own matrix.
        self.wqkv = nn.Parameter(torch.empty(3 * D // tp, D, **kw))
        self.wo = nn.Parameter(torch.empty(D, D // tp, **kw))
        if cfg.has_ve(layer):
            self.ve = nn.Parameter(torch.empty(cfg.vocab, D // tp, **kw))
            self.ve_gate = nn.Parameter(torch.empty(cfg.n_kv_head // tp, cfg.ve_gate_ch, **kw))
        else:
            self.ve = None
            self.ve_gate = None
        if cfg.is_moe_layer(layer):
            E, ME = cfg.moe.n_experts, cfg.moe.mlp_dim_e
            self.router = nn.Parameter(torch.empty(E, D, **kw))
            # with expert parallelism a rank holds E / ep experts; the router scores all E
            self.expert_fc = nn.Parameter(torch.empty(E // ep, ME, D, **kw))
            self.expert_proj = nn.Parameter(torch.empty(E // ep, D, ME, **kw))
            self.wfc = None
            self.wdn = None
        else:
            self.wfc = nn.Parameter(torch.empty(M // tp, D, **kw))
            self.wdn = nn.Parameter(torch.empty(D, M // tp, **kw))
            self.router = None
        if tp > 1:
            # Muon's learning-rate factor sqrt(max(1, m/n)) refers to the unsharded matrix
            self.wqkv.muon_full_shape = (D, D)
            self.wo.muon_full_shape = (D, D)
            if self.wfc is not None:
                self.wfc.muon_full_shape = (M, D)
                self.wdn.muon_full_shape = (D, M)


class GPT(nn.Module):
    def __init__(self, cfg: ModelConfig, backend=None, dtype=torch.float32, device="cpu",
                 layer_range: Optional[Tuple[int, int]] = None,
                 has_embedding: bool = True, has_head: bool = True, tp: int = 1, ep: int = 1,
                 ep_rank: int = 0):
        super().__init__()
        from ..ops.backend import get_backend
        self.cfg = cfg
        self.backend = backend if backend is not None else get_backend("oracle")
        self.dtype = dtype
        self.tp = tp
        self.ep, self.ep_rank = ep, ep_rank
        lo, hi = layer_range if layer_range is not None else (0, cfg.n_layer)
        self.layer_lo, self.layer_hi = lo, hi
        self.has_embedding = has_embedding
        self.has_head = has_head
        kw = dict(dtype=dtype, device=device)
        D, V = cfg.d_model, cfg.vocab
        self.wte = nn.Parameter(torch.empty(V, D, **kw)) if has_embedding else None
        self.lm_head = nn.Parameter(torch.empty(V, D, **kw)) if has_head else None
        self.resid_lambdas = nn.Parameter(torch.empty(hi - lo, **kw))
        self.x0_lambdas = nn.Parameter(torch.empty(hi - lo, **kw))
        self.blocks = nn.ModuleList([Block(cfg, l, dtype, device, tp, ep) for l in range(lo, hi)])
        cos, sin = R.rope_tables(cfg.seq_len, cfg.head_dim, cfg.rope_base, device=device)
        # bf16 tables like the reference (brain/src/train.rs:2402-2422) when running in bf16
        tdt = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
        self.register_buffer("rope_cos", cos.to(tdt), persistent=False)
        self.register_buffer("rope_sin", sin.to(tdt), persistent=False)
        self.aux_loss = None
        # {layer: bucket}: when the backward pass has produced the gradient of that layer's input, the parameter
        # gradients of gradient bucket `bucket` (that layer and everything above it) are final; the trainer sets
        # `grad_bucket_cb(bucket)` for the micro-step after which the data-parallel exchange may start early
        self.grad_bucket_boundaries = {}
        self.grad_bucket_cb = None

    # ------------------------------------------------------------------
    def embed(self, ids: torch.Tensor) -> torch.Tensor:
        be = self.backend
        emb = be.embedding(ids.reshape(-1), self.wte)
        return be.rmsnorm(emb)

    def run_layers(self, x: torch.Tensor, x0: torch.Tensor, ids: torch.Tensor,
                   B: int, T: int) -> torch.Tensor:
        cfg, be = self.cfg, self.backend
        ids_flat = ids.reshape(-1)
        aux_total = None
        for bi, blk in enumerate(self.blocks):
            l = blk.layer
            if self.grad_bucket_cb is not None and l in self.grad_bucket_boundaries and x.requires_grad:
                cb, b = self.grad_bucket_cb, self.grad_bucket_boundaries[l]
                x.register_hook(lambda g, cb=cb, b=b: cb(b))
            with nvtx_range(f"layer {l}"):
                x, xn = be.resid_scale_norm(x, x0, self.resid_lambdas, self.x0_lambdas, bi)
                a = be.attention_block(xn, blk, ids_flat, B, T, cfg, self.rope_cos, self.rope_sin,
                                       cfg.window(l))
                x, xn = be.proj_add_norm(a, blk.wo, x)
                if blk.router is not None:
                    x, aux = be.moe_mlp_add(xn, x, blk, cfg.moe)
                    aux_total = aux if aux_total is None else aux_total + aux
                else:
                    x = be.mlp_add(xn, blk.wfc, blk.wdn, x)
        self.aux_loss = aux_total
        return x

    def head_loss(self, x: torch.Tensor, targets: torch.Tensor, grad_scale: float = 1.0):
        """Returns (loss_sum scaled by grad_scale for backward, per-token losses [N] fp32,
        detached)."""
        be = self.backend
        xf = be.rmsnorm(x)
        return be.lm_head_ce(xf, self.lm_head, targets.reshape(-1), grad_scale)

    def forward(self, ids: torch.Tensor, targets: Optional[torch.Tensor] = None,
                grad_scale: float = 1.0, x_in: Optional[torch.Tensor] = None,
                x0_in: Optional[torch.Tensor] = None):
        """ids/targets: [B, T] integer tensors.  Full model: returns
        (scaled_loss_sum, per_token_losses).  Pipeline stage without a head: returns (x, x0)."""
        B, T = ids.shape
        tp = getattr(self.backend, "tp", None)
        if tp is not None and tp.size > 1:
            # sequence parallel: this rank embeds, normalises and scores only its token shard
            n = (B * T) // tp.size
            shard = slice(tp.rank * n, (tp.rank + 1) * n)
            ids_emb = ids.reshape(-1)[shard]
            targets = targets.reshape(-1)[shard] if targets is not None else None
        else:
            ids_emb = ids
        if self.has_embedding:
            x = self.embed(ids_emb)
            x0 = x
        else:
            x, x0 = x_in, x0_in
        x = self.run_layers(x, x0, ids, B, T)
        if not self.has_head:
            return x, x0
        scaled, per_tok = self.head_loss(x, targets, grad_scale)
        if self.aux_loss is not None:
            # aux loss is a per-micro-batch mean quantity; scale it like a mean loss
            scaled = scaled + self.aux_loss * (grad_scale * B * T)
        return scaled, per_tok

    # ------------------------------------------------------------------
    def named_matrix_groups(self):
        """(name, parameter, kind) for every parameter, where kind selects the optimizer
        rule (brain/src/optim.rs:198-220)."""
        out = []
        if self.wte is not None:
            out.append(("wte", self.wte, "adamw_emb"))
        if self.lm_head is not None:
            out.append(("lm_head", self.lm_head, "adamw_head"))
        out.append(("resid_lambdas", self.resid_lambdas, "adamw_lr"))
        out.append(("x0_lambdas", self.x0_lambdas, "adamw_l0"))
        for blk in self.blocks:
            l = blk.layer
            out.append((f"h.{l}.wqkv", blk.wqkv, "muon_qkv"))
            out.append((f"h.{l}.wo", blk.wo, "muon"))
            if blk.wfc is not None:
                out.append((f"h.{l}.wfc", blk.wfc, "muon"))
                out.append((f"h.{l}.wdn", blk.wdn, "muon"))
            if blk.ve is not None:
                out.append((f"h.{l}.ve", blk.ve, "adamw_ve"))
                out.append((f"h.{l}.ve_gate", blk.ve_gate, "muon"))
            if blk.router is not None:
                out.append((f"h.{l}.router", blk.router, "adamw_router"))
                out.append((f"h.{l}.expert_fc", blk.expert_fc, "muon_expert"))
                out.append((f"h.{l}.expert_proj", blk.expert_proj, "muon_expert"))
        return out
