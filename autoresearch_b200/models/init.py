"""Weight initialisation.

Scheme (brain/src/train.rs:2268-2346; original/train.py:148-180): s = 0.68*sqrt(3)/sqrt(D);
wte ~ N(0,1); lm_head ~ N(0, 0.001); Wq, Wk, Wv, Wfc, value embeddings ~ U(-s, s);
Wo, Wdn, ve_gate = 0; resid_lambdas = 1.0, x0_lambdas = 0.1; MoE: router = 0,
expert fc ~ U(-s, s), expert proj = 0.  Random numbers come from one process-wide
xorshift64 stream seeded 42 with Box-Muller normals (brain/src/train.rs:2424-2483), drawn
in the reference's order: wte, lm_head, then per layer wq, wk, wv, wfc, ve, experts.

scheme="torch" draws from PyTorch's CPU generator in the call order of the upstream Python trainer's
``init_weights`` (original/train.py:148-180, reproduced by brain/tools/generate_init_weights.py:48-91):
``torch.manual_seed(seed)``; wte normal_(0, 1); lm_head normal_(0, 0.001); for every layer c_q, c_k, c_v,
c_fc uniform_(-s, s) as separate fp32 tensors; then the value embeddings uniform_(-s, s) in layer order.
A file written with it starts this engine and the Python trainer from bit-identical bf16 weights.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import torch

from .. import native


class InitRng:
    def __init__(self, seed: int = 42):
        self.state = C.c_uint64(seed)
        self.lib = native.lib()

    def uniform(self, shape, bound: float, dtype) -> torch.Tensor:
        n = int(np.prod(shape))
        if dtype == torch.bfloat16:
            buf = np.empty(n, dtype=np.uint16)
            self.lib.ar_uniform_bf16(C.byref(self.state), n, float(bound), buf.ctypes.data)
            return torch.from_numpy(buf.view(np.int16)).view(torch.bfloat16).view(*shape)
        buf = np.empty(n, dtype=np.float32)
        self.lib.ar_uniform_f32(C.byref(self.state), n, float(bound), buf.ctypes.data)
        return torch.from_numpy(buf).view(*shape).to(dtype)

    def normal(self, shape, scale: float, dtype) -> torch.Tensor:
        n = int(np.prod(shape))
        buf = np.empty(n, dtype=np.float32)
        self.lib.ar_randn_f32(C.byref(self.state), n, float(scale), buf.ctypes.data)
        return torch.from_numpy(buf).view(*shape).to(dtype)


@torch.no_grad()
def init_weights(model, seed: int = 42, scheme: str = "reference", std: float = 0.02) -> None:
    """scheme="reference": the engine's scheme above.  scheme="normal": every matrix
    N(0, std) (used by the CPU plumbing configuration so that no output is identically
    zero at step 0)."""
    cfg = model.cfg
    D = cfg.d_model
    rng = InitRng(seed)
    s = cfg.init_scale * math.sqrt(3.0) / math.sqrt(D)

    def put(p, t):
        p.data.copy_(t.to(p.device, p.dtype).view(p.shape))

    if scheme == "normal":
        g = torch.Generator().manual_seed(seed)
        for _, p, kind in model.named_matrix_groups():
            if kind == "adamw_lr":
                p.data.fill_(1.0)
            elif kind == "adamw_l0":
                p.data.fill_(0.1)
            elif kind == "muon_expert" and getattr(model, "ep", 1) > 1:
                full = (cfg.moe.n_experts,) + tuple(p.shape[1:])
                r0 = model.ep_rank * p.shape[0]
                put(p, (torch.randn(full, generator=g) * std)[r0:r0 + p.shape[0]])
            else:
                put(p, torch.randn(p.shape, generator=g) * std)
        return

    if scheme == "torch":
        if cfg.moe is not None or getattr(model, "tp", 1) > 1 or model.layer_lo != 0 or model.layer_hi != cfg.n_layer:
            raise ValueError('scheme="torch" initialises a full dense model (shard or warm-start it afterwards)')
        g = torch.Generator().manual_seed(seed)
        V = cfg.vocab
        put(model.wte, torch.empty(V, D).normal_(0.0, 1.0, generator=g))
        put(model.lm_head, torch.empty(V, D).normal_(0.0, 0.001, generator=g))
        for blk in model.blocks:
            q, k, v = (torch.empty(D, D).uniform_(-s, s, generator=g) for _ in range(3))
            put(blk.wqkv, torch.cat([q, k, v], 0))
            blk.wo.data.zero_()
            put(blk.wfc, torch.empty(cfg.mlp_dim, D).uniform_(-s, s, generator=g))
            blk.wdn.data.zero_()
        model.resid_lambdas.data.fill_(1.0)
        model.x0_lambdas.data.fill_(0.1)
        for blk in model.blocks:
            if blk.ve is not None:
                put(blk.ve, torch.empty(V, D).uniform_(-s, s, generator=g))
                blk.ve_gate.data.zero_()
        return

    dt = model.dtype
    if model.wte is not None:
        put(model.wte, rng.normal(model.wte.shape, 1.0, dt))
    if model.lm_head is not None:
        put(model.lm_head, rng.normal(model.lm_head.shape, 0.001, dt))
    model.resid_lambdas.data.fill_(1.0)
    model.x0_lambdas.data.fill_(0.1)
    for blk in model.blocks:
        put(blk.wqkv, rng.uniform(blk.wqkv.shape, s, dt))
        blk.wo.data.zero_()
        if blk.wfc is not None:
            put(blk.wfc, rng.uniform(blk.wfc.shape, s, dt))
            blk.wdn.data.zero_()
        if blk.ve is not None:
            put(blk.ve, rng.uniform(blk.ve.shape, s, dt))
            blk.ve_gate.data.zero_()
        if blk.router is not None:
            blk.router.data.zero_()
            # draw all E experts so every expert-parallel rank sees the single-process stream
            el = blk.expert_fc.shape[0]
            full = (cfg.moe.n_experts,) + tuple(blk.expert_fc.shape[1:])
            allw = rng.uniform(full, s, dt)
            r0 = getattr(model, "ep_rank", 0) * el
            put(blk.expert_fc, allw[r0:r0 + el])
            blk.expert_proj.data.zero_()
