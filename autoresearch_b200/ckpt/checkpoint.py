"""Checkpoint save / load in the reference's layout, plus exact-resume side-cars.

Weight file (brain/src/train.rs:2632-2743): safetensors, every tensor BF16, names
``wte.weight``, ``lm_head.weight``, ``resid_lambdas``, ``x0_lambdas``,
``h.{i}.attn.c_q|c_k|c_v|c_proj.weight``, ``h.{i}.mlp.c_fc|c_proj.weight``,
``ve.{i}.weight``, ``h.{i}.attn.ve_gate.weight``, ``h.{i}.moe.router.weight``,
``h.{i}.moe.expert.{e}.fc|proj.weight``; file ``model.safetensors`` or
``model_step{N}.safetensors``.  Import also accepts the Python state-dict names and F32
tensors, warm-starts a MoE model from a dense checkpoint and expands the vocabulary
(brain/src/init_weights.rs:16-42,379-444,494-527).

The reference never stores optimizer state; resume there restarts moments, step and data
position.  Here ``optim_state.safetensors`` and ``trainer_state.json`` are written beside
the weights so that a resumed run continues exactly.
"""
from __future__ import annotations

import json
import math
import os
import re
from pathlib import Path
from typing import Dict, Optional

import torch

from .safetensors_io import load_file, save_file

_PY2ENGINE = [
    (re.compile(r"^transformer\.wte\.weight$"), "wte.weight"),
    (re.compile(r"^transformer\.h\.(\d+)\.(.+)$"), r"h.\1.\2"),
    (re.compile(r"^value_embeds\.(\d+)\.weight$"), r"ve.\1.weight"),
]


def engine_name(name: str) -> str:
    for pat, rep in _PY2ENGINE:
        if pat.match(name):
            return pat.sub(rep, name)
    return name


def model_to_engine_tensors(model, expert_gather=None, materialise: bool = True) -> Dict[str, torch.Tensor]:
    """Flat engine-named BF16 tensors of a (full or pipeline-stage) model."""
    cfg = model.cfg
    out: Dict[str, torch.Tensor] = {}
    if not materialise:
        # a rank that only takes part in the expert gathers of an expert-parallel save (collective calls)
        for blk in model.blocks:
            if blk.router is not None and expert_gather is not None:
                expert_gather(blk.expert_fc); expert_gather(blk.expert_proj)
        return out
    bf = lambda t: t.detach().to(torch.bfloat16).cpu().contiguous()
    if model.wte is not None:
        out["wte.weight"] = bf(model.wte)
    if model.lm_head is not None:
        out["lm_head.weight"] = bf(model.lm_head)
    out["resid_lambdas"] = bf(model.resid_lambdas)
    out["x0_lambdas"] = bf(model.x0_lambdas)
    for blk in model.blocks:
        i = blk.layer
        D = blk.wqkv.shape[0] // 3
        out[f"h.{i}.attn.c_q.weight"] = bf(blk.wqkv[:D])
        out[f"h.{i}.attn.c_k.weight"] = bf(blk.wqkv[D:2 * D])
        out[f"h.{i}.attn.c_v.weight"] = bf(blk.wqkv[2 * D:])
        out[f"h.{i}.attn.c_proj.weight"] = bf(blk.wo)
        if blk.wfc is not None:
            out[f"h.{i}.mlp.c_fc.weight"] = bf(blk.wfc)
            out[f"h.{i}.mlp.c_proj.weight"] = bf(blk.wdn)
        if blk.ve is not None:
            out[f"ve.{i}.weight"] = bf(blk.ve)
            out[f"h.{i}.attn.ve_gate.weight"] = bf(blk.ve_gate)
        if blk.router is not None:
            out[f"h.{i}.moe.router.weight"] = bf(blk.router)
            fc, pr = blk.expert_fc, blk.expert_proj
            if expert_gather is not None:      # expert parallelism: collect the other ranks' experts
                fc, pr = expert_gather(fc), expert_gather(pr)
            for e in range(fc.shape[0]):
                out[f"h.{i}.moe.expert.{e}.fc.weight"] = bf(fc[e])
                out[f"h.{i}.moe.expert.{e}.proj.weight"] = bf(pr[e])
    return out


def checkpoint_path(ckpt_dir: str, step: Optional[int] = None) -> str:
    name = "model.safetensors" if step is None else f"model_step{step}.safetensors"
    return str(Path(ckpt_dir) / name)


def save_checkpoint(model, ckpt_dir: str, step: Optional[int] = None, optimizer=None,
                    trainer_state: Optional[dict] = None, subdir: Optional[str] = None, expert_gather=None) -> str:
    """`expert_gather(t)`: with expert parallelism, returns the [E, ...] stack of all ranks' experts for this
    rank's [E_local, ...] stack (a collective every rank of the group has to enter, see the trainer)."""
    d = Path(ckpt_dir) / subdir if subdir else Path(ckpt_dir)
    d.mkdir(parents=True, exist_ok=True)
    path = checkpoint_path(str(d), step)
    save_file(model_to_engine_tensors(model, expert_gather=expert_gather), path)
    if optimizer is not None:
        save_file(optimizer.state_dict(), str(d / "optim_state.safetensors"))
    if trainer_state is not None:
        tmp = d / "trainer_state.json.tmp"
        tmp.write_text(json.dumps(trainer_state, indent=1, sort_keys=True))
        os.replace(tmp, d / "trainer_state.json")
    return path


def _expand_vocab(t: torch.Tensor, vocab: int, gen: torch.Generator) -> torch.Tensor:
    if t.shape[0] == vocab:
        return t
    if t.shape[0] > vocab:
        raise ValueError(f"checkpoint vocabulary {t.shape[0]} exceeds the model's {vocab}")
    extra = torch.randn(vocab - t.shape[0], t.shape[1], generator=gen) * 0.02
    return torch.cat([t.float(), extra], 0)


@torch.no_grad()
def load_weights(model, path: str, strict: bool = True, seed: int = 42) -> Dict[str, int]:
    """Load engine- or Python-named tensors (BF16 or F32) into `model`.  A dense checkpoint
    loaded into a MoE model warm-starts the experts: expert 0 is a copy of the dense MLP
    (first mlp_dim_e hidden units), the others a copy plus N(0, 0.01*||W||_F/sqrt(numel)),
    the router is zero."""
    raw = load_file(path)
    sd = {engine_name(k): v for k, v in raw.items()}
    cfg = model.cfg
    gen = torch.Generator().manual_seed(seed)
    stats = {"loaded": 0, "warm_started": 0, "missing": 0}

    def put(p, name, t=None, expand=False):
        t = sd.get(name) if t is None else t
        if t is None:
            if strict:
                raise KeyError(f"{path}: missing tensor {name}")
            stats["missing"] += 1
            return
        if expand:
            t = _expand_vocab(t, p.shape[0], gen)
        if tuple(t.shape) != tuple(p.shape):
            raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)} != model {tuple(p.shape)}")
        p.data.copy_(t.to(p.dtype))
        stats["loaded"] += 1

    if model.wte is not None:
        put(model.wte, "wte.weight", expand=True)
    if model.lm_head is not None:
        put(model.lm_head, "lm_head.weight", expand=True)
    lo, hi = model.layer_lo, model.layer_hi
    for nm, p in (("resid_lambdas", model.resid_lambdas), ("x0_lambdas", model.x0_lambdas)):
        t = sd.get(nm)
        if t is not None and t.numel() == cfg.n_layer and p.numel() != cfg.n_layer:
            t = t[lo:hi]
        put(p, nm, t)
    for blk in model.blocks:
        i = blk.layer
        q, k, v = (sd.get(f"h.{i}.attn.c_{c}.weight") for c in "qkv")
        if q is None or k is None or v is None:
            if strict:
                raise KeyError(f"{path}: missing attention weights of layer {i}")
            stats["missing"] += 3
        else:
            put(blk.wqkv, f"h.{i}.attn.qkv", torch.cat([q, k, v], 0))
            stats["loaded"] += 2
        put(blk.wo, f"h.{i}.attn.c_proj.weight")
        if blk.ve is not None:
            put(blk.ve, f"ve.{i}.weight", expand=True)
            put(blk.ve_gate, f"h.{i}.attn.ve_gate.weight")
        if blk.wfc is not None:
            put(blk.wfc, f"h.{i}.mlp.c_fc.weight")
            put(blk.wdn, f"h.{i}.mlp.c_proj.weight")
        if blk.router is not None:
            E, ME, D = blk.expert_fc.shape
            if f"h.{i}.moe.router.weight" in sd:
                put(blk.router, f"h.{i}.moe.router.weight")
                base = int(getattr(model, "ep_rank", 0)) * E if int(getattr(model, "ep", 1)) > 1 else 0
                for e in range(E):            # E = experts held by this rank; `base` = id of its first expert
                    blk.expert_fc.data[e].copy_(sd[f"h.{i}.moe.expert.{base + e}.fc.weight"].to(blk.expert_fc.dtype))
                    blk.expert_proj.data[e].copy_(sd[f"h.{i}.moe.expert.{base + e}.proj.weight"].to(blk.expert_proj.dtype))
                    stats["loaded"] += 2
            elif f"h.{i}.mlp.c_fc.weight" in sd:
                fc = sd[f"h.{i}.mlp.c_fc.weight"].float()[:ME]
                pr = sd[f"h.{i}.mlp.c_proj.weight"].float()[:, :ME]
                s_fc = 0.01 * fc.norm().item() / math.sqrt(fc.numel())
                s_pr = 0.01 * pr.norm().item() / math.sqrt(pr.numel())
                ep_on = int(getattr(model, "ep", 1)) > 1
                base = int(getattr(model, "ep_rank", 0)) * E if ep_on else 0
                n_total = model.cfg.moe.n_experts if ep_on else E
                for g in range(n_total):      # every rank draws the noise of all experts, in order, and keeps its own
                    nf = 0 if g == 0 else torch.randn(fc.shape, generator=gen) * s_fc
                    np_ = 0 if g == 0 else torch.randn(pr.shape, generator=gen) * s_pr
                    if base <= g < base + E:
                        blk.expert_fc.data[g - base].copy_((fc + nf).to(blk.expert_fc.dtype))
                        blk.expert_proj.data[g - base].copy_((pr + np_).to(blk.expert_proj.dtype))
                blk.router.data.zero_()
                stats["warm_started"] += 1
            elif strict:
                raise KeyError(f"{path}: no MLP or MoE tensors for layer {i}")
    return stats


def load_resume_state(ckpt_dir: str, optimizer=None) -> Optional[dict]:
    d = Path(ckpt_dir)
    st = None
    if (d / "trainer_state.json").exists():
        st = json.loads((d / "trainer_state.json").read_text())
    if optimizer is not None and (d / "optim_state.safetensors").exists():
        optimizer.load_state_dict(load_file(str(d / "optim_state.safetensors")))
    return st
