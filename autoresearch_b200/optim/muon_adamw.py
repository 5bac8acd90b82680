"""Muon (Nesterov momentum -> Frobenius normalise -> 5 "Polar Express" Newton-Schulz
iterations -> NorMuon variance normalisation -> cautious weight decay on fp32 masters) for
matrix parameters, AdamW for embeddings, the LM head, value embeddings, routers and the two
per-layer scalar vectors.

Rules and constants: brain/src/optim.rs:13-43,139-182,198-220,757-954 and
brain/kernels/muon.cu, brain/kernels/adamw.cu; readable statement of the same math:
original/train.py:296-352.

The optimizer works on the owner's groups of a ``ParamLayout``: with data parallelism each
rank updates only the whole matrices it owns (their summed gradients arrive through the
reduce-scatter) and the updated bf16 shards are all-gathered afterwards.  Every state
tensor is fp32 (the reference keeps the Adam moments of wte / value embeddings in bf16,
brain/src/optim.rs:253-264; fp32 is a strict refinement).
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from ..config import ScheduleConfig
from ..parallel.layout import ParamLayout
from . import schedule as S

POLAR_EXPRESS = (
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
)


# ----------------------------------------------------------------------------------------
# functional reference (batched over the leading dim)
# ----------------------------------------------------------------------------------------

def muon_nesterov(buf: torch.Tensor, g: torch.Tensor, mu: float, work_dtype) -> torch.Tensor:
    """buf = mu*buf + (1-mu)*g ; u = (1-mu)*g + mu*buf  (brain/kernels/muon.cu:63-83)."""
    buf.mul_(mu).add_(g, alpha=1.0 - mu)
    return (g * (1.0 - mu) + buf * mu).to(work_dtype)


def frob_normalise(u: torch.Tensor) -> torch.Tensor:
    """x = u / (||u||_F * 1.02 + 1e-6) per matrix (brain/kernels/muon.cu:132-177)."""
    n = u.float().pow(2).sum(dim=(-2, -1), keepdim=True).sqrt()
    return (u.float() / (n * 1.02 + 1e-6)).to(u.dtype)


def newton_schulz(x: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """A = X^T X (tall) or X X^T; C = a I + b A + c A^2; X = X C or C X.  Every
    intermediate is stored in x.dtype, products accumulate in fp32
    (brain/src/optim.rs:872-931)."""
    m, n = x.shape[-2:]
    tall = m > n
    d = n if tall else m
    eye = torch.eye(d, device=x.device, dtype=torch.float32)
    for a, b, c in POLAR_EXPRESS[:steps]:
        A = (x.mT @ x) if tall else (x @ x.mT)
        A2 = A @ A
        C = (a * eye + b * A.float() + c * A2.float()).to(x.dtype)
        x = (x @ C) if tall else (C @ x)
    return x


def normuon(x: torch.Tensor, second: torch.Tensor, beta2: float) -> torch.Tensor:
    """NorMuon (brain/kernels/muon.cu:244-356): per-row (m >= n) or per-column mean of
    squares, EMA, rescale keeping the total norm.  `second` is [G, m, 1] or [G, 1, n]."""
    m, n = x.shape[-2:]
    red = -1 if m >= n else -2
    red_size = x.shape[red]
    xf = x.float()
    v = xf.pow(2).mean(dim=red, keepdim=True)
    vn = (v.sum(dim=(-2, -1), keepdim=True) * red_size).sqrt()
    second.mul_(beta2).add_(v, alpha=1.0 - beta2)
    ss = second.clamp_min(1e-10).rsqrt()
    vn_new = ((v * red_size) * ss.pow(2)).sum(dim=(-2, -1), keepdim=True).sqrt()
    return xf * (ss * (vn / vn_new.clamp_min(1e-10)))


def cautious_update(master: torch.Tensor, g: torch.Tensor, lr: float, wd: float) -> None:
    """mask = (g*p >= 0); p -= lr*g + lr*wd*p*mask (brain/kernels/muon.cu:89-112)."""
    mask = (g * master) >= 0
    master.sub_(lr * g + (lr * wd) * master * mask)


def adamw_update(p, g, m, v, step: int, lr: float, b1: float, b2: float, eps: float,
                 wd: float) -> None:
    """p -= lr*wd*p; m,v EMA; p -= lr*(m/bc1)/(sqrt(v/bc2)+eps)
    (brain/kernels/adamw.cu:9-45)."""
    p.mul_(1.0 - lr * wd)
    m.mul_(b1).add_(g, alpha=1.0 - b1)
    v.mul_(b2).addcmul_(g, g, value=1.0 - b2)
    bc1 = 1.0 - b1 ** step
    bc2 = 1.0 - b2 ** step
    denom = (v / bc2).sqrt_().add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)


# ----------------------------------------------------------------------------------------

class MuonAdamW:
    def __init__(self, layout: ParamLayout, cfg: ScheduleConfig, d_model: int,
                 kernels=None):
        """kernels: optional object with fused CUDA implementations (same method names as
        the functional reference above); None = plain PyTorch."""
        self.layout = layout
        self.cfg = cfg
        self.d_model = d_model
        self.k = kernels
        self.state: Dict[int, Dict[str, torch.Tensor]] = {}
        self.work_dtype = (torch.bfloat16 if layout.param_dtype == torch.bfloat16
                           else torch.float32)
        dev = layout.device
        for gi, g in enumerate(layout.groups):
            if g.owner != layout.rank:
                continue
            pv = layout.group_view(layout.flat_param, g)
            st = {"master": pv.detach().float().clone()}
            if g.kind == "muon":
                m, n = g.shape
                st["momentum"] = torch.zeros_like(st["master"])
                sshape = (g.count, m, 1) if m >= n else (g.count, 1, n)
                st["second"] = torch.zeros(sshape, dtype=torch.float32, device=dev)
            else:
                st["m"] = torch.zeros_like(st["master"])
                st["v"] = torch.zeros_like(st["master"])
            self.state[gi] = st

    # ------------------------------------------------------------------
    def _adam_hparams(self, kind: str, lr_mult: float):
        c = self.cfg
        ds = S.dmodel_lr_scale(self.d_model)
        b1, b2 = c.adam_beta1, c.adam_beta2
        if kind == "adamw_emb":
            return c.embedding_lr * ds * lr_mult, c.wd_wte, b1, b2
        if kind == "adamw_head":
            return c.unembedding_lr * ds * lr_mult, c.wd_lm_head, b1, b2
        if kind == "adamw_ve":
            return c.embedding_lr * ds * lr_mult, c.wd_ve, b1, b2
        if kind == "adamw_router":
            return c.unembedding_lr * ds * lr_mult, c.wd_router, b1, b2
        if kind == "adamw_lr":
            return c.scalar_lr * 0.01 * lr_mult, 0.0, b1, b2
        if kind == "adamw_l0":
            return c.scalar_lr * lr_mult, 0.0, 0.96, b2
        raise KeyError(kind)

    @torch.no_grad()
    def step(self, step: int, progress: float, warmup_mult: float = 1.0, grad_source=None, bucket=None) -> None:
        """`step` is 1-indexed.  Expects the summed gradient of every owned group in
        ``layout.flat_grad``; writes the updated parameters into ``layout.flat_param``.
        ``grad_source(group)`` may return another gradient object for a group (the fused
        data-parallel path hands out descriptors of the un-reduced peer buckets).
        ``bucket``: update only the groups of that gradient bucket (the overlapped exchange calls this once per
        bucket, in the order in which the backward pass finishes them)."""
        c = self.cfg
        lr_mult = S.lr_multiplier(progress, c) * warmup_mult
        mu = S.muon_momentum(step, c)
        wd = S.muon_weight_decay(progress, c)
        lay = self.layout
        for gi, st in self.state.items():
            g = lay.groups[gi]
            if bucket is not None and g.bucket != bucket:
                continue
            grad = grad_source(g) if grad_source is not None else None
            if grad is None:
                grad = lay.group_view(lay.flat_grad, g)
            pv = lay.group_view(lay.flat_param, g)
            if g.kind == "muon":
                m, n = getattr(g.atoms[0].param, "muon_full_shape", g.shape)
                lr = c.peak_lr * lr_mult * math.sqrt(max(1.0, m / n))
                self._muon_group(st, grad, pv, mu, lr, wd)
            else:
                lr, awd, b1, b2 = self._adam_hparams(g.kind, lr_mult)
                self._adam_group(st, grad, pv, step, lr, b1, b2, c.adam_eps, awd)

    def _muon_group(self, st, grad, pv, mu, lr, wd):
        if self.k is not None and grad.is_cuda:
            return self.k.muon_group(st, grad, pv, mu, lr, wd, self.cfg.muon_beta2,
                                     self.cfg.ns_steps)
        u = muon_nesterov(st["momentum"], grad.float(), mu, self.work_dtype)
        x = frob_normalise(u)
        x = newton_schulz(x, self.cfg.ns_steps)
        gfin = normuon(x, st["second"], self.cfg.muon_beta2)
        cautious_update(st["master"], gfin, lr, wd)
        pv.copy_(st["master"])

    def _adam_group(self, st, grad, pv, step, lr, b1, b2, eps, wd):
        if self.k is not None and grad.is_cuda:
            return self.k.adamw_group(st, grad, pv, step, lr, b1, b2, eps, wd)
        adamw_update(st["master"], grad.float(), st["m"], st["v"], step, lr, b1, b2, eps, wd)
        pv.copy_(st["master"])

    # ------------------------------------------------------------------
    def state_dict(self) -> Dict[str, torch.Tensor]:
        """World-size independent: one entry per unit name and state kind."""
        out: Dict[str, torch.Tensor] = {}
        lay = self.layout
        for gi, st in self.state.items():
            g = lay.groups[gi]
            names = [u.name for a in g.atoms for u in a.units]
            for key, t in st.items():
                for i, nm in enumerate(names):
                    out[f"{nm}::{key}"] = t[i].detach().cpu().clone()
        return out

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        lay = self.layout
        for gi, st in self.state.items():
            g = lay.groups[gi]
            names = [u.name for a in g.atoms for u in a.units]
            for key, t in st.items():
                for i, nm in enumerate(names):
                    k = f"{nm}::{key}"
                    if k in sd:
                        t[i].copy_(sd[k].to(t.device))
