"""Plain PyTorch statement of every op of the model and the optimizer.

These functions are the numerical oracle (fp32 math on any device, differentiable
through autograd) against which the CUDA kernels are tested, and the implementation
used for the CPU path.  The math follows the reference engine's forward pass
(brain/src/forward.rs:174-273,359-739) and the kernels it launches
(brain/kernels/*.cu); the readable Python statement of the shared math is
original/train.py:42-290.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, eps: float) -> torch.Tensor:
    """Parameter-free RMSNorm over the last dim (brain/kernels/rms_norm.cu:20-47)."""
    xf = x.float()
    r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * r).to(x.dtype)


def resid_scale_norm(x, x0, lam_r, lam_0, eps):
    """x' = lam_r*x + lam_0*x0 ; xn = rmsnorm(x')
    (brain/kernels/fused_norm_residual.cu:200-253).  Returns (x', xn)."""
    xs = (lam_r.float() * x.float() + lam_0.float() * x0.float()).to(x.dtype)
    return xs, rmsnorm(xs, eps)


def add_norm(x, proj, eps):
    """x' = x + proj ; xn = rmsnorm(x') (brain/kernels/fused_norm_residual.cu:22-64)."""
    xs = (x.float() + proj.float()).to(x.dtype)
    return xs, rmsnorm(xs, eps)


def rope_tables(seq_len: int, head_dim: int, base: float, device=None, dtype=torch.float32):
    """cos/sin tables [T, head_dim/2]; theta_i = base^(-2i/hd), computed in fp64
    (brain/src/train.rs:2402-2422)."""
    half = head_dim // 2
    i = torch.arange(half, dtype=torch.float64)
    inv = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / head_dim)
    t = torch.arange(seq_len, dtype=torch.float64)
    ang = torch.outer(t, inv)
    return ang.cos().to(dtype).to(device), ang.sin().to(dtype).to(device)


def rope_qknorm(x, cos, sin, eps):
    """Rotate-half RoPE followed by per-head RMSNorm
    (brain/kernels/fused_norm_residual.cu:130-193).  x: [B, T, H, hd]."""
    B, T, H, hd = x.shape
    half = hd // 2
    xf = x.float()
    lo, hi = xf[..., :half], xf[..., half:]
    c = cos[:T].float().view(1, T, 1, half)
    s = sin[:T].float().view(1, T, 1, half)
    r = torch.cat([lo * c + hi * s, -lo * s + hi * c], dim=-1)
    r = r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + eps)
    return r.to(x.dtype)


def window_mask(T: int, window: int, device=None) -> torch.Tensor:
    """True where key j is visible to query i: i - window <= j <= i
    (brain/src/forward.rs:1134-1138, brain/tools/diagnostic.py:99-113)."""
    i = torch.arange(T, device=device).view(T, 1)
    j = torch.arange(T, device=device).view(1, T)
    return (j <= i) & (j >= i - window)


def attention(q, k, v, window: int):
    """Causal (optionally sliding-window) softmax attention, scale 1/sqrt(hd).
    q, k, v: [B, T, H, hd] -> [B, T, H, hd]."""
    B, T, H, hd = q.shape
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    s = torch.matmul(qf, kf.transpose(-1, -2)) / math.sqrt(hd)
    m = window_mask(T, window, q.device)
    s = s.masked_fill(~m, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vf).transpose(1, 2)
    return o.to(q.dtype).contiguous()


def ve_apply(v, ve, gate_logits):
    """v += 2*sigmoid(gate)[..., h, None] * ve[..., h, :]
    (brain/kernels/ve_apply.cu:10-43).  v, ve: [B,T,H,hd]; gate_logits: [B,T,H]."""
    g = 2.0 * torch.sigmoid(gate_logits.float())
    return (v.float() + g.unsqueeze(-1) * ve.float()).to(v.dtype)


def relu_sq(x):
    r = torch.relu(x.float())
    return (r * r).to(x.dtype)


def linear(x, w):
    """y = x @ w^T with fp32 accumulation."""
    if x.dtype == torch.float32:
        return x @ w.t()
    return (x @ w.t())


def softcap_ce(logits, targets, softcap: float):
    """Per-token loss of soft-capped logits: s = cap*tanh(x/cap); loss = lse(s) - s[tgt]
    (brain/kernels/cross_entropy.cu:60-99)."""
    s = softcap * torch.tanh(logits.float() / softcap)
    lse = torch.logsumexp(s, dim=-1)
    return lse - s.gather(-1, targets.view(-1, 1).long()).squeeze(-1)


def lm_head_ce(xf, w, targets, softcap: float, chunk: int):
    """Chunked LM head + soft-capped cross entropy; returns per-token losses [N] fp32
    (brain/src/forward.rs:231-272)."""
    N = xf.shape[0]
    outs = []
    for a in range(0, N, chunk):
        logits = linear(xf[a:a + chunk], w)
        outs.append(softcap_ce(logits, targets[a:a + chunk], softcap))
    return torch.cat(outs)


# --------------------------------------------------------------------------------------
# MoE (intended math of brain/kernels/moe_dispatch.cu:39-139, moe_aux_loss.cu:25-73)
# --------------------------------------------------------------------------------------

def moe_route(router_logits, top_k: int):
    """softmax over experts (fp32), top-k (ties -> lower index), gates renormalised over
    the selected experts.  Returns probs [N,E] fp32, idx [N,K] int64, gates [N,K] fp32."""
    probs = torch.softmax(router_logits.float(), dim=-1)
    # torch.topk breaks ties by lower index for sorted=True on CPU and CUDA alike when the
    # values are distinct; for exact ties use a stable sort.
    order = torch.sort(probs, dim=-1, descending=True, stable=True).indices
    idx = order[:, :top_k]
    g = probs.gather(-1, idx)
    gates = g / g.sum(-1, keepdim=True)
    return probs, idx, gates


def moe_aux_loss(probs, idx, n_experts: int, coeff: float):
    """L = coeff * E * sum_e f_e * P_e with f_e = count_e/(N*K) (no gradient) and
    P_e = mean_t probs[t, e] (brain/kernels/moe_aux_loss.cu:25-73)."""
    N, K = idx.shape
    counts = torch.bincount(idx.reshape(-1), minlength=n_experts).float()
    f = (counts / float(N * K)).detach()
    P = probs.mean(0)
    return coeff * n_experts * (f * P).sum()


def moe_capacity(n_tokens: int, n_experts: int, top_k: int, capacity_factor: float) -> int:
    """Rows per expert buffer: ceil(cf * N * K / E) rounded up to a multiple of 8 (16-byte rows
    for the tensor-core path); cf <= 0 means unlimited."""
    if capacity_factor <= 0:
        return n_tokens * top_k
    return (int(math.ceil(capacity_factor * n_tokens * top_k / n_experts)) + 7) // 8 * 8


def moe_keep_mask(idx, n_experts: int, capacity: int):
    """Token-order capacity rule: slot (t, k) is kept iff fewer than `capacity` earlier
    slots (in (t, k) lexicographic order) chose the same expert."""
    N, K = idx.shape
    flat = idx.reshape(-1)
    onehot = F.one_hot(flat, n_experts)
    pos = (onehot.cumsum(0) - 1).gather(1, flat.view(-1, 1)).squeeze(1)
    return (pos < capacity).view(N, K)


def moe_mlp(xn, router_w, w_fc, w_proj, top_k: int, aux_coeff: float,
            capacity_factor: float = 0.0):
    """Dense-equivalent MoE block.  xn [N,D]; router_w [E,D]; w_fc [E,M,D]; w_proj [E,D,M].
    Returns (y [N,D], aux_loss scalar)."""
    N, D = xn.shape
    E = router_w.shape[0]
    logits = linear(xn, router_w)
    probs, idx, gates = moe_route(logits, top_k)
    aux = moe_aux_loss(probs, idx, E, aux_coeff)
    cap = moe_capacity(N, E, top_k, capacity_factor)
    keep = moe_keep_mask(idx, E, cap)
    y = torch.zeros(N, D, dtype=torch.float32, device=xn.device)
    for e in range(E):
        sel = (idx == e) & keep
        tok, kk = sel.nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = relu_sq(linear(xn[tok], w_fc[e]))
        o = linear(h, w_proj[e]).float()
        y.index_add_(0, tok, o * gates[tok, kk].unsqueeze(-1))
    return y.to(xn.dtype), aux
