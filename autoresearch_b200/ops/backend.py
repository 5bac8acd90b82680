"""Ops backends: one interface, three implementations.

* ``oracle``   – the plain PyTorch fp32-math statement in ``ops.reference`` (CPU or GPU),
                 differentiated by autograd.  The numerical reference for everything else.
* ``baseline`` – library path on a GPU: bf16 ``torch.matmul`` (cuBLAS), library flash
                 attention / SDPA, torch elementwise ops.  This is the "cuBLAS + library
                 attention + NCCL" arm that the sm_100a kernels are measured against.
* ``sm100``    – the hand-written sm_100a kernels of ``autoresearch_b200.ops.sm100``.

The model (``models.gpt``) only talks to this interface, so swapping the implementation
never changes the training loop (the reference hard-wires its one implementation in
brain/src/forward.rs and brain/src/backward.rs).
"""
from __future__ import annotations


import torch
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from . import reference as R


class OracleBackend:
    name = "oracle"

    def __init__(self, eps: float = 1e-5, softcap: float = 15.0, ce_chunk: int = 4096):
        self.eps = eps
        self.softcap = softcap
        self.ce_chunk = ce_chunk

    def configure(self, cfg):
        self.eps, self.softcap, self.ce_chunk = cfg.eps, cfg.softcap, cfg.ce_chunk
        return self

    # -- elementwise / norms ------------------------------------------------
    def embedding(self, ids, w):
        return F.embedding(ids.long(), w)

    def rmsnorm(self, x):
        return R.rmsnorm(x, self.eps)

    def resid_scale_norm(self, x, x0, lam_r, lam_0, i):
        return R.resid_scale_norm(x, x0, lam_r[i], lam_0[i], self.eps)

    def add_norm(self, x, proj):
        return R.add_norm(x, proj, self.eps)

    def residual_add(self, x, y):
        return (x.float() + y.float()).to(x.dtype)

    def rope_qknorm(self, x, cos, sin):
        return R.rope_qknorm(x, cos, sin, self.eps)

    def ve_apply(self, v, ve, gate):
        return R.ve_apply(v, ve, gate)

    # -- contractions ---------------------------------------------------------
    def linear_col(self, x, w):
        return R.linear(x, w)

    def linear_row(self, x, w):
        return R.linear(x, w)

    def linear_col_relu_sq(self, x, w):
        return R.relu_sq(R.linear(x, w))

    def gate_linear(self, xn, w, ch):
        return R.linear(xn[:, :ch], w)

    def attention(self, q, k, v, window):
        return R.attention(q, k, v, window)

    # -- coarse blocks (a backend may fuse across these boundaries) ------------------
    def attention_block(self, xn, blk, ids_flat, B, T, cfg, cos, sin, window):
        """xn [N, D] -> attention output [N, H*hd] (before the output projection)."""
        hd = cfg.head_dim
        Dl = blk.wqkv.shape[0] // 3
        H = Dl // hd
        tp = getattr(self, "tp", None)
        if tp is not None and tp.size > 1:
            xn = tp.all_gather(xn)                    # token shards -> all tokens (local heads only)
        qkv = self.linear_col(xn, blk.wqkv)
        q, k, v = qkv[:, :Dl], qkv[:, Dl:2 * Dl], qkv[:, 2 * Dl:]
        v = v.reshape(B, T, H, hd)
        if blk.ve is not None:
            ve = self.embedding(ids_flat, blk.ve)
            gate = self.gate_linear(xn, blk.ve_gate, cfg.ve_gate_ch)
            v = self.ve_apply(v, ve.view(B, T, H, hd), gate.view(B, T, H))
        q = self.rope_qknorm(q.reshape(B, T, H, hd), cos, sin)
        k = self.rope_qknorm(k.reshape(B, T, H, hd), cos, sin)
        return self.attention(q, k, v, window).reshape(B * T, Dl)

    def proj_add_norm(self, a, w, x):
        y = self.linear_row(a, w)
        tp = getattr(self, "tp", None)
        if tp is not None and tp.size > 1:
            y = tp.reduce_scatter(y)                  # partial sums over heads -> this rank's tokens
        return self.add_norm(x, y)

    def mlp_add(self, xn, wfc, wdn, x):
        tp = getattr(self, "tp", None)
        if tp is not None and tp.size > 1:
            xn = tp.all_gather(xn)
        y = self.linear_row(self.linear_col_relu_sq(xn, wfc), wdn)
        if tp is not None and tp.size > 1:
            y = tp.reduce_scatter(y)
        return self.residual_add(x, y)

    def moe_mlp_add(self, xn, x, blk, moe):
        y, aux = self.moe_mlp(xn, blk.router, blk.expert_fc, blk.expert_proj, moe)
        return self.residual_add(x, y), aux

    def lm_head_ce(self, xf, w, targets, grad_scale):
        N = xf.shape[0]
        parts = []
        for a in range(0, N, self.ce_chunk):
            xs, ts = xf[a:a + self.ce_chunk], targets[a:a + self.ce_chunk]
            if xs.requires_grad or w.requires_grad:
                parts.append(checkpoint(self._ce_chunk, xs, w, ts, use_reentrant=False))
            else:
                parts.append(self._ce_chunk(xs, w, ts))
        per_tok = torch.cat(parts)
        return per_tok.sum() * grad_scale, per_tok.detach()

    def _ce_chunk(self, xs, w, ts):
        return R.softcap_ce(R.linear(xs, w), ts, self.softcap)

    def moe_mlp(self, xn, router, w_fc, w_proj, moe):
        return R.moe_mlp(xn, router, w_fc, w_proj, moe.top_k, moe.aux_coeff, moe.capacity_factor)


def _blocked_window_attention(q, k, v, window: int):
    """Exact sliding-window attention (key j visible to query i iff i-window <= j <= i)
    through SDPA on blocks of `window` queries that see their own and the previous block."""
    B, T, H, hd = q.shape
    W = window
    nb = T // W
    qb = q.view(B, nb, W, H, hd).permute(0, 1, 3, 2, 4)                     # B nb H W hd
    kb = k.view(B, nb, W, H, hd).permute(0, 1, 3, 2, 4)
    vb = v.view(B, nb, W, H, hd).permute(0, 1, 3, 2, 4)
    kprev = torch.cat([torch.zeros_like(kb[:, :1]), kb[:, :-1]], dim=1)
    vprev = torch.cat([torch.zeros_like(vb[:, :1]), vb[:, :-1]], dim=1)
    k2 = torch.cat([kprev, kb], dim=3)                                        # B nb H 2W hd
    v2 = torch.cat([vprev, vb], dim=3)
    qi = torch.arange(W, device=q.device).view(W, 1)
    kk = torch.arange(2 * W, device=q.device).view(1, 2 * W)
    band = (kk >= qi) & (kk <= qi + W)                                        # W x 2W
    mask = band.view(1, 1, 1, W, 2 * W).expand(1, nb, 1, W, 2 * W).clone()
    mask[:, 0, :, :, :W] = False
    o = F.scaled_dot_product_attention(qb, k2, v2, attn_mask=mask)
    return o.permute(0, 1, 3, 2, 4).reshape(B, T, H, hd)


class BaselineBackend(OracleBackend):
    """Library arm: cuBLAS matmuls, library attention, torch elementwise kernels."""

    name = "baseline"

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self._flash = None
        self.use_cudnn = True

    def _flash_fn(self):
        if self._flash is None:
            try:
                from flash_attn import flash_attn_func
                self._flash = flash_attn_func
            except Exception:
                self._flash = False
        return self._flash

    # elementwise ops stay in the activation dtype (library kernels, no fp32 copies kept for backward)
    def rmsnorm(self, x):
        return F.rms_norm(x, (x.shape[-1],), eps=self.eps)

    def resid_scale_norm(self, x, x0, lam_r, lam_0, i):
        xs = lam_r[i] * x + lam_0[i] * x0
        return xs, self.rmsnorm(xs)

    def add_norm(self, x, proj):
        xs = x + proj
        return xs, self.rmsnorm(xs)

    def residual_add(self, x, y):
        return x + y

    def linear_col_relu_sq(self, x, w):
        return F.relu(R.linear(x, w)).square()

    def rope_qknorm(self, x, cos, sin):
        B, T, H, hd = x.shape
        half = hd // 2
        lo, hi = x[..., :half], x[..., half:]
        c = cos[:T].to(x.dtype).view(1, T, 1, half)
        s = sin[:T].to(x.dtype).view(1, T, 1, half)
        return self.rmsnorm(torch.cat([lo * c + hi * s, hi * c - lo * s], dim=-1))

    def ve_apply(self, v, ve, gate):
        return v + (2.0 * torch.sigmoid(gate)).unsqueeze(-1).to(v.dtype) * ve

    # which library kernel served the full-causal and the sliding-window layers (reported by the benchmark)
    attention_used = {"causal": None, "window": None}

    def attention(self, q, k, v, window):
        """The best library attention on the image: full-causal layers go to cuDNN's fused attention through
        torch SDPA (a Blackwell-native kernel; measured on a B200 at B=2 H=8 T=32768: forward 2.9 ms = 1.5 PFLOP/s,
        against 10.9 ms for flash-attn 2 and 6.0 ms per batch element for flashinfer's fa2 backend); sliding-window
        layers go to flash-attn 2, the only library kernel here that takes a window (SDPA would need a dense mask)."""
        B, T, H, hd = q.shape
        if not q.is_cuda:
            return R.attention(q, k, v, window)
        half = q.dtype in (torch.bfloat16, torch.float16)
        if window >= T and half and self.use_cudnn:
            from torch.nn.attention import SDPBackend, sdpa_kernel
            try:
                with sdpa_kernel([SDPBackend.CUDNN_ATTENTION]):
                    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
                BaselineBackend.attention_used["causal"] = "cudnn-sdpa"
                return o.transpose(1, 2)
            except RuntimeError:
                self.use_cudnn = False            # not available for this shape / build: fall through
        fa = self._flash_fn()
        if fa and half:
            ws = (window, 0) if window < T else (-1, -1)
            BaselineBackend.attention_used["window" if window < T else "causal"] = "flash-attn-2"
            return fa(q, k, v, causal=True, window_size=ws)
        if window < T and T % window == 0:
            return _blocked_window_attention(q, k, v, window)
        if window < T:
            return R.attention(q, k, v, window)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2),
                                           v.transpose(1, 2), is_causal=True)
        return o.transpose(1, 2)


_BACKENDS = {}


def get_backend(name: str, cfg=None):
    """Return a configured backend.  ``auto`` picks ``sm100`` on a CUDA device whose
    compute capability is 10.x and ``oracle`` otherwise."""
    if name == "auto":
        name = "sm100" if (torch.cuda.is_available()
                           and torch.cuda.get_device_capability()[0] == 10) else "oracle"
    if name == "oracle":
        be = OracleBackend()
    elif name == "baseline":
        be = BaselineBackend()
    elif name == "sm100":
        from .sm100 import Sm100Backend
        be = Sm100Backend()
    else:
        raise KeyError(f"unknown ops backend {name!r}")
    if cfg is not None:
        be.configure(cfg)
    return be
