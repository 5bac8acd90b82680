"""sm_100a backend: autograd Functions over the hand-written kernels.

Granularity follows what fuses well on a B200 rather than the reference's op list
(brain/src/forward.rs:359-739, brain/src/backward.rs:203-877):

* ``AttnPreFn``   – QKV GEMM (packed [3D, D] weight) + in-place RoPE / QK-norm / value
                    embedding on the packed output; backward runs the norm/RoPE backward in
                    place on the packed gradient, one K=3D dX GEMM and one dW GEMM (no
                    pack / split copies, no recomputed q/k GEMMs).
* ``AttentionFn`` – flash attention reading q, k, v as column blocks of the packed buffer.
* ``LinearAddFn`` – O-proj / FC2 GEMM with the residual add in the epilogue.
* ``MLPFn``       – FC1 GEMM with ReLU^2 epilogue (only relu(h)^2 is kept: the backward
                    recovers 2*relu(h) as 2*sqrt of it inside the dX GEMM epilogue).
* ``LMHeadCEFn``  – chunked LM head + soft-capped CE; logits are turned into their
                    gradient in place during the forward so nothing is recomputed.
* weight gradients accumulate in fp32 (``param.main_grad``) inside the dW GEMM epilogue.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import kernels as K
from .backend import OracleBackend


def _main_grad(p: torch.Tensor) -> Optional[torch.Tensor]:
    return getattr(p, "main_grad", None)


def _acc_weight_grad(w, dy, x):
    """main_grad(w) += dy^T @ x.  Returns None when accumulated in place, else the grad."""
    mg = _main_grad(w)
    if mg is not None:
        K.gemm(dy, x, trans_a=True, trans_b=False, out=mg, epi=K.EPI_ATOMIC_F32)
        return None
    tmp = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
    K.gemm(dy, x, trans_a=True, trans_b=False, out=tmp, epi=K.EPI_ATOMIC_F32)
    return tmp.to(w.dtype)


class LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return K.gemm(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = K.gemm(dy, w, trans_b=False) if ctx.needs_input_grad[0] else None
        dw = _acc_weight_grad(w, dy, x)
        return dx, dw


class LinearAddFn(torch.autograd.Function):
    """out = resid + a @ w^T (residual add in the GEMM epilogue)."""

    @staticmethod
    def forward(ctx, a, w, resid):
        ctx.save_for_backward(a, w)
        return K.gemm(a, w, epi=K.EPI_ADD_AUX, aux=resid)

    @staticmethod
    def backward(ctx, g):
        a, w = ctx.saved_tensors
        g = g.contiguous()
        da = K.gemm(g, w, trans_b=False)
        dw = _acc_weight_grad(w, g, a)
        return da, dw, g


class MLPFn(torch.autograd.Function):
    """out = resid + relu(xn @ wfc^T)^2 @ wdn^T."""

    @staticmethod
    def forward(ctx, xn, wfc, wdn, resid):
        act = K.gemm(xn, wfc, epi=K.EPI_RELU2)
        out = K.gemm(act, wdn, epi=K.EPI_ADD_AUX, aux=resid)
        ctx.save_for_backward(xn, wfc, wdn, act)
        return out

    @staticmethod
    def backward(ctx, g):
        xn, wfc, wdn, act = ctx.saved_tensors
        g = g.contiguous()
        dh = K.gemm(g, wdn, trans_b=False, epi=K.EPI_RELU2_BWD, aux=act)
        dwdn = _acc_weight_grad(wdn, g, act)
        dwfc = _acc_weight_grad(wfc, dh, xn)
        dxn = K.gemm(dh, wfc, trans_b=False)
        return dxn, dwfc, dwdn, g


class TPRowLinearFn(torch.autograd.Function):
    """Row-parallel linear with sequence-sharded output: y_shard = reduce-scatter(a @ w^T), the transfer
    riding on the GEMM epilogue (FusedTPContext.gemm_rs).  Backward: all-gather(g) -> GEMM."""

    @staticmethod
    def forward(ctx, a, w, tp):
        ctx.tp = tp
        ctx.save_for_backward(a, w)
        return tp.gemm_rs(a, w)

    @staticmethod
    def backward(ctx, g):
        a, w = ctx.saved_tensors
        da, g_full = ctx.tp.ag_gemm(g.contiguous(), w, trans_b=False)
        dw = _acc_weight_grad(w, g_full, a)
        return da, dw, None


class TPMLPFn(torch.autograd.Function):
    """Tensor-parallel MLP on a sequence shard: out = resid + RS(relu(AG(xn) @ wfc^T)^2 @ wdn^T)."""

    @staticmethod
    def forward(ctx, xn, wfc, wdn, resid, tp):
        ctx.tp = tp
        act, xn_full = tp.ag_gemm(xn, wfc, epi=K.EPI_RELU2)
        y = tp.gemm_rs(act, wdn)
        ctx.save_for_backward(xn_full, wfc, wdn, act)
        return K.residual_add(resid, y)

    @staticmethod
    def backward(ctx, g):
        xn_full, wfc, wdn, act = ctx.saved_tensors
        tp = ctx.tp
        g = g.contiguous()
        dh, g_full = tp.ag_gemm(g, wdn, trans_b=False, epi=K.EPI_RELU2_BWD, aux=act)
        dwdn = _acc_weight_grad(wdn, g_full, act)
        dwfc = _acc_weight_grad(wfc, dh, xn_full)
        dxn = tp.gemm_rs(dh, wfc, trans_b=False)
        return dxn, dwfc, dwdn, g, None


class RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps):
        ctx.save_for_backward(x)
        ctx.eps = eps
        return K.rmsnorm_fwd(x, eps)

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        return K.rmsnorm_bwd(x, g.contiguous(), ctx.eps), None


class LinearAddNormFn(torch.autograd.Function):
    """xs = resid + a @ w^T (add in the GEMM epilogue); xn = rmsnorm(xs).  The backward fuses
    the sum of the two incoming gradients into the norm backward."""

    @staticmethod
    def forward(ctx, a, w, resid, eps):
        xs = K.gemm(a, w, epi=K.EPI_ADD_AUX, aux=resid)
        xn = K.rmsnorm_fwd(xs, eps)
        ctx.save_for_backward(a, w, xs)
        ctx.eps = eps
        return xs, xn

    @staticmethod
    def backward(ctx, g_xs, g_xn):
        a, w, xs = ctx.saved_tensors
        if g_xn is None:
            g = g_xs.contiguous()
        else:
            add = g_xs.contiguous() if g_xs is not None else None
            g = K.rmsnorm_bwd(xs, g_xn.contiguous(), ctx.eps, add_to=add)
        da = K.gemm(g, w, trans_b=False)
        dw = _acc_weight_grad(w, g, a)
        return da, dw, g, None


class AddNormFn(torch.autograd.Function):
    """xs = x + y ; xn = rmsnorm(xs); backward d = g_xs + rmsnorm_bwd(xs, g_xn) for both inputs."""

    @staticmethod
    def forward(ctx, x, y, eps):
        xs, xn = K.add_norm_fwd(x.contiguous(), y.contiguous(), eps)
        ctx.save_for_backward(xs)
        ctx.eps = eps
        return xs, xn

    @staticmethod
    def backward(ctx, g_xs, g_xn):
        (xs,) = ctx.saved_tensors
        if g_xn is None:
            g = g_xs
        else:
            g = K.rmsnorm_bwd(xs, g_xn.contiguous(), ctx.eps, add_to=g_xs.contiguous() if g_xs is not None else None)
        return g, g, None


class ResidualAddFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        return K.residual_add(a.contiguous(), b.contiguous())

    @staticmethod
    def backward(ctx, g):
        return g, g


class LinearRelu2Fn(torch.autograd.Function):
    """act = relu(x @ w^T)^2 with the activation in the GEMM epilogue; backward from act alone."""

    @staticmethod
    def forward(ctx, x, w):
        act = K.gemm(x, w, epi=K.EPI_RELU2)
        ctx.save_for_backward(x, w, act)
        return act

    @staticmethod
    def backward(ctx, g_act):
        x, w, act = ctx.saved_tensors
        # d_h = g_act * 2*sqrt(act): fold into an elementwise pass, then the two GEMMs
        dh = (g_act.float() * 2.0 * act.float().sqrt()).to(torch.bfloat16)
        dx = K.gemm(dh, w, trans_b=False)
        dw = _acc_weight_grad(w, dh, x)
        return dx, dw


class _X0GradChain:
    """The x0 gradient of one forward pass: every layer of a stage adds its share to one buffer inside its
    backward kernel, and only the stage's first layer (the last to run backward) hands the sum to autograd."""
    __slots__ = ("buf",)

    def __init__(self):
        self.buf = None


class ResidScaleNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, x0, lam_r, lam_0, idx, eps, chain=None):
        ctx.save_for_backward(x, x0, lam_r, lam_0)
        ctx.idx, ctx.eps, ctx.chain = idx, eps, chain
        xs, xn = K.resid_scale_norm_fwd(x, x0, lam_r, lam_0, idx, eps)
        return xs, xn

    @staticmethod
    def backward(ctx, g_xs, g_xn):
        x, x0, lam_r, lam_0 = ctx.saved_tensors
        if g_xs is None:
            g_xs = torch.zeros_like(x)
        if g_xn is None:
            g_xn = torch.zeros_like(x)
        mr, m0 = _main_grad(lam_r), _main_grad(lam_0)
        dr = mr if mr is not None else torch.zeros(lam_r.shape, dtype=torch.float32, device=x.device)
        d0 = m0 if m0 is not None else torch.zeros(lam_0.shape, dtype=torch.float32, device=x.device)
        chain = ctx.chain
        dx, dx0 = K.resid_scale_norm_bwd(x, x0, lam_r, lam_0, ctx.idx, g_xs.contiguous(), g_xn.contiguous(),
                                         dr, d0, ctx.eps, dx0_acc=chain.buf if chain is not None else None)
        if chain is not None:
            chain.buf = dx0
            if ctx.idx != 0:
                dx0 = None          # still being summed; layer 0 of the stage returns it
            else:
                chain.buf = None
        return (dx, dx0, None if mr is not None else dr.to(lam_r.dtype),
                None if m0 is not None else d0.to(lam_0.dtype), None, None, None)


class EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, w):
        ctx.save_for_backward(ids, w)
        return K.embedding_fwd(ids, w)

    @staticmethod
    def backward(ctx, g):
        ids, w = ctx.saved_tensors
        mg = _main_grad(w)
        if mg is not None:
            K.embedding_bwd(ids, g.contiguous(), mg)
            return None, None
        tmp = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        K.embedding_bwd(ids, g.contiguous(), tmp)
        return None, tmp.to(w.dtype)


class AttnPreFn(torch.autograd.Function):
    """packed qkv = post(xn @ wqkv^T): RoPE + QK-norm on q, k; value embedding on v."""

    @staticmethod
    def forward(ctx, xn, wqkv, ids, ve_w, gate_w, cos, sin, T, H, gate_ch, eps, tp=None):
        # tp (a FusedTPContext): xn is this rank's sequence shard; the gather is overlapped with the GEMM
        ctx.tp = tp
        if tp is None and K.qkv_post_fusable(xn.shape[0], wqkv.shape[0]):
            # RoPE, QK-norm and the value embedding run in the epilogue of the projection: qkv is written once
            N, D = xn.shape
            rstd = torch.empty(N, 2 * H, dtype=torch.float32, device=xn.device)
            gate = torch.empty(N, H, dtype=torch.float32, device=xn.device) if ve_w is not None else None
            qkv = K.gemm(xn, wqkv, epi=K.EPI_QKV_POST,
                         post=dict(cos=cos, sin=sin, rstd=rstd, T=T, H=H, xn=xn, ids=ids, ve_w=ve_w, gate_w=gate_w, gate=gate,
                                   gate_ch=gate_ch, eps=eps))
            ctx.save_for_backward(xn, wqkv, ids, ve_w, gate_w, cos, sin, qkv, rstd, gate)
            ctx.dims = (T, H, gate_ch)
            return qkv
        if tp is not None:
            qkv, xn = tp.ag_gemm(xn, wqkv)
        else:
            qkv = K.gemm(xn, wqkv)
        N, D = xn.shape
        rstd = torch.empty(N, 2 * H, dtype=torch.float32, device=xn.device)
        gate = torch.empty(N, H, dtype=torch.float32, device=xn.device) if ve_w is not None else None
        rc = K.lib().arb_qkv_post_fwd(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), rstd.data_ptr(),
                                      xn.data_ptr(), ids.data_ptr(),
                                      ve_w.data_ptr() if ve_w is not None else 0,
                                      gate_w.data_ptr() if ve_w is not None else 0,
                                      gate.data_ptr() if ve_w is not None else 0,
                                      N, T, H, D, gate_ch, eps, K._stream())
        K._check(rc, "qkv_post_fwd")
        ctx.save_for_backward(xn, wqkv, ids, ve_w, gate_w, cos, sin, qkv, rstd, gate)
        ctx.dims = (T, H, gate_ch)
        ctx.mark_non_differentiable(rstd)
        return qkv

    @staticmethod
    def backward(ctx, d_qkv):
        xn, wqkv, ids, ve_w, gate_w, cos, sin, qkv, rstd, gate = ctx.saved_tensors
        T, H, gate_ch = ctx.dims
        N, D = xn.shape
        d_qkv = d_qkv.contiguous()
        has_ve = ve_w is not None
        d_ve = d_xn_gate = dgl = None
        dgw = None
        if has_ve:
            d_ve = torch.empty(N, H * 128, dtype=torch.bfloat16, device=xn.device)
            d_xn_gate = torch.empty(N, gate_ch, dtype=torch.bfloat16, device=xn.device)
            dgl = torch.empty(N, H, dtype=torch.float32, device=xn.device)
            mg = _main_grad(gate_w)
            dgw = mg if mg is not None else torch.zeros(gate_w.shape, dtype=torch.float32, device=xn.device)
        rc = K.lib().arb_qkv_post_bwd(d_qkv.data_ptr(), qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), rstd.data_ptr(),
                                      xn.data_ptr(), ids.data_ptr(),
                                      ve_w.data_ptr() if has_ve else 0, gate_w.data_ptr() if has_ve else 0,
                                      gate.data_ptr() if has_ve else 0, d_ve.data_ptr() if has_ve else 0,
                                      dgw.data_ptr() if has_ve else 0, d_xn_gate.data_ptr() if has_ve else 0,
                                      dgl.data_ptr() if has_ve else 0, N, T, H, D, gate_ch, K._stream())
        K._check(rc, "qkv_post_bwd")
        dw = _acc_weight_grad(wqkv, d_qkv, xn)
        tp = ctx.tp
        if tp is not None:
            dxn = tp.gemm_rs(d_qkv, wqkv, trans_b=False)
            if has_ve:   # the gate's contribution to d(xn) is a partial sum over the head shards as well
                d_xn_gate = tp.reduce_scatter_rows(d_xn_gate)
        else:
            dxn = K.gemm(d_qkv, wqkv, trans_b=False)
        g_ve = g_gate = None
        if has_ve:
            K.add_cols_(dxn, d_xn_gate)
            mgv = _main_grad(ve_w)
            if mgv is not None:
                K.embedding_bwd(ids, d_ve, mgv)
            else:
                tmp = torch.zeros(ve_w.shape, dtype=torch.float32, device=xn.device)
                K.embedding_bwd(ids, d_ve, tmp)
                g_ve = tmp.to(ve_w.dtype)
            if _main_grad(gate_w) is None:
                g_gate = dgw.to(gate_w.dtype)
        return dxn, dw, None, g_ve, g_gate, None, None, None, None, None, None, None


class AttentionFn(torch.autograd.Function):
    """Flash attention over the packed qkv buffer [N, 3*H*128] -> [N, H*128]."""

    @staticmethod
    def forward(ctx, qkv, B, T, H, window):
        N = B * T
        Dl = H * 128
        out = torch.empty(N, Dl, dtype=torch.bfloat16, device=qkv.device)
        lse = torch.empty(B, H, T, dtype=torch.float32, device=qkv.device)
        ld = qkv.stride(0)
        base = qkv.data_ptr()
        scale = 1.0 / math.sqrt(128.0)
        rc = K.lib().arb_attn_fwd(base, base + 2 * Dl, base + 4 * Dl, out.data_ptr(), lse.data_ptr(), B, T, H,
                                  ld, ld, ld, Dl, window, scale, K.err_flag(qkv.device).data_ptr(), K._stream())
        K._check(rc, "attn_fwd")
        ctx.save_for_backward(qkv, out, lse)
        ctx.dims = (B, T, H, window)
        return out

    @staticmethod
    def backward(ctx, d_out):
        qkv, out, lse = ctx.saved_tensors
        B, T, H, window = ctx.dims
        N, Dl = B * T, H * 128
        d_out = d_out.contiguous()
        d_qkv = torch.empty_like(qkv)
        delta = torch.empty(B, H, T, dtype=torch.float32, device=qkv.device)
        ld = qkv.stride(0)
        b, db = qkv.data_ptr(), d_qkv.data_ptr()
        rc = K.lib().arb_attn_bwd(b, b + 2 * Dl, b + 4 * Dl, out.data_ptr(), d_out.data_ptr(), lse.data_ptr(),
                                  db, db + 2 * Dl, db + 4 * Dl, delta.data_ptr(), 0, B, T, H,
                                  ld, ld, ld, Dl, Dl, ld, ld, ld, window, 1.0 / math.sqrt(128.0),
                                  K.err_flag(qkv.device).data_ptr(), K._stream())
        K._check(rc, "attn_bwd")
        return d_qkv, None, None, None, None


class LibraryAttentionFn(torch.autograd.Function):
    """Library attention on the packed buffer (a comparison arm: everything else stays on this package's kernels):
    cuDNN's fused attention through torch SDPA for full-causal layers, flash-attn 2 for sliding windows."""

    @staticmethod
    def forward(ctx, qkv, B, T, H, window):
        Dl = H * 128
        with torch.enable_grad():
            src = qkv.detach().requires_grad_(True)
            q = src[:, :Dl].view(B, T, H, 128)
            k = src[:, Dl:2 * Dl].view(B, T, H, 128)
            v = src[:, 2 * Dl:].view(B, T, H, 128)
            o = None
            if window >= T:
                from torch.nn.attention import SDPBackend, sdpa_kernel
                try:
                    with sdpa_kernel([SDPBackend.CUDNN_ATTENTION]):
                        o = torch.nn.functional.scaled_dot_product_attention(
                            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True).transpose(1, 2)
                except RuntimeError:
                    o = None
            if o is None:
                from flash_attn import flash_attn_func
                ws = (window, 0) if window < T else (-1, -1)
                o = flash_attn_func(q, k, v, causal=True, window_size=ws)
        ctx.src, ctx.o = src, o
        return o.detach().reshape(B * T, Dl)

    @staticmethod
    def backward(ctx, d_out):
        (g,) = torch.autograd.grad(ctx.o, ctx.src, d_out.view_as(ctx.o))
        ctx.src = ctx.o = None
        return g, None, None, None, None


class LMHeadCEFn(torch.autograd.Function):
    """sum_t loss_t * grad_scale, with d_xf and dW produced during the forward."""

    @staticmethod
    def forward(ctx, xf, w, targets, softcap, grad_scale, chunk, need_grad):
        N, D = xf.shape
        per_tok = torch.empty(N, dtype=torch.float32, device=xf.device)
        d_xf = torch.empty_like(xf) if need_grad else None
        mg = _main_grad(w)
        dw_tmp = None
        if need_grad and mg is None:
            dw_tmp = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        acc = mg if mg is not None else dw_tmp
        for a in range(0, N, chunk):
            b = min(N, a + chunk)
            logits = K.gemm(xf[a:b], w)
            per_tok[a:b] = K.softcap_ce_(logits, targets[a:b], softcap, grad_scale if need_grad else 0.0)
            if need_grad:
                K.gemm(logits, w, trans_b=False, out=d_xf[a:b])
                K.gemm(logits, xf[a:b], trans_a=True, trans_b=False, out=acc, epi=K.EPI_ATOMIC_F32)
        ctx.d_xf = d_xf
        ctx.dw = dw_tmp.to(w.dtype) if dw_tmp is not None else None
        ctx.mark_non_differentiable(per_tok)
        return per_tok.sum() * grad_scale, per_tok

    @staticmethod
    def backward(ctx, g_loss, _g_per_tok):
        # Contract: the caller back-propagates the returned scalar with gradient 1 (the scale
        # is already folded into d_xf and dW).
        d_xf, dw = ctx.d_xf, ctx.dw
        ctx.d_xf = ctx.dw = None
        return d_xf, dw, None, None, None, None, None


# ----------------------------------------------------------------------------------------------
class PeerGrad:
    """A gradient that still lives in every rank's bf16 bucket: the optimizer kernels sum it over
    the ranks while they consume it (reduce-scatter fused into the update)."""

    def __init__(self, peer_ptrs, world, rank, mc_ptr, offset, shape, scale=1.0):
        self.peer_ptrs, self.world, self.rank, self.mc = peer_ptrs, world, rank, mc_ptr
        self.offset, self.shape, self.scale = offset, tuple(shape), scale
        self.is_cuda = True

    def numel(self):
        n = 1
        for d in self.shape:
            n *= d
        return n


class OptimKernels:
    """Fused optimizer steps for MuonAdamW (same math as optim.muon_adamw's reference).

    The Newton-Schulz work buffers (two copies of the stacked matrices, the Gram matrix, the combined polynomial,
    the norm partials and the NorMuon statistics) are allocated once per group shape and reused by every step and
    by every group of that shape: groups run one after the other on one stream.  The reference aliases these
    buffers onto activation gradients (brain/src/optim.rs:742-748,842-848)."""

    MIN_GEMM_DIM = 64

    def __init__(self):
        self._scratch = {}

    def scratch(self, G, m, n, dev):
        key = (G, m, n, str(dev))
        sc = self._scratch.get(key)
        if sc is None:
            d = n if m > n else m
            n_stat = m if m >= n else n
            bf = dict(dtype=torch.bfloat16, device=dev)
            f32 = dict(dtype=torch.float32, device=dev)
            sc = dict(x=torch.empty(G, m, n, **bf), x2=torch.empty(G, m, n, **bf), A=torch.empty(G, d, d, **bf),
                      C=torch.empty(G, d, d, **bf), partials=torch.empty(G * 64, **f32),
                      vmean=torch.empty(G, n_stat, **f32), scale=torch.empty(G, n_stat, **f32))
            self._scratch[key] = sc
        return sc

    def scratch_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for sc in self._scratch.values() for t in sc.values())

    def adamw_group(self, st, grad, pv, step, lr, b1, b2, eps, wd):
        n = grad.numel()
        bc1, bc2 = 1.0 - b1 ** step, 1.0 - b2 ** step
        if isinstance(grad, PeerGrad):
            shadow = pv if pv.dtype == torch.bfloat16 else None
            K._check(K.lib().arb_adamw_rs(st["master"].data_ptr(), grad.peer_ptrs, grad.world, grad.rank, grad.mc, grad.offset,
                                          grad.scale, st["m"].data_ptr(), st["v"].data_ptr(),
                                          shadow.data_ptr() if shadow is not None else 0, n, lr, b1, b2, eps, wd, bc1, bc2,
                                          K._stream()), "adamw_rs")
            if shadow is None:
                pv.copy_(st["master"])
            return
        g = grad if grad.dtype == torch.float32 else grad.float()
        shadow = pv if pv.dtype == torch.bfloat16 else None
        K._check(K.lib().arb_adamw(st["master"].data_ptr(), g.data_ptr(), st["m"].data_ptr(), st["v"].data_ptr(),
                                   shadow.data_ptr() if shadow is not None else 0, n, lr, b1, b2, eps, wd, bc1, bc2,
                                   K._stream()), "adamw")
        if shadow is None:
            pv.copy_(st["master"])

    def muon_group(self, st, grad, pv, mu, lr, wd, beta2, ns_steps):
        from ..optim import muon_adamw as MA
        G, m, n = grad.shape
        if min(m, n) < self.MIN_GEMM_DIM or pv.dtype != torch.bfloat16 or (m % 8) or (n % 8):
            if isinstance(grad, PeerGrad):
                raise RuntimeError("small Muon groups take the unfused path: reduce them first")
            u = MA.muon_nesterov(st["momentum"], grad.float(), mu, torch.bfloat16)
            x = MA.newton_schulz(MA.frob_normalise(u), ns_steps)
            gfin = MA.normuon(x, st["second"], beta2)
            MA.cautious_update(st["master"], gfin, lr, wd)
            pv.copy_(st["master"])
            return
        dev = pv.device
        L = K.lib()
        s = K._stream()
        sc = self.scratch(G, m, n, dev)
        x, x2, A, Cm, sumsq, vmean, scale = sc["x"], sc["x2"], sc["A"], sc["C"], sc["partials"], sc["vmean"], sc["scale"]
        if isinstance(grad, PeerGrad):
            K._check(L.arb_muon_nesterov_rs(st["momentum"].data_ptr(), grad.peer_ptrs, grad.world, grad.rank, grad.mc,
                                            grad.offset, grad.scale, x.data_ptr(), sumsq.data_ptr(), m * n, G, mu, s),
                     "muon_nesterov_rs")
        else:
            K._check(L.arb_muon_nesterov(st["momentum"].data_ptr(), grad.data_ptr(), x.data_ptr(), sumsq.data_ptr(),
                                         m * n, G, mu, s), "muon_nesterov")
        K._check(L.arb_muon_frob_scale(x.data_ptr(), sumsq.data_ptr(), m * n, G, s), "muon_frob_scale")
        tall = m > n
        for a, b, c in MA.POLAR_EXPRESS[:ns_steps]:
            if tall:
                K.gemm(x, x, trans_a=True, trans_b=False, out=A)          # X^T X
            else:
                K.gemm(x, x, out=A)                                        # X X^T
            K.gemm(A, A, out=Cm, epi=K.EPI_NS_COMBINE, aux=A, alpha=a, beta=b, gamma=c)
            if tall:
                K.gemm(x, Cm, out=x2)                                      # X C  (C symmetric)
            else:
                K.gemm(Cm, x, trans_b=False, out=x2)                       # C X
            x, x2 = x2, x
        n_stat = m if m >= n else n
        red = n if m >= n else m
        K._check(L.arb_normuon_stats(x.data_ptr(), vmean.data_ptr(), G, m, n, s), "normuon_stats")
        K._check(L.arb_normuon_scales(vmean.data_ptr(), st["second"].data_ptr(), scale.data_ptr(), G, n_stat, red,
                                      beta2, s), "normuon_scales")
        K._check(L.arb_muon_update(st["master"].data_ptr(), pv.data_ptr(), x.data_ptr(), scale.data_ptr(), G, m, n,
                                   lr, wd, s), "muon_update")


# ----------------------------------------------------------------------------------------------
class Sm100Backend(OracleBackend):
    name = "sm100"

    def __init__(self, attn: str = "own", **kw):
        super().__init__(**kw)
        if not torch.cuda.is_available():
            raise RuntimeError("the sm100 backend needs a CUDA device")
        K.lib()  # fail loudly when the native library is missing
        self.attn = attn
        self.big_ce_chunk = 16384
        self._x0_chain = None

    def optim_kernels(self):
        if getattr(self, "_optim_kernels", None) is None:
            self._optim_kernels = OptimKernels()      # one scratch pool for all optimizers of this backend
        return self._optim_kernels

    def embedding(self, ids, w):
        return EmbeddingFn.apply(ids.contiguous(), w)

    def rmsnorm(self, x):
        return RMSNormFn.apply(x.contiguous(), self.eps)

    def resid_scale_norm(self, x, x0, lam_r, lam_0, i):
        # layers are visited in order within one forward pass: index 0 opens a new x0-gradient chain
        if i == 0 or self._x0_chain is None:
            self._x0_chain = _X0GradChain()
        return ResidScaleNormFn.apply(x.contiguous(), x0.contiguous(), lam_r, lam_0, i, self.eps, self._x0_chain)

    def linear_col(self, x, w):
        return LinearFn.apply(x, w)

    linear_row = linear_col

    def _tp(self):
        tp = getattr(self, "tp", None)
        return tp if (tp is not None and tp.size > 1) else None

    def add_norm(self, x, y):
        return AddNormFn.apply(x, y, self.eps)

    def residual_add(self, x, y):
        return ResidualAddFn.apply(x, y)

    def attention_block(self, xn, blk, ids_flat, B, T, cfg, cos, sin, window):
        tp = self._tp()
        fused_tp = tp if (tp is not None and tp.mode == "fused") else None
        if tp is not None and fused_tp is None:
            xn = tp.all_gather(xn)
        H = blk.wqkv.shape[0] // (3 * cfg.head_dim)
        if cfg.head_dim != 128:
            raise ValueError("the sm100 kernels support head_dim = 128 only")
        qkv = AttnPreFn.apply(xn, blk.wqkv, ids_flat, blk.ve, blk.ve_gate, cos, sin, T, H, cfg.ve_gate_ch, self.eps,
                              fused_tp)
        fn = AttentionFn if self.attn == "own" else LibraryAttentionFn
        return fn.apply(qkv, B, T, H, window)

    def proj_add_norm(self, a, w, x):
        tp = self._tp()
        if tp is None:
            return LinearAddNormFn.apply(a, w, x, self.eps)
        if tp.mode == "fused":
            return AddNormFn.apply(x, TPRowLinearFn.apply(a, w, tp), self.eps)
        return AddNormFn.apply(x, tp.reduce_scatter(LinearFn.apply(a, w)), self.eps)

    def mlp_add(self, xn, wfc, wdn, x):
        tp = self._tp()
        if tp is None:
            return MLPFn.apply(xn, wfc, wdn, x)
        if tp.mode == "fused":
            return TPMLPFn.apply(xn, wfc, wdn, x, tp)
        act = LinearRelu2Fn.apply(tp.all_gather(xn), wfc)
        return ResidualAddFn.apply(x, tp.reduce_scatter(LinearFn.apply(act, wdn)))

    def moe_mlp_add(self, xn, x, blk, moe):
        """x + MoE(xn) and the auxiliary loss; `self.ep` (an EPContext) switches on expert parallelism."""
        from ..models.moe import MoEFn
        return MoEFn.apply(xn, x, blk.router, blk.expert_fc, blk.expert_proj, moe.top_k, moe.aux_coeff,
                           moe.capacity_factor, getattr(self, "ep", None), blk.layer)

    def lm_head_ce(self, xf, w, targets, grad_scale):
        need = torch.is_grad_enabled() and (xf.requires_grad or w.requires_grad)
        chunk = max(self.ce_chunk, self.big_ce_chunk)
        return LMHeadCEFn.apply(xf, w, targets.contiguous(), self.softcap, grad_scale, chunk, need)
