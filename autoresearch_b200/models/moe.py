"""Top-k mixture-of-experts MLP on the sm_100a kernels.

Math (intended math of brain/src/forward.rs:516-703 and brain/kernels/moe_*.cu): p = softmax(xn
Wr^T) in fp32; top-k experts, gates renormalised over the selected ones; y = sum_k gate_k *
Expert_k(xn) with Expert(x) = relu(x Wfc^T)^2 Wproj^T; auxiliary load-balance loss
coeff * E * sum_e f_e P_e.  Differences from the reference: fixed-capacity expert buffers (token
order decides who is dropped when an expert is over capacity; the reference never drops), no
host synchronisation when a capacity factor is set, experts run as ONE strided-batched tcgen05
GEMM per projection instead of a host loop over cuBLAS calls, deterministic slot order, and
optional expert parallelism where dispatch and combine go through NVLink peer pointers
(``parallel.ep``).
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import kernels as K
from ..ops import reference as R


def _ptr_table(t: torch.Tensor):
    """Host pointer table over the leading (expert) dimension of a local [E, rows, D] tensor."""
    step = t.stride(0) * t.element_size()
    return (C.c_void_p * t.shape[0])(*[t.data_ptr() + e * step for e in range(t.shape[0])])


def _acc_grad(w, dy, x):
    """main_grad(w) += dy^T @ x (batched over experts when 3-D); None when accumulated in place."""
    mg = getattr(w, "main_grad", None)
    tgt = mg if mg is not None else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
    K.gemm(dy, x, trans_a=True, trans_b=False, out=tgt, epi=K.EPI_ATOMIC_F32)
    return None if mg is not None else tgt.to(w.dtype)


def _gather_rows(tab, idx, row, n_rows, k, D, E, resid=None, gates=None):
    """out[t] = (resid[t]) + sum_k (gates[t,k]) * buf[idx[t,k]][row[t,k]] over kept slots."""
    out = torch.empty(n_rows, D, dtype=torch.bfloat16, device=idx.device)
    K._check(K.lib().arb_moe_combine_fwd(resid.data_ptr() if resid is not None else 0, tab, idx.data_ptr(), row.data_ptr(),
                                         gates.data_ptr() if gates is not None else 0, out.data_ptr(), n_rows, k, D, E,
                                         K._stream()), "moe_combine_fwd")
    return out


class MoEFn(torch.autograd.Function):
    """(out, aux) = (resid + MoE(xn), load-balance loss).  w_fc [E_local, M, D], w_proj [E_local, D, M];
    with expert parallelism (`ep`) E_local = E / world and the router still scores all E experts."""

    @staticmethod
    def forward(ctx, xn, resid, router_w, w_fc, w_proj, top_k, aux_coeff, capacity_factor, ep):
        N, D = xn.shape
        E = router_w.shape[0]
        dev = xn.device
        L, s = K.lib(), K._stream()
        probs = torch.empty(N, E, dtype=torch.float32, device=dev)
        idx = torch.empty(N, top_k, dtype=torch.int32, device=dev)
        gates = torch.empty(N, top_k, dtype=torch.float32, device=dev)
        K._check(L.arb_moe_router_fwd(xn.data_ptr(), router_w.data_ptr(), probs.data_ptr(), idx.data_ptr(),
                                      gates.data_ptr(), N, D, E, top_k, s), "moe_router_fwd")
        # position of each slot inside its expert (token order) and the slots per expert
        S = N * top_k
        pos = torch.empty(S, dtype=torch.int32, device=dev)
        counts = torch.empty(E, dtype=torch.int32, device=dev)
        scratch = torch.empty(((S + 1023) // 1024) * E, dtype=torch.int32, device=dev)
        K._check(L.arb_moe_slot_positions(idx.data_ptr(), S, E, scratch.data_ptr(), pos.data_ptr(), counts.data_ptr(), s),
                 "moe_slot_positions")
        if ep is not None:
            cap = ep.cap_src
        elif capacity_factor > 0:
            cap = R.moe_capacity(N, E, top_k, capacity_factor)
        else:
            cap = (int(counts.max().item()) + 7) // 8 * 8     # never drop: one host read per layer
        row = torch.where(pos < cap, pos, torch.full_like(pos, -1)).contiguous()
        f = counts.float() / float(N * top_k)
        aux = aux_coeff * E * (f * probs.mean(0)).sum()
        if ep is None:
            xg = torch.zeros(E, cap, D, dtype=torch.bfloat16, device=dev)
            K._check(L.arb_moe_dispatch(xn.data_ptr(), _ptr_table(xg), idx.data_ptr(), row.data_ptr(), N, top_k, D, E, s),
                     "moe_dispatch")
            act = K.gemm(xg, w_fc, epi=K.EPI_RELU2)
            y = K.gemm(act, w_proj)
            out = _gather_rows(_ptr_table(y), idx, row, N, top_k, D, E, resid, gates)
            y_rows = None
        else:
            ep.local("x").zero_()
            ep.barrier()                                      # every owner has cleared its slabs
            K._check(L.arb_moe_dispatch(xn.data_ptr(), ep.table("x"), idx.data_ptr(), row.data_ptr(), N, top_k, D, E, s),
                     "moe_dispatch")
            ep.barrier()                                      # all routed tokens have arrived
            xg = ep.local("x").clone()
            act = K.gemm(xg, w_fc, epi=K.EPI_RELU2)
            cs = ep.cap_src
            for i in range(ep.world):                         # peers first: their tiles have the longer way
                r = (ep.rank + 1 + i) % ep.world
                K.gemm(act[:, r * cs:(r + 1) * cs], w_proj, out=ep.recv_view("y", r))
            ep.barrier()                                      # every expert's outputs for my tokens have arrived
            out = _gather_rows(ep.recv_table("y"), idx, row, N, top_k, D, E, resid, gates)
            # unscaled expert outputs of this rank's own slots, kept for the gate gradient
            y_rows = _gather_rows(ep.recv_table("y"), idx.view(-1, 1), row.view(-1, 1), N * top_k, 1, D, E)
            y = None
        ctx.save_for_backward(xn, router_w, w_fc, w_proj, probs, idx, gates, row, xg, act,
                              y if y is not None else y_rows, f)
        ctx.cfg = (top_k, aux_coeff, ep)
        return out, aux

    @staticmethod
    def backward(ctx, d_out, g_aux):
        xn, router_w, w_fc, w_proj, probs, idx, gates, row, xg, act, y_or_rows, f = ctx.saved_tensors
        top_k, aux_coeff, ep = ctx.cfg
        N, D = xn.shape
        E = router_w.shape[0]
        dev = xn.device
        L, s = K.lib(), K._stream()
        d_out = d_out.contiguous()
        d_gates = torch.empty(N, top_k, dtype=torch.float32, device=dev)
        if ep is None:
            dy = torch.zeros_like(y_or_rows)
            K._check(L.arb_moe_combine_bwd(d_out.data_ptr(), _ptr_table(y_or_rows), 0, _ptr_table(dy), idx.data_ptr(),
                                           row.data_ptr(), gates.data_ptr(), d_gates.data_ptr(), N, top_k, D, E, s),
                     "moe_combine_bwd")
        else:
            ep.local("dy").zero_()
            ep.barrier()
            K._check(L.arb_moe_combine_bwd(d_out.data_ptr(), 0, y_or_rows.data_ptr(), ep.table("dy"), idx.data_ptr(),
                                           row.data_ptr(), gates.data_ptr(), d_gates.data_ptr(), N, top_k, D, E, s),
                     "moe_combine_bwd")
            ep.barrier()                                      # every source has pushed gate * d_out
            dy = ep.local("dy").clone()
        d_act = K.gemm(dy, w_proj, trans_b=False, epi=K.EPI_RELU2_BWD, aux=act)
        g_proj = _acc_grad(w_proj, dy, act)
        g_fc = _acc_grad(w_fc, d_act, xg)
        if ep is None:
            d_xg = K.gemm(d_act, w_fc, trans_b=False)
            d_xn = _gather_rows(_ptr_table(d_xg), idx, row, N, top_k, D, E)
        else:
            cs = ep.cap_src
            for i in range(ep.world):
                r = (ep.rank + 1 + i) % ep.world
                K.gemm(d_act[:, r * cs:(r + 1) * cs], w_fc, trans_b=False, out=ep.recv_view("dx", r))
            ep.barrier()                                      # the input gradients of my tokens have arrived
            d_xn = _gather_rows(ep.recv_table("dx"), idx, row, N, top_k, D, E)
        aux_dp = None
        if g_aux is not None and aux_coeff != 0.0:
            aux_dp = ((g_aux.float() * (aux_coeff * E / float(N))) * f).contiguous()
        e_pad = (E + 7) // 8 * 8                            # 16-byte rows for the TMA-fed GEMMs below
        d_logits = torch.zeros(N, e_pad, dtype=torch.bfloat16, device=dev)
        K._check(L.arb_moe_router_bwd(probs.data_ptr(), idx.data_ptr(), gates.data_ptr(), d_gates.data_ptr(),
                                      aux_dp.data_ptr() if aux_dp is not None else 0, d_logits.data_ptr(), e_pad, N, E,
                                      top_k, s), "moe_router_bwd")
        d_logits = d_logits[:, :E]
        d_xn = K.gemm(d_logits, router_w, trans_b=False, epi=K.EPI_ADD_AUX, aux=d_xn)
        g_router = _acc_grad(router_w, d_logits, xn)
        return d_xn, d_out, g_router, g_fc, g_proj, None, None, None, None
