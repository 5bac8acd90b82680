"""Top-k mixture-of-experts MLP on the sm_100a kernels.

Math (intended math of brain/src/forward.rs:516-703 and brain/kernels/moe_*.cu): p = softmax(xn
Wr^T) in fp32; top-k experts, gates renormalised over the selected ones; y = sum_k gate_k *
Expert_k(xn) with Expert(x) = relu(x Wfc^T)^2 Wproj^T; auxiliary load-balance loss
coeff * E * sum_e f_e P_e.  Differences from the reference: fixed-capacity expert buffers (token
order decides who is dropped when an expert is over capacity; the reference never drops), no
host synchronisation when a capacity factor is set, deterministic slot order, and the experts run
as ONE ragged grouped tcgen05 GEMM per projection instead of a host loop over cuBLAS calls: the
kernel reads the per-expert row counts from device memory, skips the tiles beyond them (the
capacity padding is never multiplied) and cuts the K range of the weight-gradient products to the
rows that hold data.  With expert parallelism (``parallel.ep``) dispatch and combine go through
NVLink peer pointers and the owner's GEMMs read the received slabs in place.
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


def _finish(L, s, table, cnt_table, counts, keep, cap, D, E, tile):
    K._check(L.arb_moe_finish_dispatch(table, cnt_table, counts.data_ptr(), keep, cap, D, E, tile, s), "moe_finish_dispatch")


class MoEFn(torch.autograd.Function):
    """(out, aux) = (resid + MoE(xn), load-balance loss).  w_fc [E_local, M, D], w_proj [E_local, D, M];
    with expert parallelism (`ep`) E_local = E / world and the router still scores all E experts."""

    TILE = 256

    @staticmethod
    def forward(ctx, xn, resid, router_w, w_fc, w_proj, top_k, aux_coeff, capacity_factor, ep, layer):
        N, D = xn.shape
        E = router_w.shape[0]
        M = w_fc.shape[1]
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
        # `keep`: slots an expert accepts (the rule of ops.reference.moe_capacity); `cap`: rows of a slab, a multiple
        # of 64 (K blocks of the weight-gradient products)
        if ep is not None:
            keep, cap = ep.keep, ep.cap_src
        elif capacity_factor > 0:
            keep = R.moe_capacity(N, E, top_k, capacity_factor)
            cap = (keep + 63) // 64 * 64
        else:
            # never drop (the reference's behaviour): the buffer size depends on the routing, one host read per layer
            keep = int(counts.max().item())
            cap = (keep + 63) // 64 * 64
        row = torch.where(pos < keep, pos, torch.full_like(pos, -1)).contiguous()
        f = counts.float() / float(N * top_k)
        aux = aux_coeff * E * (f * probs.mean(0)).sum()
        T_ = MoEFn.TILE
        lib_ep = ep is not None and ep.mode == "library"
        if ep is None or lib_ep:
            W = 1 if ep is None else ep.world
            xg = torch.empty(E, cap, D, dtype=torch.bfloat16, device=dev)
            y = torch.empty(E, cap, D, dtype=torch.bfloat16, device=dev)
            mv = torch.empty(E, dtype=torch.int32, device=dev)
            x_tab = _ptr_table(xg)
            cnt_tab = (C.c_void_p * E)(*[mv.data_ptr() + 4 * e for e in range(E)])
            K._check(L.arb_moe_dispatch(xn.data_ptr(), x_tab, idx.data_ptr(), row.data_ptr(), N, top_k, D, E, s), "moe_dispatch")
            _finish(L, s, x_tab, cnt_tab, counts, keep, cap, D, E, T_)
            if lib_ep:                                        # library all-to-all of the padded slabs and their counts
                xg, mv = ep.to_owners(xg), ep.to_owners(mv)
                y = torch.empty_like(xg)
        else:
            W = ep.world
            x_tab, y_tab = ep.table("x", layer), ep.table("y", layer)
            K._check(L.arb_moe_dispatch(xn.data_ptr(), x_tab, idx.data_ptr(), row.data_ptr(), N, top_k, D, E, s), "moe_dispatch")
            _finish(L, s, x_tab, ep.table("cnt", layer), counts, keep, cap, D, E, T_)
            ep.barrier()                                      # all routed tokens and their counts have arrived
            xg, y, mv = ep.local("x", layer), ep.local("y", layer), ep.local("cnt", layer)
        act = torch.empty(xg.shape[0], cap, M, dtype=torch.bfloat16, device=dev)
        K.gemm(xg, w_fc, out=act, epi=K.EPI_RELU2, m_valid=mv, b_div=W)
        K.gemm(act, w_proj, out=y, m_valid=mv, b_div=W)
        if lib_ep:
            y_src = ep.to_sources(y)                          # expert outputs of this rank's tokens, by expert
            y_tab = _ptr_table(y_src)
            y = y_src                                         # what the backward reads for the gate gradient
        elif ep is None:
            y_tab = _ptr_table(y)
        else:
            ep.barrier()                                      # every expert's outputs are complete
        out = _gather_rows(y_tab, idx, row, N, top_k, D, E, resid, gates)
        ctx.save_for_backward(xn, router_w, w_fc, w_proj, probs, idx, gates, row, xg, act, y, f, counts, mv)
        ctx.cfg = (top_k, aux_coeff, ep, layer, keep, cap)
        return out, aux

    @staticmethod
    def backward(ctx, d_out, g_aux):
        xn, router_w, w_fc, w_proj, probs, idx, gates, row, xg, act, y, f, counts, mv = ctx.saved_tensors
        top_k, aux_coeff, ep, layer, keep, cap = ctx.cfg
        N, D = xn.shape
        E = router_w.shape[0]
        El = w_fc.shape[0]
        dev = xn.device
        L, s = K.lib(), K._stream()
        T_ = MoEFn.TILE
        d_out = d_out.contiguous()
        d_gates = torch.empty(N, top_k, dtype=torch.float32, device=dev)
        lib_ep = ep is not None and ep.mode == "library"
        if ep is None or lib_ep:
            W = 1 if ep is None else ep.world
            dy = torch.empty_like(y)
            d_xg = torch.empty_like(xg)
            y_tab, dy_tab, dx_tab = _ptr_table(y), _ptr_table(dy), _ptr_table(d_xg)
        else:
            W = ep.world
            y_tab, dy_tab, dx_tab = ep.table("y", layer), ep.table("dy"), ep.table("dx")
            dy, d_xg = ep.local("dy"), ep.local("dx")
        # d(expert output) = gate * d_out scattered to the owners; d(gate) = <expert output, d_out> (outputs read in place)
        K._check(L.arb_moe_combine_bwd(d_out.data_ptr(), y_tab, 0, dy_tab, idx.data_ptr(), row.data_ptr(), gates.data_ptr(),
                                       d_gates.data_ptr(), N, top_k, D, E, s), "moe_combine_bwd")
        _finish(L, s, dy_tab, None, counts, keep, cap, D, E, T_)
        if lib_ep:
            dy = ep.to_owners(dy)
        elif ep is not None:
            ep.barrier()                                      # every source has pushed gate * d_out
        d_act = torch.empty_like(act)
        K.gemm(dy, w_proj, trans_b=False, out=d_act, epi=K.EPI_RELU2_BWD, aux=act, m_valid=mv, b_div=W)
        kv = mv.view(El, W)
        flat = lambda t: t.view(El, W * cap, t.shape[-1])

        def acc_grad(w, a, b):
            mg = getattr(w, "main_grad", None)
            tgt = mg if mg is not None else torch.zeros(w.shape, dtype=torch.float32, device=dev)
            K.gemm(flat(a), flat(b), trans_a=True, trans_b=False, out=tgt, epi=K.EPI_ATOMIC_F32, k_valid=kv, k_seg=cap)
            return None if mg is not None else tgt.to(w.dtype)

        g_proj = acc_grad(w_proj, dy, act)
        g_fc = acc_grad(w_fc, d_act, xg)
        K.gemm(d_act, w_fc, trans_b=False, out=d_xg, m_valid=mv, b_div=W)
        if lib_ep:
            dx_tab = _ptr_table(ep.to_sources(d_xg))
        elif ep is not None:
            ep.barrier()                                      # the input gradients of my tokens are complete
        d_xn = _gather_rows(dx_tab, idx, row, N, top_k, D, E)
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
        return d_xn, d_out, g_router, g_fc, g_proj, None, None, None, None, None
