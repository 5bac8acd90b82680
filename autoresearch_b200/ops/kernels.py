"""ctypes binding of ``_arb_kernels.so`` plus thin tensor-level wrappers.

Every wrapper validates dtype / device / contiguity and raises on a non-zero return code,
so a missing or failing native kernel is never silently replaced by a PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from . import build as _build

_lib = None
_gemm_mode = 0       # as set by gemm_set_mode: 0 automatic, 1 always 1-CTA tiles, 2 always 2-CTA tiles
_err_flag = {}

EPI_STORE_BF16, EPI_RELU2, EPI_ATOMIC_F32, EPI_NS_COMBINE, EPI_RELU2_BWD, EPI_STORE_F32, EPI_ADD_AUX, EPI_QKV_POST = range(8)
ERR_NAMES = {1: "GEMM barrier wait timed out", 2: "attention barrier wait timed out",
             3: "peer barrier wait timed out", 4: "MoE dispatch wait timed out",
             5: "dynamic shared memory base is not 1 KB aligned"}

launch_count = 0  # number of kernel-launching calls made through this module
# B operands whose up-to-date copy still sits on another rank: data_ptr -> (peer pointer, bytes), registered by
# parallel/fused_dp.py after every optimizer step.  GEMMs on the stream the entries were registered on work the
# list off: a GEMM whose own B is still pending copies it in its prologue; every GEMM also lets a spare warp copy
# the oldest other pending entry while its tiles are computed ("ahead" copy), so that from the second GEMM of a
# step on the operand is already local when its consumer starts.  pull_use_order remembers in which order the
# operands were consumed, and fused_dp registers them in that order.
pending_pulls = {}
pull_stream = None
pull_use_order = {}
PULL_AHEAD = True


class KernelError(RuntimeError):
    pass


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not _build.is_current():
        _build.build()
    L = C.CDLL(str(_build.SO))
    for name, args in _signatures().items():
        if hasattr(L, name):
            f = getattr(L, name)
            f.restype = C.c_int
            f.argtypes = args
    _lib = L
    return L


def _signatures() -> dict:
    """ctypes argument lists of the entry points declared in csrc/api.h (a CPU test counts them against the header)."""
    vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float
    return {
        "arb_gemm_bf16": [vp, vp, vp, vp, i32, i32, i32, i32, i64, i64, i64, i64, i64, i64, i32, i32, i32, i32,
                          f32, f32, f32, vp, vp],
        "arb_gemm_bf16_ex": [vp, vp, vp, vp, i32, i32, i32, i32, i64, i64, i64, i64, i64, i64, i32, i32, i32, i32,
                             f32, f32, f32, vp, vp, vp, i64, vp, vp, i64],
        "arb_gemm_bf16_ragged": [vp, vp, vp, vp, i32, i32, i32, i32, i64, i64, i64, i64, i64, i64, i32, i32, i32, i32,
                                 f32, f32, f32, vp, vp, vp, i64, vp, vp, i64, vp, i32, vp, i32],
        "arb_attn_fwd": [vp, vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, i32, f32, vp, vp],
        "arb_attn_bwd": [vp] * 11 + [i32, i32, i32] + [i64] * 8 + [i32, f32, vp, vp],
        "arb_rmsnorm_fwd": [vp, vp, i64, i32, f32, vp],
        "arb_rmsnorm_bwd": [vp, vp, vp, vp, i64, i32, f32, vp],
        "arb_resid_scale_norm_fwd": [vp, vp, vp, vp, i32, vp, vp, i64, i32, f32, vp],
        "arb_resid_scale_norm_bwd": [vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, vp, vp, i64, i32, f32, vp],
        "arb_add_norm_fwd": [vp, vp, vp, vp, i64, i32, f32, vp],
        "arb_residual_add": [vp, vp, vp, i64, vp],
        "arb_relu_sq_fwd": [vp, vp, i64, vp],
        "arb_relu_sq_bwd": [vp, vp, vp, i64, vp],
        "arb_qkv_post_fwd": [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, f32, vp],
        "arb_gemm_qkv_post_args": [vp, vp, vp, i32, i32, vp, i64, vp, vp, vp, vp, i32, f32],
        "arb_qkv_post_bwd": [vp] * 14 + [i64, i32, i32, i32, i32, vp],
        "arb_embedding_fwd": [vp, vp, vp, i64, i32, i32, vp],
        "arb_embedding_bwd": [vp, vp, vp, i64, i32, i32, vp],
        "arb_embedding_bwd_sorted": [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp],
        "arb_add_cols": [vp, i64, vp, i64, i32, vp],
        "arb_cast_f32_to_bf16": [vp, vp, i64, f32, vp],
        "arb_accum_bf16_into_f32": [vp, vp, i64, vp],
        "arb_softcap_ce": [vp, i64, vp, vp, i64, i32, f32, f32, vp],
        "arb_adamw": [vp, vp, vp, vp, vp, i64, f32, f32, f32, f32, f32, f32, f32, vp],
        "arb_muon_nesterov": [vp, vp, vp, vp, i64, i32, f32, vp],
        "arb_muon_frob_scale": [vp, vp, i64, i32, vp],
        "arb_muon_nesterov_rs": [vp, vp, i32, i32, vp, i64, f32, vp, vp, i64, i32, f32, vp],
        "arb_adamw_rs": [vp, vp, i32, i32, vp, i64, f32, vp, vp, vp, i64, f32, f32, f32, f32, f32, f32, f32, vp],
        "arb_normuon_stats": [vp, vp, i32, i32, i32, vp],
        "arb_normuon_scales": [vp, vp, vp, i32, i32, i32, f32, vp],
        "arb_muon_update": [vp, vp, vp, vp, i32, i32, i32, f32, f32, vp],
        "arb_reduce_scatter_peers": [vp, i32, i64, i64, i32, vp, f32, vp],
        "arb_reduce_scatter_multimem": [vp, i64, i64, i32, vp, f32, vp],
        "arb_sum_slabs_bf16": [vp, i32, i64, vp, vp],
        "arb_all_gather_push": [vp, i32, i32, vp, i64, i64, vp],
        "arb_all_gather_pull": [vp, i32, i32, vp, i64, vp],
        "arb_peer_barrier": [vp, i32, i32, i32, vp, vp],
        "arb_pull_ranges": [vp, vp, vp, i32, vp],
        "arb_moe_router_fwd": [vp, vp, vp, vp, vp, i64, i32, i32, i32, vp],
        "arb_moe_router_bwd": [vp, vp, vp, vp, vp, vp, i64, i64, i32, i32, vp],
        "arb_moe_slot_positions": [vp, i64, i32, vp, vp, vp, vp],
        "arb_moe_dispatch": [vp, vp, vp, vp, i64, i32, i32, i32, vp],
        "arb_moe_finish_dispatch": [vp, vp, vp, i32, i32, i32, i32, i32, vp],
        "arb_moe_combine_fwd": [vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, vp],
        "arb_moe_combine_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, vp],
    }


def available() -> bool:
    try:
        lib()
        return True
    except Exception:
        return False


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, what: str):
    global launch_count
    launch_count += 1
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


def err_flag(device=None) -> torch.Tensor:
    """Per-device int32 status word written by kernels whose bounded waits expire."""
    dev = torch.device(device if device is not None else torch.cuda.current_device())
    if dev.type != "cuda":
        dev = torch.device("cuda", torch.cuda.current_device())
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _err_flag:
        _err_flag[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _err_flag[key]


def check_err_flag(device=None) -> None:
    """Host-side check (one device->host read); raises if any kernel reported a timeout."""
    f = err_flag(device)
    v = int(f.item())
    if v != 0:
        f.zero_()
        raise KernelError(ERR_NAMES.get(v, f"kernel error {v}"))


def _bf16(t: torch.Tensor, name: str):
    if not (t.is_cuda and t.dtype == torch.bfloat16):
        raise TypeError(f"{name} must be a CUDA bf16 tensor")


def _row_major_2d(t: torch.Tensor, name: str):
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with unit inner stride")


# --------------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = True,
         out: Optional[torch.Tensor] = None, epi: int = EPI_STORE_BF16, aux: Optional[torch.Tensor] = None,
         splitk: int = 0, alpha: float = 0.0, beta: float = 0.0, gamma: float = 1.0,
         m_valid: Optional[torch.Tensor] = None, b_div: int = 1, k_valid: Optional[torch.Tensor] = None,
         k_seg: int = 0, post: Optional[dict] = None) -> torch.Tensor:
    """C = op(A) @ op(B) on the tcgen05 kernel.

    2-D or batched 3-D bf16 operands with unit inner stride.  ``trans_a=False``: ``a`` is
    [M, K]; True: ``a`` is [K, M] (A = a^T).  ``trans_b=True`` (default, "NT"): ``b`` is
    [N, K] (B = b^T); False: ``b`` is [K, N].

    Ragged batches (grouped expert GEMMs): ``m_valid`` int32 [G] = rows of each batch item that hold data (output
    tiles beyond are neither computed nor written); ``b_div``: ``b`` holds G / b_div matrices, item g uses matrix
    g // b_div; ``k_valid`` int32 [G, K // k_seg] with ``k_seg`` rows per segment: for EPI_ATOMIC_F32 products over
    rows, only the 64-row blocks below ``k_valid`` of each segment are multiplied.

    ``epi=EPI_QKV_POST`` with ``post`` = the arguments of :func:`qkv_post_args`: the packed q|k|v projection with
    RoPE + RMS norm of the q / k heads and the value embedding of the v heads done in the epilogue.
    """
    _bf16(a, "a"); _bf16(b, "b")
    batched = a.dim() == 3
    if batched:
        G = a.shape[0]
        a2, b2 = a[0], b[0]
        sa, sb = a.stride(0), b.stride(0)
        if b.shape[0] * b_div != G:
            raise ValueError(f"b holds {b.shape[0]} matrices for {G} batch items with b_div={b_div}")
    else:
        G, a2, b2, sa, sb = 1, a, b, 0, 0
    _row_major_2d(a2, "a"); _row_major_2d(b2, "b")
    if trans_a:
        K, M = a2.shape
    else:
        M, K = a2.shape
    if trans_b:
        N, Kb = b2.shape
    else:
        Kb, N = b2.shape
    if K != Kb:
        raise ValueError(f"inner dimensions differ: {K} vs {Kb}")
    f32_out = epi in (EPI_ATOMIC_F32, EPI_STORE_F32)
    if out is None:
        shape = (G, M, N) if batched else (M, N)
        if epi == EPI_ATOMIC_F32:
            raise ValueError("EPI_ATOMIC_F32 accumulates into an existing tensor: pass out=")
        out = torch.empty(shape, dtype=torch.float32 if f32_out else torch.bfloat16, device=a.device)
    o2 = out[0] if batched else out
    _row_major_2d(o2, "out")
    if tuple(o2.shape) != (M, N) or out.dtype != (torch.float32 if f32_out else torch.bfloat16):
        raise ValueError("out has the wrong shape or dtype")
    so = out.stride(0) if batched else 0
    pull = ahead = None
    if pending_pulls:
        stream = _stream()
        pull = pending_pulls.pop(b.data_ptr(), None)
        if pull is not None:
            pull_use_order.setdefault(b.data_ptr(), len(pull_use_order))
        if PULL_AHEAD and stream == pull_stream and pending_pulls:
            dst = next(iter(pending_pulls))
            ahead = (dst,) + pending_pulls.pop(dst)
            pull_use_order.setdefault(dst, len(pull_use_order))
    auxp = 0
    if aux is not None:
        _bf16(aux, "aux")
        ax2 = aux[0] if batched else aux
        if ax2.stride(0) != o2.stride(0) or tuple(ax2.shape) != (M, N) or (batched and aux.stride(0) != so):
            raise ValueError("aux must have the layout of out")
        auxp = aux.data_ptr()
    for t, n_want, nm in ((m_valid, G, "m_valid"), (k_valid, G * (K // k_seg) if k_seg else -1, "k_valid")):
        if t is not None and (t.dtype != torch.int32 or not t.is_cuda or not t.is_contiguous() or t.numel() != n_want):
            raise ValueError(f"{nm} must be a contiguous CUDA int32 tensor of {n_want} elements")
    try:
        if (epi == EPI_QKV_POST) != (post is not None):
            raise ValueError("EPI_QKV_POST and post= go together")
        if post is not None:
            qkv_post_args(**post)
        rc = lib().arb_gemm_bf16_ragged(a.data_ptr(), b.data_ptr(), out.data_ptr(), auxp, M, N, K, G,
                                        a2.stride(0), b2.stride(0), o2.stride(0), sa, sb, so,
                                        int(trans_a), int(not trans_b), epi, splitk, alpha, beta, gamma,
                                        err_flag(a.device).data_ptr(), _stream(),
                                        pull[0] if pull else None, pull[1] if pull else 0,
                                        ahead[1] if ahead else None, ahead[0] if ahead else None, ahead[2] if ahead else 0,
                                        m_valid.data_ptr() if m_valid is not None else None, b_div,
                                        k_valid.data_ptr() if k_valid is not None else None, k_seg)
        _check(rc, "arb_gemm_bf16")
    except Exception:
        # nothing was launched: the copies are still owed
        if ahead is not None:
            pending_pulls[ahead[0]] = ahead[1:]
        if pull is not None:
            pending_pulls[b.data_ptr()] = pull
        raise
    return out


def qkv_post_args(cos, sin, rstd, T, H, xn=None, ids=None, ve_w=None, gate_w=None, gate=None, gate_ch=0, eps=1e-6) -> None:
    """Parameters of the next EPI_QKV_POST product on this thread (rstd [rows, 2H] fp32 and, with a value embedding,
    gate [rows, H] fp32 are outputs)."""
    has_ve = ve_w is not None
    _check(lib().arb_gemm_qkv_post_args(cos.data_ptr(), sin.data_ptr(), rstd.data_ptr(), T, H,
                                        xn.data_ptr() if has_ve else None, xn.stride(0) if has_ve else 0,
                                        ids.data_ptr() if has_ve else None, ve_w.data_ptr() if has_ve else None,
                                        gate_w.data_ptr() if has_ve else None, gate.data_ptr() if has_ve else None,
                                        gate_ch if has_ve else 0, eps), "gemm_qkv_post_args")


def qkv_post_fusable(rows: int, cols: int) -> bool:
    """The fused epilogue exists in the 2-CTA kernel only (products of at least 512 rows and 256 columns)."""
    if os.environ.get("ARB_QKV_EPILOGUE", "1") == "0" or _gemm_mode == 1:
        return False
    return _gemm_mode == 2 or (rows >= 512 and cols >= 256)


def gemm_set_mode(mode: int) -> None:
    """0 = automatic tile choice, 1 = always 1-CTA tiles, 2 = always 2-CTA (cta_group::2) tiles."""
    global _gemm_mode
    f = lib().arb_gemm_set_mode
    f.restype, f.argtypes = C.c_int, [C.c_int]
    if f(mode) != 0:
        raise ValueError(f"bad GEMM mode {mode}")
    _gemm_mode = mode


def flush_pending_pulls() -> None:
    """Materialise every operand that no GEMM has pulled yet (before anything else reads the parameters)."""
    if not pending_pulls:
        return
    items = list(pending_pulls.items())
    pending_pulls.clear()
    n = len(items)
    src = (C.c_void_p * n)(*[v[0] for _, v in items])
    dst = (C.c_void_p * n)(*[k for k, _ in items])
    nb = (C.c_longlong * n)(*[v[1] for _, v in items])
    _check(lib().arb_pull_ranges(src, dst, nb, n, _stream()), "pull_ranges")


def attn_set_mode(mode: int) -> None:
    """4 = as 2, with the register-split two-query-tile forward (attn_fwd3) for every shape;
    3 = as 2, with the forward on two query tiles per CTA in ping-pong; 2 = backward on 128 x 128 tiles with
    the two-phase softmax; 1 = 64-wide sub-tiles with P / dS operands in TMEM; 0 = 64-wide sub-tiles with P / dS
    in shared memory (forward too)."""
    f = lib().arb_attn_set_mode
    f.restype, f.argtypes = None, [C.c_int]
    f(int(mode))


def rmsnorm_fwd(x, eps):
    _bf16(x, "x")
    y = torch.empty_like(x)
    _check(lib().arb_rmsnorm_fwd(x.data_ptr(), y.data_ptr(), x.numel() // x.shape[-1], x.shape[-1], eps, _stream()), "rmsnorm_fwd")
    return y


def rmsnorm_bwd(x, g, eps, add_to=None):
    gx = torch.empty_like(x)
    _check(lib().arb_rmsnorm_bwd(x.data_ptr(), g.data_ptr(), add_to.data_ptr() if add_to is not None else 0,
                                 gx.data_ptr(), x.numel() // x.shape[-1], x.shape[-1], eps, _stream()), "rmsnorm_bwd")
    return gx


def resid_scale_norm_fwd(x, x0, lam_r, lam_0, idx, eps):
    xo, xn = torch.empty_like(x), torch.empty_like(x)
    _check(lib().arb_resid_scale_norm_fwd(x.data_ptr(), x0.data_ptr(), lam_r.data_ptr(), lam_0.data_ptr(), idx,
                                          xo.data_ptr(), xn.data_ptr(), x.shape[0], x.shape[1], eps, _stream()),
           "resid_scale_norm_fwd")
    return xo, xn


def resid_scale_norm_bwd(x, x0, lam_r, lam_0, idx, g_xs, g_xn, dlam_r, dlam_0, eps, dx0_acc=None):
    """dx0_acc: the x0 gradient summed over the layers above; this layer's share is added to it in place and the
    same tensor is returned, which saves one pass over [N, D] per layer."""
    dx = torch.empty_like(x)
    dx0 = dx0_acc if dx0_acc is not None else torch.empty_like(x)
    _check(lib().arb_resid_scale_norm_bwd(x.data_ptr(), x0.data_ptr(), lam_r.data_ptr(), lam_0.data_ptr(), idx,
                                          g_xs.data_ptr(), g_xn.data_ptr(), dx.data_ptr(), dx0.data_ptr(),
                                          dx0_acc.data_ptr() if dx0_acc is not None else None,
                                          dlam_r.data_ptr(), dlam_0.data_ptr(), x.shape[0], x.shape[1], eps, _stream()),
           "resid_scale_norm_bwd")
    return dx, dx0


def add_norm_fwd(x, proj, eps):
    xo, xn = torch.empty_like(x), torch.empty_like(x)
    _check(lib().arb_add_norm_fwd(x.data_ptr(), proj.data_ptr(), xo.data_ptr(), xn.data_ptr(), x.shape[0], x.shape[1],
                                  eps, _stream()), "add_norm_fwd")
    return xo, xn


def residual_add(a, b):
    o = torch.empty_like(a)
    _check(lib().arb_residual_add(a.data_ptr(), b.data_ptr(), o.data_ptr(), a.numel(), _stream()), "residual_add")
    return o


def relu_sq_fwd(x):
    y = torch.empty_like(x)
    _check(lib().arb_relu_sq_fwd(x.data_ptr(), y.data_ptr(), x.numel(), _stream()), "relu_sq_fwd")
    return y


def relu_sq_bwd(x, g):
    o = torch.empty_like(x)
    _check(lib().arb_relu_sq_bwd(x.data_ptr(), g.data_ptr(), o.data_ptr(), x.numel(), _stream()), "relu_sq_bwd")
    return o


def embedding_fwd(ids, w):
    out = torch.empty(ids.numel(), w.shape[1], dtype=w.dtype, device=w.device)
    _check(lib().arb_embedding_fwd(ids.data_ptr(), w.data_ptr(), out.data_ptr(), ids.numel(), w.shape[1], w.shape[0],
                                   _stream()), "embedding_fwd")
    return out


EMB_BWD_DETERMINISTIC = True   # sorted, atomic-free embedding gradient (False: fp32 atomics)
EMB_BWD_ROWS_PER_ITEM = 64
_emb_plan = {}


def _embedding_plan(ids, vocab: int):
    """Sort order and work-item tables of one batch of token ids; cached, since the word-embedding and every
    value-embedding gradient of a micro-batch use the same ids.  Fixed-size tensors only (no host sync)."""
    key = (ids.data_ptr(), ids._version, ids.numel(), vocab)
    hit = _emb_plan.get(("plan", ids.device.index))
    if hit is not None and hit[0] == key:
        return hit[1]
    R = EMB_BWD_ROWS_PER_ITEM
    N = ids.numel()
    flat = ids.reshape(-1).long().clamp(0, vocab - 1)
    perm = torch.sort(flat, stable=True).indices.contiguous()                     # int64 [N]
    # (torch.bincount reads the largest id back to the host to size its result: a sync per micro-batch)
    counts = torch.zeros(vocab, dtype=torch.int64, device=ids.device).scatter_add_(0, flat, torch.ones_like(flat))
    seg_start = (torch.cumsum(counts, 0) - counts).to(torch.int32)
    n_it = (counts + R - 1) // R
    it_end = torch.cumsum(n_it, 0)
    item_start = (it_end - n_it).to(torch.int32)
    n_max = N // R + vocab + 1                                                     # upper bound of the item count
    item = torch.arange(n_max, device=ids.device)
    item_id = torch.searchsorted(it_end, item, right=True)
    item_id = torch.where(item < it_end[-1], item_id, torch.full_like(item_id, -1)).to(torch.int32)
    plan = (perm, item_id.contiguous(), item_start.contiguous(), seg_start.contiguous(), counts.to(torch.int32).contiguous(), n_max)
    _emb_plan[("plan", ids.device.index)] = (key, plan)
    return plan


def embedding_bwd(ids, g, dw_f32):
    """dw[id] += sum of the rows of g whose token is id."""
    D, vocab = g.shape[-1], dw_f32.shape[0]
    if not EMB_BWD_DETERMINISTIC:
        _check(lib().arb_embedding_bwd(ids.data_ptr(), g.data_ptr(), dw_f32.data_ptr(), ids.numel(), D, vocab, _stream()),
               "embedding_bwd")
        return
    perm, item_id, item_start, seg_start, counts, n_max = _embedding_plan(ids, vocab)
    scratch = _emb_plan.get(("scratch", g.device.index))
    if scratch is None or scratch.numel() < n_max * D:
        scratch = torch.empty(n_max * D, dtype=torch.float32, device=g.device)
        _emb_plan[("scratch", g.device.index)] = scratch
    _check(lib().arb_embedding_bwd_sorted(perm.data_ptr(), item_id.data_ptr(), item_start.data_ptr(), seg_start.data_ptr(),
                                          counts.data_ptr(), g.data_ptr(), dw_f32.data_ptr(), scratch.data_ptr(), n_max, D,
                                          EMB_BWD_ROWS_PER_ITEM, vocab, _stream()), "embedding_bwd_sorted")


def softcap_ce_(logits, targets, softcap, dlogits_scale):
    """Returns per-row losses; overwrites logits with their gradient when dlogits_scale != 0."""
    loss = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
    _check(lib().arb_softcap_ce(logits.data_ptr(), logits.stride(0), targets.data_ptr(), loss.data_ptr(),
                                logits.shape[0], logits.shape[1], softcap, dlogits_scale, _stream()), "softcap_ce")
    return loss


def cast_f32_to_bf16(src, dst, scale=1.0):
    _check(lib().arb_cast_f32_to_bf16(src.data_ptr(), dst.data_ptr(), src.numel(), scale, _stream()), "cast_f32_to_bf16")


def accum_bf16_into_f32(src, dst):
    _check(lib().arb_accum_bf16_into_f32(src.data_ptr(), dst.data_ptr(), src.numel(), _stream()), "accum_bf16_into_f32")


def add_cols_(dst, src):
    """dst[:, :src.shape[1]] += src (dst may be wider)."""
    _check(lib().arb_add_cols(dst.data_ptr(), dst.stride(0), src.data_ptr(), src.shape[0], src.shape[1], _stream()), "add_cols")
