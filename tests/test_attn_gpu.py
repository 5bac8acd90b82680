"""tcgen05 flash attention (forward, dQ, dK/dV) against explicit-mask fp32 attention."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(B, T, H, window, seed=0, mode=2):
    from autoresearch_b200.ops import kernels as K, reference as R, sm100
    K.attn_set_mode(mode)
    try:
        _check(B, T, H, window, seed)
    finally:
        K.attn_set_mode(2)


def _check(B, T, H, window, seed):
    from autoresearch_b200.ops import kernels as K, reference as R, sm100
    torch.manual_seed(seed)
    Dl = H * 128
    qkv = (torch.randn(B * T, 3 * Dl, device="cuda") * 1.0).to(torch.bfloat16).requires_grad_(True)
    out = sm100.AttentionFn.apply(qkv, B, T, H, window)
    g = (torch.randn(B * T, Dl, device="cuda")).to(torch.bfloat16)
    out.backward(g)
    torch.cuda.synchronize()
    K.check_err_flag()
    ref_in = qkv.detach().float().requires_grad_(True)
    q = ref_in[:, :Dl].reshape(B, T, H, 128)
    k = ref_in[:, Dl:2 * Dl].reshape(B, T, H, 128)
    v = ref_in[:, 2 * Dl:].reshape(B, T, H, 128)
    ref = R.attention(q, k, v, window).reshape(B * T, Dl)
    ref.backward(g.float())

    def rel(a, b):
        return ((a.float() - b).norm() / (b.norm() + 1e-12)).item()

    assert rel(out, ref) < 2e-2, f"out {rel(out, ref)}"
    gq, gk, gv = (qkv.grad[:, i * Dl:(i + 1) * Dl] for i in range(3))
    rq, rk, rv = (ref_in.grad[:, i * Dl:(i + 1) * Dl] for i in range(3))
    assert rel(gv, rv) < 3e-2, f"dv {rel(gv, rv)}"
    assert rel(gk, rk) < 3e-2, f"dk {rel(gk, rk)}"
    assert rel(gq, rq) < 3e-2, f"dq {rel(gq, rq)}"


@pytest.mark.parametrize("B,T,H,window", [(1, 128, 1, 128), (2, 256, 2, 256), (1, 512, 2, 256), (1, 1024, 1, 256),
                                         (1, 640, 1, 64), (2, 320, 1, 100), (1, 1536, 2, 1536)])
def test_attention_matches_reference(B, T, H, window):
    _run(B, T, H, window)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("B,T,H,window", [(1, 512, 2, 256), (2, 320, 1, 100), (1, 1536, 2, 1536)])
def test_attention_narrow_variants(B, T, H, window, mode):
    """The 64-wide sub-tile backward (operands in shared memory or TMEM) stays selectable and correct."""
    _run(B, T, H, window, mode=mode)


@pytest.mark.parametrize("B,T,H,window", [(1, 128, 1, 128), (2, 256, 2, 256), (1, 384, 1, 384), (1, 512, 2, 256), (1, 1024, 1, 256),
                                         (1, 640, 1, 64), (2, 320, 1, 100), (1, 1536, 2, 1536), (1, 2000, 1, 700),
                                         (1, 4096, 1, 4096)])
def test_attention_two_query_tiles_forward(B, T, H, window):
    """Forward with two query tiles per CTA in ping-pong (odd tile counts, windows that start mid-pair, ragged tails)."""
    _run(B, T, H, window, mode=3)


@pytest.mark.parametrize("B,T,H,window", [(1, 128, 1, 128), (2, 256, 2, 256), (1, 384, 1, 384), (1, 512, 2, 256), (1, 1024, 1, 256),
                                         (1, 640, 1, 64), (2, 320, 1, 100), (1, 1536, 2, 1536), (1, 2000, 1, 700),
                                         (1, 4096, 1, 4096)])
def test_attention_register_split_forward(B, T, H, window):
    """Forward with the register file split between the roles (score rows held in registers, packed fp32 arithmetic,
    one exponential in four as a polynomial): same cases as the two-query-tile kernel it is derived from."""
    _run(B, T, H, window, mode=4)


def test_attention_long_sequence():
    """Enough tiles for every ring slot and barrier phase to wrap several times."""
    _run(1, 4096, 1, 4096)
    _run(1, 4096, 1, 512, seed=3)


def test_lse_matches_reference():
    from autoresearch_b200.ops import kernels as K, reference as R, sm100
    torch.manual_seed(1)
    B, T, H = 1, 384, 1
    qkv = torch.randn(B * T, 3 * 128, device="cuda").to(torch.bfloat16)
    out = torch.empty(B * T, 128, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, H, T, dtype=torch.float32, device="cuda")
    base = qkv.data_ptr()
    rc = K.lib().arb_attn_fwd(base, base + 256, base + 512, out.data_ptr(), lse.data_ptr(), B, T, H, 384, 384, 384, 128,
                              T, 1 / math.sqrt(128), K.err_flag().data_ptr(), K._stream())
    assert rc == 0
    q, k = qkv[:, :128].float(), qkv[:, 128:256].float()
    s = (q @ k.t()) / math.sqrt(128)
    s = s.masked_fill(~R.window_mask(T, T, "cuda"), float("-inf"))
    assert (torch.logsumexp(s, -1) - lse.view(-1)).abs().max().item() < 2e-2
