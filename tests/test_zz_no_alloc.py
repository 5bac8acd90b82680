"""Allocation-free attention backward (exported C symbol ``arb_attn_bwd_noalloc``).

For callers that cannot hand the library any scratch memory (a host without an allocator at
hand, a thread that must not block in cudaMalloc), the statistic buffer of the backward pass
sits in a fixed array inside the library.  The results must equal those of the regular entry
point bit for bit (the kernels are deterministic), also on a second call that reuses the array with
a different problem size.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(lib, B, T, H, window, seed):
    from autoresearch_b200.ops import kernels as K
    torch.manual_seed(seed)
    Dl = H * 128
    qkv = torch.randn(B * T, 3 * Dl, device="cuda").to(torch.bfloat16)
    d_o = torch.randn(B * T, Dl, device="cuda").to(torch.bfloat16)
    out = torch.empty(B * T, Dl, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, H, T, dtype=torch.float32, device="cuda")
    scale = 1.0 / math.sqrt(128.0)
    err = K.err_flag().data_ptr()
    st = K._stream()
    ld = 3 * Dl
    b = qkv.data_ptr()
    assert lib.arb_attn_fwd(b, b + 2 * Dl, b + 4 * Dl, out.data_ptr(), lse.data_ptr(), B, T, H, ld, ld, ld, Dl,
                            window, scale, err, st) == 0
    ref = torch.zeros_like(qkv)
    delta = torch.empty(B, H, T, dtype=torch.float32, device="cuda")
    r = ref.data_ptr()
    assert lib.arb_attn_bwd(b, b + 2 * Dl, b + 4 * Dl, out.data_ptr(), d_o.data_ptr(), lse.data_ptr(),
                            r, r + 2 * Dl, r + 4 * Dl, delta.data_ptr(), 0, B, T, H, ld, ld, ld, Dl, Dl, ld, ld, ld,
                            window, scale, err, st) == 0
    got = torch.zeros_like(qkv)
    g = got.data_ptr()
    rc = lib.arb_attn_bwd_noalloc(b, b + 2 * Dl, b + 4 * Dl, out.data_ptr(), d_o.data_ptr(), lse.data_ptr(),
                                  g, g + 2 * Dl, g + 4 * Dl, B, T, H, ld, ld, ld, Dl, Dl, ld, ld, ld,
                                  window, scale, err, st)
    assert rc == 0
    torch.cuda.synchronize()
    K.check_err_flag()
    # both entry points run the same deterministic kernels: the results are bitwise equal
    assert torch.equal(got, ref)


def test_noalloc_backward_matches_regular_entry_point_twice():
    from autoresearch_b200.ops import kernels as K
    lib = K.lib()
    vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float
    fn = lib.arb_attn_bwd_noalloc
    fn.restype = C.c_int
    fn.argtypes = [vp] * 9 + [i32, i32, i32] + [i64] * 8 + [i32, f32, vp, vp]
    _case(lib, 2, 384, 2, 384, seed=0)
    _case(lib, 1, 640, 1, 256, seed=1)   # second call: other size, array still holds the first call's data


def test_noalloc_rejects_oversized_problem():
    from autoresearch_b200.ops import kernels as K
    lib = K.lib()
    vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float
    fn = lib.arb_attn_bwd_noalloc
    fn.restype = C.c_int
    fn.argtypes = [vp] * 9 + [i32, i32, i32] + [i64] * 8 + [i32, f32, vp, vp]
    rc = fn(0, 0, 0, 0, 0, 0, 0, 0, 0, 64, 32768, 8, 0, 0, 0, 0, 0, 0, 0, 0, 256, 1.0, 0, 0)
    assert rc == -20
