"""Fused elementwise / norm / CE / optimizer kernels against the PyTorch fp32 reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

EPS = 1e-5


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _close(a, b, tol=2e-2, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    den = b.abs().max().item() + 1e-6
    assert err / den < tol, f"{what} rel err {err / den:.4g}"


@pytest.mark.parametrize("rows,D", [(37, 256), (64, 512), (100, 1024), (9, 2048), (16, 136)])
def test_rmsnorm_fwd_bwd(rows, D):
    from autoresearch_b200.ops import kernels as K, reference as R
    torch.manual_seed(0)
    x, g = _bf(rows, D), _bf(rows, D)
    _close(K.rmsnorm_fwd(x, EPS), R.rmsnorm(x.float(), EPS), what="fwd")
    xf = x.float().requires_grad_(True)
    R.rmsnorm(xf, EPS).backward(g.float())
    _close(K.rmsnorm_bwd(x, g, EPS), xf.grad, what="bwd")
    add = _bf(rows, D)
    _close(K.rmsnorm_bwd(x, g, EPS, add_to=add), xf.grad + add.float(), what="bwd+add")


def test_resid_scale_norm_fwd_bwd():
    from autoresearch_b200.ops import kernels as K, reference as R
    torch.manual_seed(1)
    rows, D, L, idx = 50, 512, 4, 2
    x, x0 = _bf(rows, D), _bf(rows, D)
    lr = torch.tensor([1.0, 0.9, 1.1, 0.8], device="cuda").to(torch.bfloat16)
    l0 = torch.tensor([0.1, 0.2, 0.3, 0.05], device="cuda").to(torch.bfloat16)
    xs, xn = K.resid_scale_norm_fwd(x, x0, lr, l0, idx, EPS)
    xf, x0f = x.float().requires_grad_(True), x0.float().requires_grad_(True)
    lrf, l0f = lr.float().requires_grad_(True), l0.float().requires_grad_(True)
    rs, rn = R.resid_scale_norm(xf, x0f, lrf[idx], l0f[idx], EPS)
    _close(xs, rs, what="xs"); _close(xn, rn, what="xn")
    g1, g2 = _bf(rows, D), _bf(rows, D)
    (rs * g1.float()).sum().backward(retain_graph=True)
    (rn * g2.float()).sum().backward()
    dr = torch.zeros(L, device="cuda"); d0 = torch.zeros(L, device="cuda")
    dx, dx0 = K.resid_scale_norm_bwd(x, x0, lr, l0, idx, g1, g2, dr, d0, EPS)
    _close(dx, xf.grad, what="dx"); _close(dx0, x0f.grad, what="dx0")
    _close(dr, lrf.grad, 3e-2, "dlam_r"); _close(d0, l0f.grad, 3e-2, "dlam_0")
    # accumulate form: the x0 gradient of the layers above is added in place
    acc = _bf(rows, D)
    want = acc.float() + x0f.grad
    dr2 = torch.zeros(L, device="cuda"); d02 = torch.zeros(L, device="cuda")
    dx2, out = K.resid_scale_norm_bwd(x, x0, lr, l0, idx, g1, g2, dr2, d02, EPS, dx0_acc=acc)
    assert out.data_ptr() == acc.data_ptr() and torch.equal(dx2, dx)
    _close(out, want, what="dx0 accumulated")


def test_add_norm_relu_residual_embedding():
    from autoresearch_b200.ops import kernels as K, reference as R
    torch.manual_seed(2)
    x, p = _bf(33, 512), _bf(33, 512)
    xs, xn = K.add_norm_fwd(x, p, EPS)
    rs, rn = R.add_norm(x.float(), p.float(), EPS)
    _close(xs, rs); _close(xn, rn)
    _close(K.residual_add(x, p), x.float() + p.float())
    _close(K.relu_sq_fwd(x), torch.relu(x.float()) ** 2)
    _close(K.relu_sq_bwd(x, p), 2 * torch.relu(x.float()) * p.float())
    w = _bf(100, 256)
    ids = torch.randint(0, 100, (77,), device="cuda", dtype=torch.int32)
    assert torch.equal(K.embedding_fwd(ids, w), w[ids.long()])
    g = _bf(77, 256)
    dw = torch.zeros(100, 256, device="cuda")
    K.embedding_bwd(ids, g, dw)
    ref = torch.zeros(100, 256, device="cuda").index_add_(0, ids.long(), g.float())
    _close(dw, ref, 1e-3)


@pytest.mark.parametrize("V", [1024, 8192, 264])
def test_softcap_ce(V):
    from autoresearch_b200.ops import kernels as K, reference as R
    torch.manual_seed(3)
    rows = 65
    logits = _bf(rows, V, scale=6.0)
    tgt = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
    lf = logits.float().requires_grad_(True)
    ref = R.softcap_ce(lf, tgt, 15.0)
    (ref.sum() * 0.125).backward()
    work = logits.clone()
    loss = K.softcap_ce_(work, tgt, 15.0, 0.125)
    _close(loss, ref, 1e-3, "loss")
    _close(work, lf.grad, 2e-2, "dlogits")
    keep = logits.clone()
    loss2 = K.softcap_ce_(keep, tgt, 15.0, 0.0)
    assert torch.equal(keep, logits)
    _close(loss2, ref, 1e-3)


# 16 heads x 32 gate channels = more (head, channel) pairs than threads in a CTA; 1024 rows take the projection whose
# epilogue does RoPE / QK-norm / value embedding itself, 128 rows the separate kernel
@pytest.mark.parametrize("H,B,T", [(2, 2, 64), (16, 2, 64), (2, 4, 256), (3, 3, 256)])
def test_qkv_post_matches_reference(H, B, T):
    from autoresearch_b200.ops import kernels as K, reference as R, sm100
    torch.manual_seed(4)
    D, V, ch = 128 * H, 50, 32
    assert K.qkv_post_fusable(B * T, 3 * D) == (B * T >= 512)
    N = B * T
    xn = _bf(N, D).requires_grad_(True)
    w = _bf(3 * D, D, scale=0.05).requires_grad_(True)
    ve = _bf(V, D, scale=0.5).requires_grad_(True)
    gw = _bf(H, ch, scale=0.3).requires_grad_(True)
    ids = torch.randint(0, V, (N,), device="cuda", dtype=torch.int32)
    cos, sin = R.rope_tables(T, 128, 200000.0, device="cuda")
    cos, sin = cos.to(torch.bfloat16), sin.to(torch.bfloat16)
    qkv = sm100.AttnPreFn.apply(xn, w, ids, ve, gw, cos, sin, T, H, ch, EPS)
    g = _bf(N, 3 * D)
    qkv.backward(g.clone())
    # reference
    xr, wr, ver, gwr = (t.detach().float().requires_grad_(True) for t in (xn, w, ve, gw))
    raw = xr @ wr.t()
    q = R.rope_qknorm(raw[:, :D].reshape(B, T, H, 128), cos, sin, EPS)
    k = R.rope_qknorm(raw[:, D:2 * D].reshape(B, T, H, 128), cos, sin, EPS)
    gate = xr[:, :ch] @ gwr.t()
    v = R.ve_apply(raw[:, 2 * D:].reshape(B, T, H, 128), ver[ids.long()].view(B, T, H, 128), gate.view(B, T, H))
    ref = torch.cat([q.reshape(N, D), k.reshape(N, D), v.reshape(N, D)], 1)
    _close(qkv, ref, 3e-2, "qkv")
    ref.backward(g.float())
    _close(xn.grad, xr.grad, 4e-2, "d_xn")
    _close(w.grad, wr.grad, 4e-2, "d_w")
    _close(ve.grad, ver.grad, 4e-2, "d_ve")
    _close(gw.grad, gwr.grad, 5e-2, "d_gate_w")


def test_adamw_and_muon_kernels_match_reference():
    from autoresearch_b200.ops.sm100 import OptimKernels
    from autoresearch_b200.optim import muon_adamw as MA
    torch.manual_seed(5)
    ok = OptimKernels()
    n = 4096 + 24
    p0 = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda") * 0.1
    st = dict(master=p0.clone(), m=torch.zeros(n, device="cuda"), v=torch.zeros(n, device="cuda"))
    pv = p0.to(torch.bfloat16)
    rp, rm, rv = p0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    for step in (1, 2, 3):
        ok.adamw_group(st, g, pv, step, 0.01, 0.8, 0.95, 1e-10, 0.01)
        MA.adamw_update(rp, g, rm, rv, step, 0.01, 0.8, 0.95, 1e-10, 0.01)
    _close(st["master"], rp, 1e-4, "adamw")
    _close(pv, rp, 1e-2, "adamw shadow")
    for (G, m, nn) in [(3, 256, 256), (2, 512, 128), (2, 128, 512)]:
        master = torch.randn(G, m, nn, device="cuda") * 0.05
        grad = torch.randn(G, m, nn, device="cuda") * 0.01
        sshape = (G, m, 1) if m >= nn else (G, 1, nn)
        st = dict(master=master.clone(), momentum=torch.zeros_like(master), second=torch.zeros(sshape, device="cuda"))
        pv = master.to(torch.bfloat16)
        rmaster, rmom, rsec = master.clone(), torch.zeros_like(master), torch.zeros(sshape, device="cuda")
        for _ in range(2):
            ok.muon_group(st, grad, pv, 0.9, 0.02, 0.1, 0.95, 5)
            u = MA.muon_nesterov(rmom, grad, 0.9, torch.bfloat16)
            x = MA.newton_schulz(MA.frob_normalise(u), 5)
            MA.cautious_update(rmaster, MA.normuon(x, rsec, 0.95), 0.02, 0.1)
        upd, rupd = st["master"] - master, rmaster - master
        rel = (upd - rupd).norm() / rupd.norm()
        assert rel < 0.05, f"muon update mismatch {rel:.4f} for {(G, m, nn)}"
        _close(st["second"], rsec, 5e-2, "second moment")


def test_muon_step_is_bitwise_reproducible_and_handles_ragged_shapes():
    """The Frobenius norm is summed in a fixed order (no atomics), so two runs of a Muon step from the same state
    give the same bits; a matrix whose column count is not a multiple of 8 takes the scalar kernels."""
    from autoresearch_b200.ops.sm100 import OptimKernels
    from autoresearch_b200.optim import muon_adamw as MA
    torch.manual_seed(11)
    ok = OptimKernels()
    for (G, m, nn) in [(5, 512, 256), (2, 192, 1024), (3, 256, 264)]:
        master = torch.randn(G, m, nn, device="cuda") * 0.05
        grad = torch.randn(G, m, nn, device="cuda") * 0.01
        sshape = (G, m, 1) if m >= nn else (G, 1, nn)
        outs = []
        for _ in range(2):
            st = dict(master=master.clone(), momentum=torch.zeros_like(master), second=torch.zeros(sshape, device="cuda"))
            pv = master.to(torch.bfloat16)
            for _ in range(2):
                ok.muon_group(st, grad, pv, 0.9, 0.02, 0.1, 0.95, 5)
            outs.append((st["master"].clone(), st["momentum"].clone(), pv.clone()))
        for a, b in zip(*outs):
            assert torch.equal(a, b)
        rmaster, rmom, rsec = master.clone(), torch.zeros_like(master), torch.zeros(sshape, device="cuda")
        for _ in range(2):
            u = MA.muon_nesterov(rmom, grad, 0.9, torch.bfloat16)
            MA.cautious_update(rmaster, MA.normuon(MA.newton_schulz(MA.frob_normalise(u), 5), rsec, 0.95), 0.02, 0.1)
        upd, rupd = outs[0][0] - master, rmaster - master
        assert (upd - rupd).norm() / rupd.norm() < 0.05
    assert ok.scratch_bytes() > 0


def test_embedding_backward_sorted_is_exact_and_deterministic():
    """The sorted, atomic-free embedding gradient: equal to an fp64 index_add within fp32 rounding, bitwise
    reproducible, also with ids that fill many 64-row work items and ids that never occur."""
    from autoresearch_b200.ops import kernels as K
    torch.manual_seed(11)
    N, D, vocab = 20000, 256, 1000
    ids = (torch.rand(N, device="cuda") ** 6 * vocab).long().clamp(0, vocab - 1).to(torch.int32)
    ids[ids == 7] = 8                                          # id 7 never occurs
    g = torch.randn(N, D, device="cuda").to(torch.bfloat16)
    outs = []
    for _ in range(2):
        dw = torch.full((vocab, D), 0.5, dtype=torch.float32, device="cuda")
        K.embedding_bwd(ids, g, dw)
        outs.append(dw.clone())
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])
    ref = torch.full((vocab, D), 0.5, dtype=torch.float64, device="cuda").index_add_(0, ids.long(), g.double())
    assert (outs[0].double() - ref).abs().max().item() < 2e-3
    assert torch.equal(outs[0][7], torch.full((D,), 0.5, device="cuda"))
    counts = torch.bincount(ids.long(), minlength=vocab)
    assert counts.max().item() > 5 * K.EMB_BWD_ROWS_PER_ITEM         # the multi-item path was exercised
    # the atomic variant gives the same numbers up to summation order
    K.EMB_BWD_DETERMINISTIC = False
    try:
        dw2 = torch.full((vocab, D), 0.5, dtype=torch.float32, device="cuda")
        K.embedding_bwd(ids, g, dw2)
    finally:
        K.EMB_BWD_DETERMINISTIC = True
    assert (dw2 - outs[0]).abs().max().item() < 2e-3


def test_bounded_device_wait_expires_into_the_error_word_and_the_context_stays_usable():
    """A peer barrier whose partner never arrives (a flag that nothing sets): the kernel gives up after its wait
    limit, returns normally and leaves ERR_COMM_TIMEOUT in the status word; the next kernels run as usual."""
    import ctypes as C
    import time
    from autoresearch_b200.ops import kernels as K
    K.check_err_flag()
    mine = torch.zeros(64, dtype=torch.int32, device="cuda")
    absent_peer = torch.zeros(64, dtype=torch.int32, device="cuda")       # stands in for a rank that never shows up
    ptrs = (C.c_void_p * 2)(mine.data_ptr(), absent_peer.data_ptr())
    t0 = time.time()
    rc = K.lib().arb_peer_barrier(ptrs, 2, 0, 1, K.err_flag().data_ptr(), K._stream())
    assert rc == 0
    torch.cuda.synchronize()                                              # returns: the wait is bounded (2 s of device time)
    assert 1.0 < time.time() - t0 < 20.0
    assert int(absent_peer[0].item()) == 1                                # this rank did announce itself
    with pytest.raises(K.KernelError, match="peer barrier wait timed out"):
        K.check_err_flag()
    K.check_err_flag()                                                    # the word was cleared by the read above
    x = _bf(64, 512)
    _close(K.rmsnorm_fwd(x, EPS), torch.nn.functional.rms_norm(x.float(), (512,), eps=EPS))
    torch.cuda.synchronize()
    K.check_err_flag()


def test_kernels_are_bitwise_reproducible_and_stay_inside_their_outputs():
    """Run twice -> identical bits (no atomics on these paths), and canary rows around the outputs stay untouched."""
    from autoresearch_b200.ops import kernels as K, sm100
    torch.manual_seed(21)
    # GEMM into the middle of a larger buffer
    a, w = _bf(300, 256), _bf(200, 256)
    buf = torch.full((300 + 16, 200), 7.0, device="cuda", dtype=torch.bfloat16)
    outs = []
    for _ in range(2):
        buf.fill_(7.0)
        K.gemm(a, w, out=buf[8:308])
        outs.append(buf.clone())
    assert torch.equal(outs[0], outs[1])
    assert torch.all(outs[0][:8] == 7.0) and torch.all(outs[0][308:] == 7.0)
    # attention forward + backward (deterministic two-kernel backward)
    B, T, H = 1, 640, 2
    qkv = _bf(B * T, 3 * H * 128).requires_grad_(True)
    g = _bf(B * T, H * 128)
    res = []
    for _ in range(2):
        out = sm100.AttentionFn.apply(qkv, B, T, H, 200)
        out.backward(g)
        res.append((out.detach().clone(), qkv.grad.clone()))
        qkv.grad = None
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
    # fused norm kernels next to canaries
    x = _bf(37, 1024)
    y1, y2 = K.rmsnorm_fwd(x, EPS), K.rmsnorm_fwd(x, EPS)
    assert torch.equal(y1, y2)
    torch.cuda.synchronize()
    K.check_err_flag()
