"""tcgen05 GEMM against a plain fp32 PyTorch matmul of the same bf16 operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=[1, 2, 0], ids=["one_cta", "cta_pair", "auto"])
def tile_mode(request):
    """Every case runs on the 1-CTA kernel, on the 2-CTA (cta_group::2) kernel and with the
    automatic choice."""
    from autoresearch_b200.ops import kernels as K_
    K_.gemm_set_mode(request.param)
    yield request.param
    K_.gemm_set_mode(0)


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _close(out, ref, tol=2e-2):
    err = (out.float() - ref).abs().max().item()
    den = ref.abs().max().item() + 1e-6
    assert err / den < tol, f"rel err {err / den:.4g}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 128, 192), (200, 328, 136),
                                   (1024, 1024, 1024), (129, 72, 520)])
def test_nt(M, N, K):
    from autoresearch_b200.ops import kernels as K_
    torch.manual_seed(0)
    a, b = _rand(M, K), _rand(N, K)
    out = K_.gemm(a, b)
    _close(out, a.float() @ b.float().t())
    K_.check_err_flag()


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (200, 328, 136), (512, 1024, 768)])
def test_nn(M, N, K):
    from autoresearch_b200.ops import kernels as K_
    torch.manual_seed(1)
    a, b = _rand(M, K), _rand(K, N)
    out = K_.gemm(a, b, trans_b=False)
    _close(out, a.float() @ b.float())


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (264, 136, 1000), (1024, 512, 4096)])
def test_tn_atomic_accumulate(M, N, K):
    from autoresearch_b200.ops import kernels as K_
    torch.manual_seed(2)
    a, b = _rand(K, M), _rand(K, N)
    acc = torch.randn(M, N, device="cuda")
    ref = acc.clone() + a.float().t() @ b.float()
    K_.gemm(a, b, trans_a=True, trans_b=False, out=acc, epi=K_.EPI_ATOMIC_F32)
    _close(acc, ref, 1e-2)
    # explicit split-K
    acc2 = torch.zeros(M, N, device="cuda")
    K_.gemm(a, b, trans_a=True, trans_b=False, out=acc2, epi=K_.EPI_ATOMIC_F32, splitk=3)
    _close(acc2, a.float().t() @ b.float(), 1e-2)


def test_tn_nt_mixed_and_f32_store():
    from autoresearch_b200.ops import kernels as K_
    torch.manual_seed(3)
    a, b = _rand(320, 192), _rand(256, 320)      # A = a^T [192, 320], B = b^T
    out = K_.gemm(a, b, trans_a=True, trans_b=True, epi=K_.EPI_STORE_F32)
    _close(out, a.float().t() @ b.float().t(), 1e-2)


def test_epilogues():
    from autoresearch_b200.ops import kernels as K_
    torch.manual_seed(4)
    M, N, Kd = 256, 384, 128
    a, b = _rand(M, Kd, scale=0.3), _rand(N, Kd, scale=0.3)
    ref = a.float() @ b.float().t()
    _close(K_.gemm(a, b, epi=K_.EPI_RELU2), torch.relu(ref) ** 2)
    aux = _rand(M, N)
    _close(K_.gemm(a, b, epi=K_.EPI_ADD_AUX, aux=aux), ref + aux.float())
    act = (torch.relu(aux.float()) ** 2).to(torch.bfloat16)
    _close(K_.gemm(a, b, epi=K_.EPI_RELU2_BWD, aux=act), ref * 2 * torch.sqrt(act.float()))
    sq = _rand(256, 256, scale=0.1)
    got = K_.gemm(sq, sq, epi=K_.EPI_NS_COMBINE, aux=sq, alpha=1.5, beta=-2.0, gamma=0.5)
    want = 1.5 * torch.eye(256, device="cuda") - 2.0 * sq.float() + 0.5 * (sq.float() @ sq.float().t())
    _close(got, want)


def test_batched():
    from autoresearch_b200.ops import kernels as K_
    torch.manual_seed(5)
    G, m, n = 5, 256, 512
    x = _rand(G, m, n, scale=0.2)
    A = K_.gemm(x, x)                                        # X X^T
    _close(A, x.float() @ x.float().transpose(1, 2))
    At = K_.gemm(x, x, trans_a=True, trans_b=False)          # X^T X
    _close(At, x.float().transpose(1, 2) @ x.float())
    y = K_.gemm(A, x, trans_b=False)                         # A X
    _close(y, A.float() @ x.float())


def test_strided_views():
    """Operands that are column blocks of a wider buffer (packed qkv) and row slices."""
    from autoresearch_b200.ops import kernels as K_
    torch.manual_seed(6)
    big = _rand(512, 768)
    w = _rand(256, 256)
    a = big[:, 256:512]
    _close(K_.gemm(a, w), a.float() @ w.float().t())
    out = torch.zeros(512, 512, dtype=torch.bfloat16, device="cuda")
    K_.gemm(a, w, out=out[:, 256:])
    _close(out[:, 256:], a.float() @ w.float().t())
    assert out[:, :256].abs().max().item() == 0


def test_rejects_bad_arguments():
    from autoresearch_b200.ops import kernels as K_
    a, b = _rand(128, 60), _rand(128, 60)      # K not a multiple of 8
    with pytest.raises(K_.KernelError):
        K_.gemm(a, b)


@pytest.mark.parametrize("shape", [(1024, 512, 256), (192, 128, 64), (4096, 3072, 1024)])
def test_gemm_pulls_its_b_operand_in_the_prologue(shape):
    """A registered pending pull makes the GEMM copy its B operand from another buffer first (the mechanism
    that fuses the parameter all-gather into the first consuming GEMM); here the source is local memory."""
    from autoresearch_b200.ops import kernels as K
    M, N, Kd = shape
    torch.manual_seed(3)
    x = torch.randn(M, Kd, device="cuda").to(torch.bfloat16)
    w_new = (torch.randn(N, Kd, device="cuda") * 0.05).to(torch.bfloat16)
    w = torch.zeros_like(w_new)                       # stale local copy
    K.pending_pulls[w.data_ptr()] = (w_new.data_ptr(), w.numel() * 2)
    for _ in range(3):                                # the counter barrier must work launch after launch
        y = K.gemm(x, w)
        torch.cuda.synchronize()
        K.check_err_flag()
        assert w.data_ptr() not in K.pending_pulls
        assert torch.equal(w, w_new)
        ref = x.float() @ w_new.float().t()
        assert ((y.float() - ref).norm() / ref.norm()).item() < 1e-2
        w.zero_()
        K.pending_pulls[w.data_ptr()] = (w_new.data_ptr(), w.numel() * 2)
    K.flush_pending_pulls()
    torch.cuda.synchronize()
    assert torch.equal(w, w_new) and not K.pending_pulls


@pytest.mark.parametrize("shape", [(1024, 512, 256), (4096, 3072, 1024)])
def test_gemm_copies_the_next_operand_while_it_computes(shape):
    """With two operands pending, the first GEMM copies its own B in the prologue and, in a spare warp, the
    OTHER pending operand while its tiles run; the second GEMM then finds its operand local already."""
    from autoresearch_b200.ops import kernels as K
    M, N, Kd = shape
    torch.manual_seed(4)
    x = torch.randn(M, Kd, device="cuda").to(torch.bfloat16)
    new = [(torch.randn(N, Kd, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(2)]
    # the second operand's size is not a multiple of the copy loop's stride: exercises its tail
    new.append((torch.randn(N + 8, Kd, device="cuda") * 0.05).to(torch.bfloat16))
    stale = [torch.zeros_like(w) for w in new]
    K.pending_pulls.clear()
    for s, w in zip(stale, new):
        K.pending_pulls[s.data_ptr()] = (w.data_ptr(), w.numel() * 2)
    K.pull_stream = K._stream()
    y0 = K.gemm(x, stale[0])
    assert len(K.pending_pulls) == 1                  # own operand + one ahead
    torch.cuda.synchronize()
    assert torch.equal(stale[0], new[0]) and torch.equal(stale[1], new[1]) and stale[2].abs().max().item() == 0
    y1 = K.gemm(x, stale[1])                          # nothing pending for it; copies operand 2 ahead
    assert not K.pending_pulls
    y2 = K.gemm(x, stale[2])
    torch.cuda.synchronize()
    K.check_err_flag()
    assert torch.equal(stale[2], new[2])
    for y, w in zip((y0, y1, y2), new):
        ref = x.float() @ w.float().t()
        assert ((y.float() - ref).norm() / ref.norm()).item() < 1e-2
    # a GEMM on another stream leaves the ahead copies to the stream they were registered on
    stale[1].zero_()
    K.pending_pulls[stale[1].data_ptr()] = (new[1].data_ptr(), new[1].numel() * 2)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        K.gemm(x, stale[0])
    assert len(K.pending_pulls) == 1
    K.flush_pending_pulls()
    torch.cuda.synchronize()
    assert torch.equal(stale[1], new[1])


@pytest.mark.parametrize("mode", [1, 2])
def test_ragged_batches_skip_rows_beyond_the_valid_count(mode):
    """Grouped expert GEMM: per-item row counts (device array), several row slabs per weight matrix; tiles beyond the
    count are left untouched and the K range of the transposed product is cut to the valid rows."""
    from autoresearch_b200.ops import kernels as K
    torch.manual_seed(7)
    E, W, cap, D, M = 2, 3, 640, 256, 512          # E weights, W slabs each, cap rows per slab
    G = E * W
    counts = torch.tensor([640, 0, 130, 257, 512, 5], dtype=torch.int32, device="cuda")
    x = (torch.randn(G, cap, D, device="cuda") * 0.5).to(torch.bfloat16)
    for g in range(G):                               # rows between the count and the next tile boundary are zero
        x[g, int(counts[g]):] = 0
    w = (torch.randn(E, M, D, device="cuda") * 0.1).to(torch.bfloat16)
    K.gemm_set_mode(mode)
    try:
        out = torch.full((G, cap, M), 7.0, dtype=torch.bfloat16, device="cuda")
        K.gemm(x, w, out=out, epi=K.EPI_RELU2, m_valid=counts, b_div=W)
        tile = 256 if mode == 2 else 128
        for g in range(G):
            c = int(counts[g])
            ref = torch.relu(x[g, :c].float() @ w[g // W].float().t()) ** 2
            if c:
                assert ((out[g, :c].float() - ref).norm() / ref.norm()).item() < 1e-2
            done = (c + tile - 1) // tile * tile
            assert (out[g, min(done, cap):] == 7.0).all()           # untouched
            assert (out[g, c:min(done, cap)] == 0).all()            # computed from zero rows
        # dW[e] += sum over the slabs of e of dy^T x, K cut to the valid rows; poison what lies beyond the padding
        dy = (torch.randn(G, cap, M, device="cuda") * 0.1).to(torch.bfloat16)
        for g in range(G):
            c = int(counts[g])
            dy[g, c:] = 0
            pad = (c + 63) // 64 * 64
            dy[g, pad:] = float("nan")
            x[g, pad:] = float("nan")
        dw = torch.zeros(E, M, D, dtype=torch.float32, device="cuda")
        K.gemm(dy.view(E, W * cap, M), x.view(E, W * cap, D), trans_a=True, trans_b=False, out=dw, epi=K.EPI_ATOMIC_F32,
               k_valid=counts.view(E, W).contiguous(), k_seg=cap)
        torch.cuda.synchronize()
        K.check_err_flag()
        for e in range(E):
            ref = sum(dy[e * W + j, :int(counts[e * W + j])].float().t() @ x[e * W + j, :int(counts[e * W + j])].float()
                      for j in range(W))
            assert torch.isfinite(dw[e]).all()
            assert ((dw[e] - ref).norm() / ref.norm()).item() < 1e-2
    finally:
        K.gemm_set_mode(0)
