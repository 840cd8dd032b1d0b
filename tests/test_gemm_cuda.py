"""The 3xTF32 tcgen05 GEMM against fp64 (and the fp32 FMA kernel against the same oracle)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(actual, expected):
    return float((actual.double() - expected).norm() / expected.norm())


def _operands(K, M, N, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(K, M, generator=g)
    b = torch.randn(K, N, generator=g)
    return a, b


SHAPES = [(32, 128, 128), (64, 128, 256), (200, 130, 70), (8, 8, 8), (33, 1, 5), (512, 384, 640),
          (1000, 257, 300), (4096, 256, 512)]


@pytest.mark.parametrize("K,M,N", SHAPES)
@pytest.mark.parametrize("narrow", [False, True])
def test_store_matches_fp64(K, M, N, narrow):
    from soap_tp_b200.engine import kernels as k

    a, b = _operands(K, M, N, 1)
    expected = a.double().T @ b.double()
    ap, bp = k.split_planes(a.cuda()), k.split_planes(b.cuda())
    torch.testing.assert_close(ap.dense().cpu(), a, rtol=0, atol=0)
    backing = torch.full((N + 1, M + 3), 7.0, device="cuda")
    out = backing.T[:M, :N]  # column-major, padded pitch
    k.gemm(ap, bp, out=out, force_narrow=narrow)
    k.check_status()
    assert _rel(out.cpu(), expected) < 2e-6, _rel(out.cpu(), expected)
    assert bool((backing[:, M:] == 7.0).all()) and bool((backing[N:, :] == 7.0).all())  # padding untouched
    ref = torch.empty(M, N, device="cuda")
    k.gemm_simt(a.cuda(), b.cuda(), ref)
    assert _rel(ref.cpu(), expected) < 2e-6


def test_large_and_wide_tiles():
    from soap_tp_b200.engine import kernels as k

    a, b = _operands(1024, 2560, 2048, 2)      # 20 x 8 wide tiles >= 148 -> BN = 256 path
    expected = a.double().T @ b.double()
    out = torch.empty(2048, 2560, device="cuda").T
    k.gemm(k.split_planes(a.cuda()), k.split_planes(b.cuda()), out=out)
    k.check_status()
    assert _rel(out.cpu(), expected) < 2e-6


def test_transposed_split_and_row_major_store():
    from soap_tp_b200.engine import kernels as k

    a, b = _operands(300, 200, 150, 3)
    ap = k.split_planes(a.T.contiguous().cuda(), transpose=True)   # source is M x K row-major
    torch.testing.assert_close(ap.dense().cpu(), a, rtol=0, atol=0)
    out = torch.empty(200, 150, device="cuda")
    k.gemm(ap, k.split_planes(b.cuda()), mode=k.EPI_ROW_MAJOR, out=out, alpha=0.5)
    k.check_status()
    assert _rel(out.cpu(), 0.5 * (a.double().T @ b.double())) < 2e-6


def test_ema_and_symmetric_mirror():
    from soap_tp_b200.engine import kernels as k

    g = torch.Generator().manual_seed(4)
    a = torch.randn(500, 700, generator=g)
    old = torch.randn(700, 700, generator=g)
    old = old + old.T
    expected = 0.9 * old.double() + 0.1 * (a.double().T @ a.double())
    ap = k.split_planes(a.cuda())
    for symmetric in (False, True):
        out = old.cuda().T.contiguous().T
        k.gemm(ap, ap, out=out, alpha=0.1, beta=0.9, symmetric=symmetric)
        k.check_status()
        assert _rel(out.cpu(), expected) < 2e-6
        if symmetric:
            assert torch.equal(out, out.T)


def test_split_epilogue_chain_and_adam():
    from soap_tp_b200.engine import kernels as k

    g = torch.Generator().manual_seed(5)
    x = torch.randn(256, 192, generator=g)
    q = torch.randn(256, 256, generator=g)
    r = torch.randn(192, 192, generator=g)
    xp, qp, rp = (k.split_planes(t.cuda()) for t in (x, q, r))
    t_planes = k.Planes.empty(192, 256, "cuda")
    k.gemm(xp, qp, mode=k.EPI_SPLIT, out_planes=t_planes)        # T = X^T Q  (192 x 256)
    k.check_status()
    expected_t = x.double().T @ q.double()
    assert _rel(t_planes.dense().cpu(), expected_t) < 2e-6
    m = torch.randn(192, 256, generator=g).T.contiguous().T.cuda()
    v = torch.rand(192, 256, generator=g).T.contiguous().T.cuda()
    m0, v0 = m.clone(), v.clone()
    y_planes = k.Planes.empty(256, 192, "cuda")
    proj = torch.empty(192, 256, device="cuda").T
    adam = dict(beta1=0.9, beta2=0.99, eps=1e-6, bias_correction1=1 - 0.9**3, bias_correction2=1 - 0.99**3)
    mt = torch.zeros(192, 256, device="cuda").T  # 256 x 192 column-major
    vt = torch.zeros(192, 256, device="cuda").T
    mt.copy_(m0.T); vt.copy_(v0.T)
    k.gemm(t_planes, rp, mode=k.EPI_ADAM, out_planes=y_planes, out=proj, momentum=mt, variance=vt, adam=adam)
    k.check_status()
    y = expected_t.T @ r.double()                                # (Q^T X) R : 256 x 192
    em = 0.9 * m0.T.cpu().double() + 0.1 * y
    ev = 0.99 * v0.T.cpu().double() + 0.01 * y * y
    eu = (em / adam["bias_correction1"]) / (ev.sqrt() / adam["bias_correction2"] ** 0.5 + 1e-6)
    assert _rel(mt.cpu(), em) < 2e-6 and _rel(vt.cpu(), ev) < 6e-6
    assert _rel(y_planes.dense().cpu(), eu) < 1e-5
    assert _rel(proj.cpu(), eu) < 1e-5          # plain copy of the update


MIXED_SHAPES = [(32, 128, 128), (64, 128, 256), (200, 130, 70), (40, 8, 8), (512, 384, 640), (1000, 257, 300),
                (4096, 256, 512), (8192, 512, 512)]


@pytest.mark.parametrize("K,M,N", MIXED_SHAPES)
def test_mixed_corrections_match_fp64(K, M, N):
    """The accuracy gate of the mixed form (correction products as bf16 MMAs): still fp32-class against fp64,
    within a factor of the three-tf32-MMA form, at every depth up to the benchmark's 8192."""
    from soap_tp_b200.engine import kernels as k

    a, b = _operands(K, M, N, 11)
    expected = a.double().T @ b.double()
    classic = torch.empty(N, M, device="cuda").T
    k.gemm(k.split_planes(a.cuda()), k.split_planes(b.cuda()), out=classic)
    am, bm = k.split_planes(a.cuda(), mixed=True), k.split_planes(b.cuda(), mixed=True)
    assert am.mixed and am.lo is None
    assert float((am.dense().cpu() - a).abs().max()) <= 2.0 ** -18 * float(a.abs().max())     # hi + bf16(lo)
    mixed = torch.empty(N, M, device="cuda").T
    k.gemm(am, bm, out=mixed)
    k.check_status()
    error_classic, error_mixed = _rel(classic.cpu(), expected), _rel(mixed.cpu(), expected)
    print(f"K={K}: 3xTF32 {error_classic:.2e}, tf32 + 2 bf16 corrections {error_mixed:.2e}")
    assert error_mixed < 2e-6, error_mixed
    assert error_mixed < 8 * max(error_classic, 1e-7)


def test_mixed_output_planes_and_adam_epilogue():
    """Epilogues that write the operand of the next product in the mixed form: split, and Adam in the eigenbasis."""
    from soap_tp_b200.engine import kernels as k

    K, M, N = 256, 384, 200
    a, b = _operands(K, M, N, 12)
    expected = a.double().T @ b.double()
    am, bm = k.split_planes(a.cuda(), mixed=True), k.split_planes(b.cuda(), mixed=True)
    out_planes = k.Planes.empty(M, N, "cuda", mixed=True)
    plain = torch.empty(N, M, device="cuda").T
    k.gemm(am, bm, mode=k.EPI_SPLIT, out_planes=out_planes, out=plain)
    assert _rel(plain.cpu(), expected) < 2e-6
    assert _rel(out_planes.dense().cpu(), expected) < 1e-5                     # hi + bf16(lo)
    assert _rel(out_planes.halves()[0].T.cpu(), expected) < 5e-3               # bf16(value)
    # chained: the mixed planes are the operand of the next product
    c = torch.randn(M, 96, generator=torch.Generator().manual_seed(13))
    chained = torch.empty(96, N, device="cuda").T
    k.gemm(out_planes, k.split_planes(c.cuda(), mixed=True), out=chained)
    assert _rel(chained.cpu(), expected.T @ c.double()) < 3e-6
    # Adam epilogue, update as mixed planes
    momentum, variance = torch.zeros(N, M, device="cuda").T, torch.zeros(N, M, device="cuda").T
    adam = dict(beta1=0.9, beta2=0.99, eps=1e-8, bias_correction1=0.1, bias_correction2=0.01)
    update = k.Planes.empty(M, N, "cuda", mixed=True)
    k.gemm(am, bm, mode=k.EPI_ADAM, out_planes=update, momentum=momentum, variance=variance, adam=adam)
    k.check_status()
    m = 0.1 * expected
    v = 0.01 * expected * expected
    want = (m / 0.1) / (v.sqrt() / 0.1 + 1e-8)
    assert _rel(momentum.cpu(), m) < 2e-6
    assert _rel(update.dense().cpu(), want) < 1e-4
    with pytest.raises(ValueError, match="both operands"):
        k.gemm(am, k.split_planes(b.cuda()), out=plain)
