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
