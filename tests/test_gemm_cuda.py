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


@pytest.fixture
def single_cta_reference():
    """Runs a product once on CTA pairs (the default for large problems) and once on single CTAs."""
    from soap_tp_b200.engine import kernels as k

    def both(run):
        results = []
        for pairs in (True, False):
            k.use_cta_pairs(pairs)
            try:
                results.append(run())
            finally:
                k.use_cta_pairs(True)
        return results

    return both


@pytest.mark.parametrize("mixed", [False, True])
@pytest.mark.parametrize("K,M,N", [(1024, 2560, 2048), (520, 2500, 2100), (96, 4096, 2304)])
def test_cta_pairs_store(K, M, N, mixed, single_cta_reference):
    """256 x 256 tiles on CTA pairs (cta_group::2): ragged edges, padded pitch, EMA form, against fp64 and against the
    single-CTA kernel (same MMA order and promotion cadence, hence the same bits)."""
    from soap_tp_b200.engine import kernels as k

    a, b = _operands(K, M, N, 21)
    old = torch.randn(N + 1, M + 4, generator=torch.Generator().manual_seed(22))
    expected = 0.25 * (a.double().T @ b.double()) + 0.5 * old.T[:M, :N].double()
    ap, bp = k.split_planes(a.cuda(), mixed=mixed), k.split_planes(b.cuda(), mixed=mixed)

    def run():
        backing = old.cuda()
        out = backing.T[:M, :N]
        k.gemm(ap, bp, out=out, alpha=0.25, beta=0.5)
        k.check_status()
        assert torch.equal(backing[:, M:].cpu(), old[:, M:]) and torch.equal(backing[N:, :].cpu(), old[N:, :])
        return out.cpu()

    pair, single = single_cta_reference(run)
    assert _rel(pair, expected) < 2e-6, _rel(pair, expected)
    assert torch.equal(pair, single)


def test_cta_pairs_symmetric_and_row_major(single_cta_reference):
    from soap_tp_b200.engine import kernels as k

    g = torch.Generator().manual_seed(23)
    a = torch.randn(300, 2600, generator=g)
    old = torch.randn(2600, 2600, generator=g)
    old = old + old.T
    expected = 0.9 * old.double() + 0.1 * (a.double().T @ a.double())
    ap = k.split_planes(a.cuda())

    def symmetric():
        out = old.cuda().T.contiguous().T
        k.gemm(ap, ap, out=out, alpha=0.1, beta=0.9, symmetric=True)
        k.check_status()
        assert torch.equal(out, out.T)
        return out.cpu()

    pair, single = single_cta_reference(symmetric)
    assert _rel(pair, expected) < 2e-6
    assert torch.equal(pair, single)
    b = torch.randn(300, 2304, generator=g)
    bp = k.split_planes(b.cuda())

    def row_major():
        out = torch.empty(2600, 2304, device="cuda")
        k.gemm(ap, bp, mode=k.EPI_ROW_MAJOR, out=out, alpha=0.5)
        k.check_status()
        return out.cpu()

    pair, single = single_cta_reference(row_major)
    assert _rel(pair, 0.5 * (a.double().T @ b.double())) < 2e-6
    assert torch.equal(pair, single)


@pytest.mark.parametrize("mixed", [False, True])
def test_cta_pairs_split_and_adam_epilogues(mixed, single_cta_reference):
    """The rotation chain of the optimizer step at a size that runs on CTA pairs: T = X^T Q written as operand planes,
    then Adam in the eigenbasis fused into (Q^T X) R."""
    from soap_tp_b200.engine import kernels as k

    g = torch.Generator().manual_seed(24)
    rows, cols = 2560, 2304
    x = torch.randn(rows, cols, generator=g)
    q = torch.randn(rows, rows, generator=g) / rows ** 0.5
    r = torch.randn(cols, cols, generator=g) / cols ** 0.5
    xp, qp, rp = (k.split_planes(t.cuda(), mixed=mixed) for t in (x, q, r))
    m0 = torch.randn(cols, rows, generator=g)
    v0 = torch.rand(cols, rows, generator=g)
    adam = dict(beta1=0.9, beta2=0.99, eps=1e-6, bias_correction1=1 - 0.9**3, bias_correction2=1 - 0.99**3)

    def run():
        t_planes = k.Planes.empty(cols, rows, "cuda", mixed=mixed)
        k.gemm(xp, qp, mode=k.EPI_SPLIT, out_planes=t_planes)            # T = X^T Q  (cols x rows)
        y_planes = k.Planes.empty(rows, cols, "cuda", mixed=mixed)
        mt, vt = m0.cuda().T, v0.cuda().T                                # rows x cols, column-major
        k.gemm(t_planes, rp, mode=k.EPI_ADAM, out_planes=y_planes, momentum=mt, variance=vt, adam=adam)
        k.check_status()
        return t_planes.dense().cpu(), y_planes.dense().cpu(), mt.cpu(), vt.cpu()

    pair, single = single_cta_reference(run)
    expected_t = x.double().T @ q.double()
    y = expected_t.T @ r.double()
    em = 0.9 * m0.T.double() + 0.1 * y
    ev = 0.99 * v0.T.double() + 0.01 * y * y
    eu = (em / adam["bias_correction1"]) / (ev.sqrt() / adam["bias_correction2"] ** 0.5 + 1e-6)
    assert _rel(pair[0], expected_t) < (1e-5 if mixed else 2e-6)
    assert _rel(pair[2], em) < 2e-6 and _rel(pair[3], ev) < 6e-6
    assert _rel(pair[1], eu) < 1e-5
    for got, want in zip(pair, single):
        assert torch.equal(got, want)


@pytest.mark.parametrize("mixed", [False, True])
@pytest.mark.parametrize("I,J,nb,grid,K", [(300, 260, 4, (2, 2), 96), (2560, 2304, 128, (2, 2), 200), (520, 390, 64, (2, 4), 64),
                                           (384, 384, 128, (1, 2), 40)])
def test_push_epilogue_fills_the_consumers_planes(I, J, nb, grid, K, mixed):
    """GEMM -> all-gather in the epilogue: every rank of a grid (run one after the other on this GPU) computes its
    block of the block-cyclic matrix T = A^T B and stores it, as operand planes, into the gathered operand
    T[:, row class] of the ranks of the consuming grid row; afterwards every rank's planes hold exactly that."""
    from soap_tp_b200.engine import kernels as k
    from soap_tp_b200.layout import owned_indices

    Pr, Pc = grid
    a, b = _operands(K, I, J, 31)
    expected = (a.double().T @ b.double())                       # T, I x J
    most = max(len(owned_indices(J, nb, p, Pr)) for p in range(Pr))
    ld, ld16 = max(4, k.round_up(I, 4)), 2 * k.round_up(I, 32)
    targets, entries = [], []
    for rank in range(Pr * Pc):
        hi = torch.full((most, ld), float("nan"), device="cuda")
        low = torch.zeros((most, ld16), dtype=torch.bfloat16, device="cuda") if mixed else torch.full((most, ld), float("nan"), device="cuda")
        targets.append((hi, low))
        entries += [hi.data_ptr(), low.data_ptr()]
    table = torch.tensor(entries, dtype=torch.int64, device="cuda")
    for pr in range(Pr):
        for pc in range(Pc):
            rows, cols = owned_indices(I, nb, pr, Pr), owned_indices(J, nb, pc, Pc)
            if not (len(rows) and len(cols)):
                continue
            ap = k.split_planes(a[:, rows].contiguous().cuda(), mixed=mixed)
            bp = k.split_planes(b[:, cols].contiguous().cuda(), mixed=mixed)
            k.gemm(ap, bp, mode=k.EPI_PUSH, push=dict(table=table, ld=ld, ld16=ld16, nb=nb, Pr=Pr, Pc=Pc, pr=pr, pc=pc,
                                                        mixed=mixed))
    k.check_status()
    for pr in range(Pr):
        wanted = owned_indices(J, nb, pr, Pr)
        for pc in range(Pc):
            hi, low = targets[pr * Pc + pc]
            planes = k.Planes(hi, None, I, len(wanted), ld, low, ld16) if mixed else k.Planes(hi, low, I, len(wanted), ld)
            got = planes.dense().cpu()                            # I x len(wanted)
            assert _rel(got, expected[:, wanted]) < (1e-5 if mixed else 2e-6), (pr, pc)
