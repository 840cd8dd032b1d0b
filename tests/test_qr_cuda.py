"""Blocked Householder QR on the GPU against its defining properties (fp64 checks).

The reference tests its QR binding on sizes 8 to 13 against ``numpy.linalg.qr``
(``tests/unit/test_slate_bindings.py:244-323``); here the factorisation kernel chain itself is exercised on sizes that
span several panels, ragged last panels, a rank-deficient input, and the concurrent two-job driver.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(matrix: torch.Tensor, Q: torch.Tensor, tolerance: float) -> None:
    a, q = matrix.double(), Q.double()         # float64 products on the device
    n = a.shape[0]
    orthogonality = float((q.T @ q - torch.eye(n, dtype=torch.float64, device=a.device)).abs().max())
    r = q.T @ a
    below = float(torch.tril(r, -1).norm() / a.norm().clamp_min(1e-30))
    assert orthogonality < tolerance, f"|Q^T Q - I|_max = {orthogonality}"
    assert below < tolerance, f"|tril(Q^T A)| / |A| = {below}"


@pytest.mark.parametrize("n", [128, 200, 384, 1000, 2048, 8192])
def test_householder_qr_properties(n):
    from soap_tp_b200.engine import kernels as k
    from soap_tp_b200.engine import qr

    device = torch.device("cuda", 0)
    generator = torch.Generator(device=device).manual_seed(n)
    matrix = torch.randn(n, n, generator=generator, device=device).T
    Q = torch.empty(n, n, device=device).T
    qr.householder_qr(matrix, Q)
    k.check_status()
    _check(matrix, Q, 2e-5)


def test_rank_deficient_and_column_order():
    from soap_tp_b200.engine import kernels as k
    from soap_tp_b200.engine import qr

    device = torch.device("cuda", 0)
    generator = torch.Generator(device=device).manual_seed(7)
    n, rank = 512, 100
    left = torch.randn(n, rank, generator=generator, device=device)
    matrix = (left @ torch.randn(rank, n, generator=generator, device=device)).T.contiguous().T
    order = torch.randperm(n, generator=generator, device=device)
    Q = torch.empty(n, n, device=device).T
    qr.householder_qr(matrix, Q, order)
    k.check_status()
    _check(matrix[:, order], Q, 5e-5)


def test_pair_driver_matches_single_jobs():
    from soap_tp_b200.engine import kernels as k
    from soap_tp_b200.engine import qr

    device = torch.device("cuda", 0)
    generator = torch.Generator(device=device).manual_seed(11)
    sizes = (640, 896)
    jobs = []
    for n in sizes:
        jobs.append((torch.randn(n, n, generator=generator, device=device).T, torch.empty(n, n, device=device).T, None))
    qr.householder_qr_pair(jobs)
    torch.cuda.synchronize()
    k.check_status()
    for matrix, Q, _ in jobs:
        _check(matrix, Q, 2e-5)
        single = torch.empty_like(Q)
        qr.householder_qr(matrix, single)
        assert float((single - Q).abs().max()) < 1e-4


@pytest.mark.parametrize("rows", [200, 1000, 2304])
def test_panel_kernels_agree(rows):
    """One panel through the one-column kernel and through the two-column kernel with both CTA heights:
    the same reflectors up to rounding (V, tau and the compact-WY factor T)."""
    from soap_tp_b200.engine import kernels as k
    from soap_tp_b200.engine import qr

    device = torch.device("cuda", 0)
    generator = torch.Generator(device=device).manual_seed(rows)
    ws = qr._workspace(rows, device, slot=7)
    source = torch.randn(rows, rows, generator=generator, device=device)
    results = []
    for variant in ("one", 256, 128):
        k.split_planes(source, out=ws["C"])
        panel, v, vt, T, Tt = ws["C"].sub(0, 0, rows, 128), ws["V"].sub(0, 0, rows, 128), ws["Vt"][0], ws["T"][0], ws["Tt"][0]
        arguments = (panel.hi.data_ptr(), panel.lo.data_ptr(), panel.ld, rows, 128, v.hi.data_ptr(), v.lo.data_ptr(), v.ld,
                     vt.hi.data_ptr(), vt.lo.data_ptr(), vt.ld, ws["tau"].data_ptr(), T.hi.data_ptr(), T.lo.data_ptr(),
                     Tt.hi.data_ptr(), Tt.lo.data_ptr(), T.ld, ws["exchange"].data_ptr(),
                     k.status_word(device).data_ptr(), k._stream())
        if variant == "one":
            k._C.qr_panel(*arguments)
        else:
            k._C.qr_panel_pairs(*arguments, variant)
        torch.cuda.synchronize()
        k.check_status()
        results.append((v.dense().clone(), ws["tau"][:128].clone(), k.Planes(T.hi, T.lo, 128, 128, T.ld).dense().clone(),
                        vt.sub(0, 0, 128, rows).dense().clone()))
    qr.release_workspaces_for(rows, device)
    reference = results[0]
    for other in results[1:]:
        for a, b in zip(reference, other):
            assert float((a - b).abs().max()) < 2e-4 * max(1.0, float(a.abs().max()))
        assert torch.allclose(other[0], other[3].T, atol=1e-6)       # V and V^T outputs are the same matrix
