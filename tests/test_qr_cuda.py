"""Blocked Householder QR on the GPU against its defining properties (fp64 checks).

The reference tests its QR through ``power_iteration_qr`` on tiny sizes
(``tests/test_gpu_ops.py``); here the factorisation kernel chain itself is exercised on sizes that
span several panels, ragged last panels, a rank-deficient input, and the concurrent two-job driver.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(matrix: torch.Tensor, Q: torch.Tensor, tolerance: float) -> None:
    a, q = matrix.double().cpu(), Q.double().cpu()
    n = a.shape[0]
    orthogonality = float((q.T @ q - torch.eye(n, dtype=torch.float64)).abs().max())
    r = q.T @ a
    below = float(torch.tril(r, -1).norm() / a.norm().clamp_min(1e-30))
    assert orthogonality < tolerance, f"|Q^T Q - I|_max = {orthogonality}"
    assert below < tolerance, f"|tril(Q^T A)| / |A| = {below}"


@pytest.mark.parametrize("n", [128, 200, 384, 1000, 2048])
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
