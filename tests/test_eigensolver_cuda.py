"""The block-Jacobi eigensolver against LAPACK (fp64) on one GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _spectrum_case(n, seed, rank=None):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(n, rank or n, generator=g, dtype=torch.float64)
    return a @ a.T / (rank or n)


@pytest.mark.parametrize("n,rank", [(8, None), (100, None), (128, None), (130, None), (300, 120), (1000, None)])
def test_jacobi_matches_lapack(n, rank):
    from soap_tp_b200.engine import jacobi, kernels as k

    P64 = _spectrum_case(n, n, rank)
    P = P64.float().cuda().T.contiguous().T
    Q = torch.empty(n, n, device="cuda").T
    values = torch.empty(n, device="cuda")
    jacobi.symmetric_eigenbasis(P, Q, torch.empty(n, n, device="cuda").T, values)
    k.check_status()
    expected = torch.linalg.eigvalsh(P64).flip(0)
    scale = float(expected.abs().max())
    Qd, vd = Q.double().cpu(), values.double().cpu()
    assert bool((vd[:-1] >= vd[1:] - 2e-5 * scale).all()), "eigenvalues must be descending"
    assert float((vd - expected).abs().max()) <= 1e-5 * scale
    assert float((Qd.T @ Qd - torch.eye(n, dtype=torch.float64)).abs().max()) <= 2e-5
    assert float((P64 @ Qd - Qd * vd).abs().max()) <= 5e-5 * scale
    assert jacobi.symmetric_eigenbasis.last_sweeps <= 20
