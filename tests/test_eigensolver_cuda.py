"""The two symmetric eigensolvers (block Jacobi, Householder tridiagonalisation) against LAPACK (fp64) on one GPU.

Bounds follow the reference's eigensolver test (``tests/unit/test_elpa_bindings.py:478-501``: eigenvalues,
orthogonality and residual at 2e-4), tightened to what both solvers deliver.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _spectrum_case(n, seed, rank=None):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(n, rank or n, generator=g, dtype=torch.float64)
    return a @ a.T / (rank or n)


def _solve(solver, P64):
    from soap_tp_b200.engine import kernels as k

    n = P64.shape[0]
    P = P64.float().cuda().T.contiguous().T
    before = P.clone()
    Q = torch.empty(n, n, device="cuda").T
    values = torch.empty(n, device="cuda")
    solver.symmetric_eigenbasis(P, Q, torch.empty(n, n, device="cuda").T, values)
    k.check_status()
    assert torch.equal(P, before), "the input matrix must not be modified"
    return Q.double().cpu(), values.double().cpu()


def _check(P64, Qd, vd, value_tol=1e-5, ortho_tol=2e-5, residual_tol=5e-5):
    n = P64.shape[0]
    expected = torch.linalg.eigvalsh(P64).flip(0)
    scale = float(expected.abs().max())
    assert bool((vd[:-1] >= vd[1:] - 2e-5 * scale).all()), "eigenvalues must be descending"
    assert float((vd - expected).abs().max()) <= value_tol * scale, float((vd - expected).abs().max()) / scale
    ortho = float((Qd.T @ Qd - torch.eye(n, dtype=torch.float64)).abs().max())
    assert ortho <= ortho_tol, ortho
    residual = float((P64 @ Qd - Qd * vd).abs().max())
    assert residual <= residual_tol * scale, residual / scale


@pytest.mark.parametrize("n,rank", [(8, None), (100, None), (128, None), (130, None), (300, 120), (1000, None)])
def test_jacobi_matches_lapack(n, rank):
    from soap_tp_b200.engine import jacobi

    P64 = _spectrum_case(n, n, rank)
    Qd, vd = _solve(jacobi, P64)
    _check(P64, Qd, vd)
    assert jacobi.symmetric_eigenbasis.last_sweeps <= 20


@pytest.mark.parametrize("n,rank", [(3, None), (8, None), (33, None), (100, None), (128, None), (130, None), (300, 120),
                                    (1000, None), (1025, 400), (4096, None)])
def test_householder_matches_lapack(n, rank):
    from soap_tp_b200.engine import tridiag

    P64 = _spectrum_case(n, n, rank)
    before = getattr(tridiag.symmetric_eigenbasis, "fallbacks", 0)
    Qd, vd = _solve(tridiag, P64)
    _check(P64, Qd, vd)
    assert getattr(tridiag.symmetric_eigenbasis, "fallbacks", 0) == before, "a generic matrix must not need the fallback"


def test_householder_hands_repeated_eigenvalues_to_jacobi():
    """Exactly repeated eigenvalues (an identity block, a diagonal matrix with ties) cannot be separated by
    bisection; the solver must notice and still return a complete orthonormal eigenbasis."""
    from soap_tp_b200.engine import tridiag

    n = 96
    P64 = torch.eye(n, dtype=torch.float64) * 2.0
    P64[:10, :10] += _spectrum_case(10, 5)
    before = getattr(tridiag.symmetric_eigenbasis, "fallbacks", 0)
    Qd, vd = _solve(tridiag, P64)
    _check(P64, Qd, vd)
    assert getattr(tridiag.symmetric_eigenbasis, "fallbacks", 0) == before + 1


def test_factor_routes_names_to_different_solvers():
    from soap_tp_b200.engine import factor, kernels as k

    P64 = _spectrum_case(200, 7)
    P = P64.float().cuda().T.contiguous().T
    counts = {}
    for name in ("jacobi", "householder", "elpa", "eigh"):
        Q, values = torch.empty(200, 200, device="cuda").T, torch.empty(200, device="cuda")
        before = dict(k.LAUNCH_COUNTS)
        factor.symmetric_eigenbasis(P, Q, torch.empty(200, 200, device="cuda").T, values, name)
        counts[name] = {key: k.LAUNCH_COUNTS.get(key, 0) - before.get(key, 0) for key in ("jacobi_small_kernel", "sytrd_panel_kernel")}
        _check(P64, Q.double().cpu(), values.double().cpu())
    assert counts["jacobi"]["jacobi_small_kernel"] > 0 and counts["jacobi"]["sytrd_panel_kernel"] == 0
    for name in ("householder", "elpa", "eigh"):
        assert counts[name]["sytrd_panel_kernel"] > 0 and counts[name]["jacobi_small_kernel"] == 0
