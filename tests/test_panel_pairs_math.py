"""The algebra of the two-columns-per-exchange panel kernel, checked on the CPU through its NumPy
restatement: the block reflector is orthogonal and triangularises the panel on well-conditioned,
graded, rank-deficient and duplicated inputs, and the cancellation guard decides what it should."""
import numpy as np
import pytest

from soap_tp_b200.utils.panel_pairs_reference import factor_panel


def _check(A, V, T, tolerance):
    Vd, Td = V.astype(np.float64), T.astype(np.float64)
    Q = np.eye(A.shape[0]) - Vd @ Td @ Vd.T
    orthogonality = np.abs(Q.T @ Q - np.eye(A.shape[0])).max()
    reduced = Q.T @ A.astype(np.float32).astype(np.float64)
    below = np.linalg.norm(np.tril(reduced, -1)) / max(np.linalg.norm(A), 1e-30)
    assert orthogonality < tolerance, orthogonality
    assert below < tolerance, below


@pytest.mark.parametrize("name", ["gauss", "graded", "lowrank", "duplicated", "odd_width", "wide"])
def test_two_column_steps(name):
    rng = np.random.default_rng(3)
    A = {
        "gauss": lambda: rng.standard_normal((768, 64)),
        "graded": lambda: np.cumsum(rng.standard_normal((768, 64)) * np.logspace(0, -5, 64), axis=1),
        "lowrank": lambda: rng.standard_normal((768, 10)) @ rng.standard_normal((10, 64)),
        "duplicated": lambda: np.repeat(rng.standard_normal((512, 32)), 2, axis=1),
        "odd_width": lambda: rng.standard_normal((300, 31)),
        "wide": lambda: rng.standard_normal((20, 32)),
    }[name]()
    V, tau, T, (single, paired) = factor_panel(A)
    _check(A, V, T, 2e-5)
    assert single + 2 * paired == min(A.shape)
    if name == "gauss":
        assert single == 0 and paired == 32
    if name == "duplicated":
        assert single >= 2                   # a repeated column cannot share a step with its twin


def test_guard_is_what_keeps_rank_deficient_panels_orthogonal():
    """Rank-20 panels of 128 columns: without the guard the derived norm of the second column cancels on
    some instances (1.5e-3 on the first one here); with it every instance stays at the one-column level
    while nearly all steps still retire two columns."""
    worst_unguarded, worst_guarded = 0.0, 0.0
    for seed in (1, 3, 5):
        rng = np.random.default_rng(seed)
        rng.standard_normal((2048, 128))
        A = rng.standard_normal((2048, 20)) @ rng.standard_normal((20, 128))
        for threshold in (0.0, 0.5):
            V, tau, T, (single, paired) = factor_panel(A, threshold=threshold)
            Vd, Td = V.astype(np.float64), T.astype(np.float64)
            Q = np.eye(A.shape[0]) - Vd @ Td @ Vd.T
            error = float(np.abs(Q.T @ Q - np.eye(A.shape[0])).max())
            if threshold == 0.0:
                worst_unguarded = max(worst_unguarded, error)
            else:
                worst_guarded = max(worst_guarded, error)
                assert paired >= 60
    assert worst_guarded < 1e-5
    assert worst_unguarded > 1e-4
