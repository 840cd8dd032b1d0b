"""Dense factorisations on one GPU: Householder QR and the symmetric eigensolver.

These operate on column-major device matrices that are entirely local (grid (1, 1), or a panel a
rank has gathered).  See ``csrc/qr.cu`` and ``csrc/jacobi.cu`` for the kernels.
"""
from __future__ import annotations

from typing import Optional

from torch import Tensor


def householder_qr(matrix: Tensor, Q: Tensor, column_order: Optional[Tensor] = None) -> Tensor:
    """``Q <- explicit orthogonal factor of matrix[:, column_order]``; ``matrix`` is scratch."""
    from ..ops.basis import count_qr_call
    from . import qr

    count_qr_call()
    return qr.householder_qr(matrix, Q, column_order)


def householder_qr_pair(jobs) -> None:
    """Several independent QR factorisations issued concurrently; ``jobs``: ``(matrix, Q, column_order)``."""
    from ..ops.basis import count_qr_call
    from . import qr

    for _ in jobs:
        count_qr_call()
    qr.householder_qr_pair(jobs)


def symmetric_eigenbasis(P: Tensor, Q: Tensor, work: Tensor, values: Tensor, implementation: str) -> Tensor:
    """Eigenvectors of symmetric ``P`` into ``Q`` and eigenvalues into ``values``, both descending.

    ``"jacobi"`` runs the two-sided block-Jacobi solver (``engine/jacobi.py``); every other accepted name
    (``"householder"``, and the reference's ``"elpa"`` and ``"eigh"``) runs Householder tridiagonalisation,
    bisection and twisted factorisation with back-transformation (``engine/tridiag.py``) -- the method of the
    reference's ELPA default (``src/soap_tp/ops/factorizations.py:472-547``)."""
    if implementation == "jacobi":
        from . import jacobi

        return jacobi.symmetric_eigenbasis(P, Q, work, values)
    from . import tridiag

    return tridiag.symmetric_eigenbasis(P, Q, work, values)
