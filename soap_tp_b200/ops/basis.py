"""Eigenbasis initialisation, power-iteration + QR refresh and optimizer-state transport.

Public functions and their reference counterparts (``src/soap_tp/ops/factorizations.py``):

* ``estimated_eigenvalue_order_2d_block_cyclic_``  (``:187-271``) -- ``work <- P Q``, then the
  descending order of ``diag(Q^T P Q)``;
* ``qr_2d_block_cyclic_``                          (``:274-320``) -- explicit Householder ``Q``;
* ``power_iteration_qr_2d_block_cyclic_``          (``:323-360``);
* ``initialize_basis_2d_block_cyclic_``            (``:363-547``) -- descending eigenbasis;
* ``refresh_bases_and_transport_optimizer_state_`` (``:550-614``).

The reference reaches SLATE (GEMM, ``geqrf``/``unmqr``) and ELPA (fp64 one-stage eigensolver)
through two pybind11 modules.  Here the CUDA path uses this package's own sm_100a kernels: the
3xTF32 tcgen05 GEMM for ``P Q`` with the column-dot epilogue, a blocked Householder QR whose
panel is factored by a cooperative kernel and whose trailing updates are tensor-core GEMMs, and
two symmetric eigensolvers: Householder tridiagonalisation with bisection and twisted factorisation
(``"householder"``, and the reference's names ``"elpa"`` and ``"eigh"``) and two-sided block Jacobi
(``"jacobi"``).  On CPU tensors every name resolves to LAPACK ``torch.linalg.eigh`` on rank 0 followed by a
broadcast, as ``"eigh"`` does in the reference.
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from . import _hostpath as host
from .permute import permute_2d_block_cyclic_
from .rotate import _synchronize, rotate_2d_block_cyclic_, validate_float_buffer, validate_world
from ..layout import local_2d_block_cyclic_shape
from ..parallel.guard import check_collective

BASIS_IMPLEMENTATIONS = ("elpa", "eigh", "jacobi", "householder")

_QR_CALLS = 0


def qr_call_count() -> int:
    """Number of QR factorisations run by this process (the reference's tests count
    ``slate_qr_float`` calls through a proxy binding, ``tests/unit/test_soap.py:402-412``)."""
    return _QR_CALLS


def count_qr_call() -> None:
    """Called by every QR factorisation, host path or device engine."""
    global _QR_CALLS
    _QR_CALLS += 1


def _stable_descending_order(values: Tensor) -> Tensor:
    return torch.argsort(values, descending=True, stable=True)


@torch.no_grad()
def estimated_eigenvalue_order_2d_block_cyclic_(
    preconditioner: Tensor,
    Q: Tensor,
    work: Tensor,
    size: int,
    block_size: int,
    process_grid_shape: Tuple[int, int],
    *,
    slate_binding: Optional[Any] = None,
) -> Tensor:
    """Overwrite ``work`` with ``P @ Q`` and return ``argsort(diag(Q.T P Q), descending)``.

    The returned int64 tensor is identical on every rank; ties are broken by index (stable).
    """
    check_collective("estimated_eigenvalue_order_2d_block_cyclic_", size, block_size, tuple(process_grid_shape))
    rank, _ = validate_world(process_grid_shape)
    buffers = (("preconditioner", preconditioner), ("Q", Q), ("work", work))
    for name, matrix in buffers:
        validate_float_buffer(name, matrix, (size, size), block_size, process_grid_shape, rank)
        if matrix.device != preconditioner.device:
            raise ValueError("preconditioner, Q, and work must share a device.")
    if len({matrix.data_ptr() for _, matrix in buffers}) != len(buffers):
        raise ValueError("preconditioner, Q, and work must not overlap.")
    if not (preconditioner.stride(1) == Q.stride(1) == work.stride(1)):
        raise ValueError("preconditioner, Q, and work LDAs must match.")
    grid = process_grid_shape
    if slate_binding is not None:
        # the injected binding forms work = P Q (src/soap_tp/ops/factorizations.py:235-244); the estimates follow
        _synchronize(preconditioner.device)
        slate_binding.slate_symmetric_multiply_float(preconditioner.data_ptr(), Q.data_ptr(), work.data_ptr(), size,
                                                     preconditioner.stride(1), block_size, grid[0], grid[1])
        _synchronize(preconditioner.device)
        Qf = host.gather_block_cyclic(Q.cpu(), (size, size), block_size, grid)
        W = host.gather_block_cyclic(work.cpu(), (size, size), block_size, grid)
        return _stable_descending_order((Qf * W).sum(dim=0)).to(preconditioner.device)
    if preconditioner.is_cuda:
        from ..engine import api as engine

        return engine.estimated_order(preconditioner, Q, work, size, block_size, process_grid_shape)
    P = host.gather_block_cyclic(preconditioner, (size, size), block_size, grid)
    Qf = host.gather_block_cyclic(Q, (size, size), block_size, grid)
    W = P @ Qf
    host.store_block_cyclic_(work, W, (size, size), block_size, grid)
    estimates = (Qf * W).sum(dim=0)
    return _stable_descending_order(estimates)


@torch.no_grad()
def qr_2d_block_cyclic_(
    matrix: Tensor,
    Q: Tensor,
    size: int,
    block_size: int,
    process_grid_shape: Tuple[int, int],
    *,
    slate_binding: Optional[Any] = None,
) -> Tensor:
    """Overwrite ``Q`` with the explicit orthogonal factor of ``matrix`` (Householder QR).

    ``matrix`` is scratch afterwards.  Column signs are those of an unnormalised Householder
    factorisation (``R`` may have negative diagonal entries).
    """
    check_collective("qr_2d_block_cyclic_", size, block_size, tuple(process_grid_shape))
    rank, _ = validate_world(process_grid_shape)
    for name, buffer in (("matrix", matrix), ("Q", Q)):
        validate_float_buffer(name, buffer, (size, size), block_size, process_grid_shape, rank)
    if matrix.device != Q.device:
        raise ValueError("matrix and Q must share a device.")
    if matrix.data_ptr() == Q.data_ptr():
        raise ValueError("matrix and Q must not overlap.")
    if slate_binding is not None:
        count_qr_call()
        _synchronize(matrix.device)
        slate_binding.slate_qr_float(matrix.data_ptr(), Q.data_ptr(), size, matrix.stride(1), Q.stride(1), block_size,
                                     process_grid_shape[0], process_grid_shape[1])
        _synchronize(matrix.device)
        return Q
    if matrix.is_cuda:
        from ..engine import api as engine

        return engine.qr(matrix, Q, size, block_size, process_grid_shape)
    count_qr_call()
    grid = process_grid_shape
    M = host.gather_block_cyclic(matrix, (size, size), block_size, grid)
    Qf, _ = torch.linalg.qr(M)
    return host.store_block_cyclic_(Q, Qf, (size, size), block_size, grid)


@torch.no_grad()
def power_iteration_qr_2d_block_cyclic_(
    preconditioner: Tensor,
    Q: Tensor,
    work: Tensor,
    size: int,
    block_size: int,
    process_grid_shape: Tuple[int, int],
    *,
    slate_binding: Optional[Any] = None,
) -> Tensor:
    """One power iteration: sort ``P Q`` by estimated eigenvalue, QR it into ``Q``; returns the order."""
    check_collective("power_iteration_qr_2d_block_cyclic_", size, block_size, tuple(process_grid_shape))
    if preconditioner.is_cuda and slate_binding is None:
        # Validation happens inside the two public ops on the host path; the fused device path
        # validates once and folds the column permutation into the QR's panel gather.
        rank, _ = validate_world(process_grid_shape)
        for name, matrix in (("preconditioner", preconditioner), ("Q", Q), ("work", work)):
            validate_float_buffer(name, matrix, (size, size), block_size, process_grid_shape, rank)
        if len({preconditioner.data_ptr(), Q.data_ptr(), work.data_ptr()}) != 3:
            raise ValueError("preconditioner, Q, and work must not overlap.")
        from ..engine import api as engine

        return engine.power_iteration_qr(preconditioner, Q, work, size, block_size, process_grid_shape)
    order = estimated_eigenvalue_order_2d_block_cyclic_(
        preconditioner, Q, work, size, block_size, process_grid_shape, slate_binding=slate_binding
    )
    identity = torch.arange(size, dtype=torch.int64, device=work.device)
    permute_2d_block_cyclic_(work, (size, size), identity, order, block_size, process_grid_shape)
    qr_2d_block_cyclic_(work, Q, size, block_size, process_grid_shape, slate_binding=slate_binding)
    return order


@torch.no_grad()
def initialize_basis_2d_block_cyclic_(
    preconditioner: Tensor,
    Q: Tensor,
    work: Tensor,
    eigenvalues: Tensor,
    size: int,
    block_size: int,
    process_grid_shape: Tuple[int, int],
    *,
    implementation: str = "elpa",
    elpa_binding: Optional[Any] = None,
) -> Tensor:
    """Fill ``Q`` with eigenvectors of the packed symmetric ``preconditioner`` and
    ``eigenvalues`` with its eigenvalues, both in descending eigenvalue order.

    ``preconditioner`` must hold both triangles and is left untouched; ``work`` may be
    clobbered.  Unlike the reference's ELPA path there is no requirement that every rank owns
    at least one row and column, nor that the leading dimension is exact.
    """
    check_collective("initialize_basis_2d_block_cyclic_", size, block_size, tuple(process_grid_shape), implementation)
    if implementation not in BASIS_IMPLEMENTATIONS:
        raise ValueError(
            f"implementation must be one of {BASIS_IMPLEMENTATIONS}, got {implementation!r}."
        )
    rank, _ = validate_world(process_grid_shape)
    buffers = (("preconditioner", preconditioner), ("Q", Q), ("work", work))
    for name, matrix in buffers:
        validate_float_buffer(name, matrix, (size, size), block_size, process_grid_shape, rank)
        if matrix.device != preconditioner.device:
            raise ValueError("preconditioner, Q, and work must share a device.")
    if len({preconditioner.data_ptr(), Q.data_ptr(), work.data_ptr()}) != 3:
        raise ValueError("preconditioner, Q, and work must not overlap.")
    if eigenvalues.shape != (size,) or eigenvalues.dtype != torch.float32:
        raise ValueError(
            f"eigenvalues must be float32 with shape {(size,)}, got {eigenvalues.dtype} "
            f"{tuple(eigenvalues.shape)}."
        )
    if not eigenvalues.is_contiguous():
        raise ValueError("eigenvalues must be contiguous.")
    if eigenvalues.device != preconditioner.device:
        raise ValueError("eigenvalues must share the matrix device.")
    if elpa_binding is not None and implementation == "elpa":
        # An injected eigensolver with the reference's entry point: fp64 copies, -A so that its ascending order
        # is the descending order of A (src/soap_tp/ops/factorizations.py:495-546)
        local_rows, local_columns = local_2d_block_cyclic_shape((size, size), block_size, process_grid_shape, rank)
        work.copy_(preconditioner).neg_()
        work64 = torch.empty_strided(work.size(), work.stride(), dtype=torch.float64, device=work.device).copy_(work)
        Q64 = torch.empty_strided(Q.size(), Q.stride(), dtype=torch.float64, device=Q.device)
        values64 = torch.empty_like(eigenvalues, dtype=torch.float64)
        gpu_id = -1 if not preconditioner.is_cuda else (preconditioner.device.index or 0)
        _synchronize(preconditioner.device)
        elpa_binding.elpa_eigenvectors_2d_block_cyclic_double(
            work64.data_ptr(), values64.data_ptr(), Q64.data_ptr(), size, local_rows, local_columns, block_size,
            process_grid_shape[0], process_grid_shape[1], gpu_id)
        _synchronize(preconditioner.device)
        Q.copy_(Q64)
        eigenvalues.copy_(values64).neg_()
        return Q
    if preconditioner.is_cuda:
        from ..engine import api as engine

        return engine.initialize_basis(
            preconditioner, Q, work, eigenvalues, size, block_size, process_grid_shape, implementation
        )
    grid = process_grid_shape
    full = host.gather_block_cyclic(preconditioner, (size, size), block_size, grid)
    if rank == 0:
        values, vectors = torch.linalg.eigh(full)
        eigenvalues.copy_(values.flip(0))
        full.copy_(vectors.flip(1))
    if dist.get_world_size() > 1:
        dist.broadcast(eigenvalues, src=0)
        dist.broadcast(full, src=0)
    return host.store_block_cyclic_(Q, full, (size, size), block_size, grid)


@torch.no_grad()
def refresh_bases_and_transport_optimizer_state_(
    momentum: Tensor,
    variance: Tensor,
    left_preconditioner: Tensor,
    right_preconditioner: Tensor,
    Q_left: Tensor,
    Q_right: Tensor,
    left_work: Tensor,
    right_work: Tensor,
    global_shape: Tuple[int, int],
    block_size: int,
    process_grid_shape: Tuple[int, int],
    *,
    slate_binding: Optional[Any] = None,
) -> tuple[Tensor, Tensor]:
    """Refresh both bases by one power iteration + QR while keeping SOAP's state consistent.

    Momentum is rotated out of the old bases and into the new ones; the variance (which lives
    in rotated coordinates) is permuted by the two eigenvalue orders.  Returns
    ``(left_order, right_order)``.
    """
    check_collective("refresh_bases_and_transport_optimizer_state_", tuple(global_shape), block_size, tuple(process_grid_shape))
    rows, columns = global_shape
    grid = process_grid_shape
    injected = dict(slate_binding=slate_binding)
    rotate_2d_block_cyclic_(momentum, Q_left, Q_right, global_shape, block_size, grid, direction="backward", **injected)
    left_order = power_iteration_qr_2d_block_cyclic_(
        left_preconditioner, Q_left, left_work, rows, block_size, grid, **injected
    )
    right_order = power_iteration_qr_2d_block_cyclic_(
        right_preconditioner, Q_right, right_work, columns, block_size, grid, **injected
    )
    permute_2d_block_cyclic_(variance, global_shape, left_order, right_order, block_size, grid)
    rotate_2d_block_cyclic_(momentum, Q_left, Q_right, global_shape, block_size, grid, direction="forward", **injected)
    return left_order, right_order


__all__ = [
    "BASIS_IMPLEMENTATIONS",
    "estimated_eigenvalue_order_2d_block_cyclic_",
    "initialize_basis_2d_block_cyclic_",
    "power_iteration_qr_2d_block_cyclic_",
    "qr_2d_block_cyclic_",
    "qr_call_count",
    "refresh_bases_and_transport_optimizer_state_",
]
