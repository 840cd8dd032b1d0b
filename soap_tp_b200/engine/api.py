"""Entry points the public ops call for CUDA tensors.

Grid (1, 1) runs the single-GPU pipeline of :mod:`.local`; larger grids run the distributed
pipeline of :mod:`.distributed`, whose kernels read peers' symmetric memory directly.
"""
from __future__ import annotations

from typing import Any, MutableMapping

import torch
import torch.distributed as dist
from torch import Tensor

from ..layout import empty_2d_block_cyclic_like_shape
from . import kernels as k
from . import local


def _world(group=None) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def _distributed():
    from . import distributed

    return distributed


def soap_step(gradient_shard: Tensor, state: MutableMapping[str, Any], *, global_shape, shard_dim, block_size, grid,
              preconditioner_beta, beta1, beta2, eps, basis_refresh_interval, basis_implementation, initializing) -> Tensor:
    if _world() == 1:
        update = local.soap_step(
            gradient_shard, state, global_shape=global_shape, beta=preconditioner_beta, beta1=beta1, beta2=beta2,
            eps=eps, interval=basis_refresh_interval, implementation=basis_implementation, initializing=initializing,
        ).view(gradient_shard.shape)
    else:
        update = _distributed().soap_step(
            gradient_shard, state, global_shape=global_shape, shard_dim=shard_dim, block_size=block_size, grid=grid,
            beta=preconditioner_beta, beta1=beta1, beta2=beta2, eps=eps, interval=basis_refresh_interval,
            implementation=basis_implementation, initializing=initializing,
        )
    # Every bounded wait of the kernels reports through the device status word; look at the copy taken at the
    # end of the previous step (no synchronisation) and raise SoapKernelError / SoapCommTimeout if it was set.
    k.poll_status(gradient_shard.device)
    return update


def redistribute_tp_to_bc(matrix, global_shape, block_size, grid, shard_dim, group) -> Tensor:
    if _world(group) == 1:
        rows, cols = global_shape
        packed = empty_2d_block_cyclic_like_shape(rows, cols, dtype=torch.float32, device=matrix.device, zero=False)
        source = matrix if matrix.dtype == torch.float32 else matrix.float()
        k.gather2d(source, packed[:rows, :cols], None, None)
        return packed if matrix.dtype == torch.float32 else packed.to(matrix.dtype)
    return _distributed().redistribute_tp_to_bc(matrix, global_shape, block_size, grid, shard_dim, group)


def redistribute_bc_to_tp(matrix, global_shape, block_size, grid, shard_dim, group) -> Tensor:
    if _world(group) == 1:
        rows, cols = global_shape
        shard = torch.empty((rows, cols), dtype=torch.float32, device=matrix.device)
        k.gather2d(matrix[:rows, :cols].float(), shard, None, None)
        return shard.to(matrix.dtype)
    return _distributed().redistribute_bc_to_tp(matrix, global_shape, block_size, grid, shard_dim, group)


def rotate(matrix, Q_left, Q_right, global_shape, block_size, grid, direction) -> Tensor:
    if _world() == 1:
        return local.rotate(matrix, Q_left, Q_right, global_shape, direction)
    return _distributed().rotate(matrix, Q_left, Q_right, global_shape, block_size, grid, direction)


def gram_update(G_local, preconditioner, beta, block_size, grid, shard_dim, side) -> Tensor:
    if _world() == 1:
        rows, cols = G_local.shape
        g32 = G_local if G_local.dtype == torch.float32 else G_local.float()
        size = rows if side == "left" else cols
        from ..layout import validate_2d_block_cyclic_buffer

        validate_2d_block_cyclic_buffer(f"{side}_preconditioner", preconditioner, (size, size), block_size, grid, 0)
        planes = k.split_planes(g32, transpose=(side == "left"),
                                out=local.workspace_planes("GT" if side == "left" else "X",
                                                           cols if side == "left" else rows, size, g32.device))
        k.gemm(planes, planes, out=preconditioner[:size, :size], alpha=1.0 - beta, beta=beta, symmetric=True)
        return preconditioner
    return _distributed().gram_update(G_local, preconditioner, beta, block_size, grid, shard_dim, side)


def estimated_order(P, Q, work, size, block_size, grid) -> Tensor:
    if _world() == 1:
        return local.estimated_order(P, Q, work, size)
    return _distributed().estimated_order(P, Q, work, size, block_size, grid)


def qr(matrix, Q, size, block_size, grid) -> Tensor:
    if _world() == 1:
        from . import factor

        factor.householder_qr(matrix[:size, :size], Q[:size, :size])
        return Q
    return _distributed().qr(matrix, Q, size, block_size, grid)


def power_iteration_qr(P, Q, work, size, block_size, grid) -> Tensor:
    if _world() == 1:
        return local.power_iteration_qr(P, Q, work, size)
    return _distributed().power_iteration_qr(P, Q, work, size, block_size, grid)


def initialize_basis(P, Q, work, eigenvalues, size, block_size, grid, implementation) -> Tensor:
    if _world() == 1:
        from . import factor

        factor.symmetric_eigenbasis(P[:size, :size], Q[:size, :size], work[:size, :size], eigenvalues, implementation)
        return Q
    return _distributed().initialize_basis(P, Q, work, eigenvalues, size, block_size, grid, implementation)


def permute(matrix, global_shape, row_order, column_order, block_size, grid, group) -> Tensor:
    if _world(group) == 1:
        return local.permute(matrix, global_shape, row_order, column_order)
    return _distributed().permute(matrix, global_shape, row_order, column_order, block_size, grid, group)
