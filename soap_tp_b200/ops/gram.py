"""Gram-matrix (Shampoo preconditioner) exponential moving averages in packed layout.

``L <- beta L + (1 - beta) G G^T`` and ``R <- beta R + (1 - beta) G^T G`` where ``G`` is given
as this rank's tensor-parallel shard and ``L``/``R`` are packed 2-D block-cyclic fp32 buffers
holding BOTH triangles.  Contract of the reference's
``update_left_preconditioner_2d_block_cyclic_`` / ``update_right_...``
(``src/soap_tp/ops/preconditioners.py:678-777``): in place, returns the buffer, the gradient
may be any float dtype, and shards may be unequal along the sharded dimension.

The reference computes one 128 x 128 tile at a time and reduces every tile with its own
``dist.reduce`` (``preconditioners.py:339-367``) or fetches 128-row panels with blocking
point-to-point messages (``preconditioners.py:523-582``).  The CUDA path here gathers the two
operand panels a rank needs by peer loads (all-gather fused with the 3xTF32 hi/lo split) and
runs one tcgen05 GEMM whose epilogue applies the EMA directly on the packed tiles.
"""
from __future__ import annotations

from typing import Literal

import torch
import torch.distributed as dist
from torch import Tensor

from ..layout import validate_2d_block_cyclic_buffer
from . import _hostpath as host
from ..parallel.guard import check_collective


def _check(G_local: Tensor, preconditioner: Tensor, beta: float, shard_dim: int, name: str) -> None:
    host.require_dist()
    if G_local.ndim != 2:
        raise ValueError(f"G_local must be 2D, got {G_local.ndim}D.")
    if shard_dim not in (0, 1):
        raise ValueError(f"shard_dim must be 0 or 1, got {shard_dim}.")
    if not 0.0 <= beta <= 1.0:
        raise ValueError(f"beta must be in [0, 1], got {beta}.")
    if preconditioner.dtype != torch.float32:
        raise ValueError(f"{name} must use float32, got {preconditioner.dtype}.")
    if preconditioner.device != G_local.device:
        raise ValueError(f"{name} is on {preconditioner.device}, expected {G_local.device}.")


def _update(G_local: Tensor, preconditioner: Tensor, beta: float, block_size: int, grid, shard_dim: int, side: str) -> Tensor:
    name = f"{side}_preconditioner"
    _check(G_local, preconditioner, beta, shard_dim, name)
    rank = dist.get_rank()
    if G_local.is_cuda:
        from ..engine import api as engine

        return engine.gram_update(G_local, preconditioner, beta, block_size, grid, shard_dim, side)
    full = host.gather_tp_shards(G_local.to(torch.float32).contiguous(), shard_dim)
    size = full.shape[0] if side == "left" else full.shape[1]
    validate_2d_block_cyclic_buffer(name, preconditioner, (size, size), block_size, grid, rank)
    gram = full @ full.T if side == "left" else full.T @ full
    row_index, column_index = host.local_index_pair((size, size), block_size, grid, rank)
    if row_index.numel() and column_index.numel():
        view = preconditioner[: row_index.numel(), : column_index.numel()]
        view.lerp_(gram[row_index[:, None], column_index], 1.0 - beta)
    return preconditioner


@torch.no_grad()
def update_left_preconditioner_2d_block_cyclic_(
    G_local: Tensor,
    left_preconditioner: Tensor,
    beta: float,
    block_size: int,
    process_grid_shape: tuple[int, int],
    *,
    shard_dim: Literal[0, 1],
) -> Tensor:
    """Update packed ``L = beta * L + (1 - beta) * G @ G.T`` in place."""
    check_collective("update_left_preconditioner_2d_block_cyclic_", block_size, tuple(process_grid_shape), shard_dim, float(beta))
    return _update(G_local, left_preconditioner, beta, block_size, process_grid_shape, shard_dim, "left")


@torch.no_grad()
def update_right_preconditioner_2d_block_cyclic_(
    G_local: Tensor,
    right_preconditioner: Tensor,
    beta: float,
    block_size: int,
    process_grid_shape: tuple[int, int],
    *,
    shard_dim: Literal[0, 1],
) -> Tensor:
    """Update packed ``R = beta * R + (1 - beta) * G.T @ G`` in place."""
    check_collective("update_right_preconditioner_2d_block_cyclic_", block_size, tuple(process_grid_shape), shard_dim, float(beta))
    return _update(G_local, right_preconditioner, beta, block_size, process_grid_shape, shard_dim, "right")


__all__ = [
    "update_left_preconditioner_2d_block_cyclic_",
    "update_right_preconditioner_2d_block_cyclic_",
]
