"""Tensor-parallel shard <-> packed 2-D block-cyclic redistribution.

API parity with ``redistribute_tp_shard_to_2d_block_cyclic`` and
``redistribute_2d_block_cyclic_to_tp_shard`` of the reference
(``src/soap_tp/ops/optimizer.py:222-392`` and ``:64-219``): equal contiguous shards of the
sharded dimension, shard boundaries may cut blocks, the packed output is a fresh
column-major buffer, the shard output is a fresh row-major tensor.

The reference packs per-destination index_select results, runs a variable-split
``all_to_all_single`` and scatters with advanced indexing.  Here the CUDA path is a single
pull kernel: every rank reads the elements it owns straight out of its peers' shards
(symmetric memory, plain peer loads over NVLink) and writes its packed buffer, so there is
no pack, no unpack and no intermediate message.  CPU tensors use the dense host path.
"""
from __future__ import annotations

from typing import Literal, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from ..layout import (
    empty_2d_block_cyclic_like_shape,
    local_2d_block_cyclic_shape,
)
from . import _hostpath as host
from ..parallel.guard import check_collective


def _common_checks(matrix: Tensor, global_shape, block_size, process_grid_shape, shard_dim, group):
    if matrix.ndim != 2:
        raise ValueError(f"matrix must be 2D, got {matrix.ndim}D.")
    if shard_dim not in (0, 1):
        raise ValueError(f"shard_dim must be 0 or 1, got {shard_dim}.")
    if block_size <= 0:
        raise ValueError(f"block_size must be positive, got {block_size}.")
    host.require_dist()
    world_size = dist.get_world_size(group)
    rank = dist.get_rank(group)
    rows, columns = global_shape
    if rows < 0 or columns < 0:
        raise ValueError(f"global_shape must be non-negative, got {global_shape}.")
    process_rows, process_columns = process_grid_shape
    if process_rows <= 0 or process_columns <= 0:
        raise ValueError(
            f"process_grid_shape must contain positive dimensions, got {process_grid_shape}."
        )
    if process_rows * process_columns != world_size:
        raise ValueError("process grid must contain every process-group rank.")
    if (rows, columns)[shard_dim] % world_size != 0:
        raise ValueError(f"global dimension {shard_dim} must be divisible by the world size.")
    return rank, world_size


@torch.no_grad()
def redistribute_tp_shard_to_2d_block_cyclic(
    matrix: Tensor,
    global_shape: Tuple[int, int],
    block_size: int,
    process_grid_shape: Tuple[int, int],
    *,
    shard_dim: Literal[0, 1],
    group=None,
) -> Tensor:
    """Return the calling rank's packed block-cyclic part of a TP-sharded matrix."""
    check_collective("redistribute_tp_shard_to_2d_block_cyclic", tuple(global_shape), block_size, tuple(process_grid_shape), shard_dim, group=group)
    rank, world_size = _common_checks(matrix, global_shape, block_size, process_grid_shape, shard_dim, group)
    rows, columns = global_shape
    expected = [rows, columns]
    expected[shard_dim] //= world_size
    if tuple(matrix.shape) != tuple(expected):
        raise ValueError(
            f"matrix has local shape {tuple(matrix.shape)}, expected {tuple(expected)} for "
            f"shard_dim={shard_dim}."
        )
    if matrix.is_cuda:
        from ..engine import api as engine

        return engine.redistribute_tp_to_bc(matrix, global_shape, block_size, process_grid_shape, shard_dim, group)
    full = host.gather_tp_shards(matrix.contiguous(), shard_dim, group=group)
    local_rows, local_columns = local_2d_block_cyclic_shape(global_shape, block_size, process_grid_shape, rank)
    packed = empty_2d_block_cyclic_like_shape(local_rows, local_columns, dtype=matrix.dtype, device=matrix.device)
    return host.store_block_cyclic_(packed, full, global_shape, block_size, process_grid_shape, group=group)


@torch.no_grad()
def redistribute_2d_block_cyclic_to_tp_shard(
    matrix: Tensor,
    global_shape: Tuple[int, int],
    block_size: int,
    process_grid_shape: Tuple[int, int],
    *,
    shard_dim: Literal[0, 1],
    group=None,
) -> Tensor:
    """Return the calling rank's contiguous TP shard of a packed block-cyclic matrix."""
    check_collective("redistribute_2d_block_cyclic_to_tp_shard", tuple(global_shape), block_size, tuple(process_grid_shape), shard_dim, group=group)
    rank, world_size = _common_checks(matrix, global_shape, block_size, process_grid_shape, shard_dim, group)
    local_rows, local_columns = local_2d_block_cyclic_shape(global_shape, block_size, process_grid_shape, rank)
    if matrix.size(0) < local_rows or matrix.size(1) < local_columns:
        raise ValueError(
            f"matrix shape {tuple(matrix.shape)} is smaller than its logical block-cyclic shape "
            f"{(local_rows, local_columns)}."
        )
    if matrix.is_cuda:
        from ..engine import api as engine

        return engine.redistribute_bc_to_tp(matrix, global_shape, block_size, process_grid_shape, shard_dim, group)
    full = host.gather_block_cyclic(matrix, global_shape, block_size, process_grid_shape, group=group)
    shard = (global_shape[shard_dim]) // world_size
    return full.narrow(shard_dim, rank * shard, shard).contiguous()


__all__ = [
    "redistribute_2d_block_cyclic_to_tp_shard",
    "redistribute_tp_shard_to_2d_block_cyclic",
]
