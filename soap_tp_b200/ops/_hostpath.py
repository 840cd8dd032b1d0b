"""Host (CPU tensor) correctness path shared by the ops.

Every public op dispatches on the device of its buffers.  CUDA buffers go to the sm_100a
engine (hand-written kernels that read and write peers' memory); CPU buffers come here.
This path is deliberately simple: it rebuilds dense matrices with ``torch.distributed``
collectives (any backend that moves CPU tensors, normally gloo), computes with dense fp32
torch, and writes the owned entries back into the packed buffer.  It is the oracle every
kernel is tested against and the path of the CPU configuration (world size 4, grid (2, 2),
1024 x 1024), not a performance path.

The reference gathers full matrices only for tracing (``src/soap_tp/soap.py:60-120``) and
for its ``"eigh"`` initialisation (``src/soap_tp/ops/factorizations.py:421-470``); the
scatter-into-zeros + ``all_reduce`` idiom used there is the one used here.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from ..layout import (
    Grid,
    Shape2,
    grid_coords,
    local_2d_block_cyclic_shape,
    owned_indices,
    validate_process_grid,
)


def require_dist() -> None:
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed must be initialized first.")


def world(group=None) -> Tuple[int, int]:
    require_dist()
    return dist.get_rank(group), dist.get_world_size(group)


def local_index_pair(global_shape: Shape2, block_size: int, grid: Grid, rank: int, device=None):
    process_row, process_column = grid_coords(rank, grid)
    rows, columns = global_shape
    return (
        owned_indices(rows, block_size, process_row, grid[0], device),
        owned_indices(columns, block_size, process_column, grid[1], device),
    )


def gather_block_cyclic(
    matrix: Tensor,
    global_shape: Shape2,
    block_size: int,
    grid: Grid,
    *,
    group=None,
    dtype: Optional[torch.dtype] = None,
) -> Tensor:
    """Dense ``global_shape`` copy of a packed matrix on every rank."""
    rank, world_size = world(group)
    validate_process_grid(grid, world_size)
    row_index, column_index = local_index_pair(global_shape, block_size, grid, rank, matrix.device)
    full = torch.zeros(global_shape, dtype=dtype or matrix.dtype, device=matrix.device)
    if row_index.numel() and column_index.numel():
        full[row_index[:, None], column_index] = matrix[
            : row_index.numel(), : column_index.numel()
        ].to(full.dtype)
    if world_size > 1:
        dist.all_reduce(full, group=group)
    return full


def store_block_cyclic_(
    matrix: Tensor,
    full: Tensor,
    global_shape: Shape2,
    block_size: int,
    grid: Grid,
    *,
    group=None,
) -> Tensor:
    """Write the entries of dense ``full`` that the calling rank owns into packed ``matrix``."""
    rank, _ = world(group)
    row_index, column_index = local_index_pair(global_shape, block_size, grid, rank, matrix.device)
    if row_index.numel() and column_index.numel():
        matrix[: row_index.numel(), : column_index.numel()] = full[
            row_index[:, None], column_index
        ].to(matrix.dtype)
    return matrix


def gather_tp_shards(shard: Tensor, shard_dim: int, *, group=None) -> Tensor:
    """Concatenate (possibly unequal) contiguous TP shards into the dense matrix."""
    _, world_size = world(group)
    if world_size == 1:
        return shard
    shape = torch.tensor(list(shard.shape), dtype=torch.int64)
    shapes = [torch.empty_like(shape) for _ in range(world_size)]
    dist.all_gather(shapes, shape, group=group)
    dims = [tuple(int(v) for v in s.tolist()) for s in shapes]
    replicated = 1 - shard_dim
    if any(d[replicated] != dims[0][replicated] for d in dims):
        raise ValueError(f"non-sharded dimension {replicated} must match on every rank.")
    longest = max(d[shard_dim] for d in dims)
    padded_shape = list(shard.shape)
    padded_shape[shard_dim] = longest
    padded = shard.new_zeros(padded_shape)
    padded.narrow(shard_dim, 0, shard.shape[shard_dim]).copy_(shard)
    parts: List[Tensor] = [torch.empty_like(padded) for _ in range(world_size)]
    dist.all_gather(parts, padded.contiguous(), group=group)
    return torch.cat(
        [part.narrow(shard_dim, 0, d[shard_dim]) for part, d in zip(parts, dims)], dim=shard_dim
    )


def logical_view(matrix: Tensor, global_shape: Shape2, block_size: int, grid: Grid, rank: int) -> Tensor:
    local_rows, local_columns = local_2d_block_cyclic_shape(global_shape, block_size, grid, rank)
    return matrix[:local_rows, :local_columns]
