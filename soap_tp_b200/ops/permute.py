"""In-place global row/column permutation of a packed block-cyclic matrix.

Semantics of the reference's ``permute_2d_block_cyclic_``
(``src/soap_tp/ops/optimizer.py:395-567``): the result is ``matrix[row_order][:, column_order]``
without ever forming the global matrix on one rank, all ranks must pass identical orders
(verified with a MIN/MAX reduction, ``optimizer.py:439-452``) and call in the same sequence.

The reference plans the exchange with a triple-nested Python loop over every local element
(``optimizer.py:478-489``).  Here a permutation is an index map: the CUDA path hands the two
order vectors to a pull kernel that, for each owned destination element ``(i, j)``, loads
source element ``(row_order[i], column_order[j])`` from whichever peer owns it.  There is no
plan, no message and no host loop.
"""
from __future__ import annotations

from typing import Sequence, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from ..layout import local_2d_block_cyclic_shape
from . import _hostpath as host
from ..parallel.guard import check_collective


def validated_permutation(order, size: int, name: str, device=None) -> Tensor:
    """Return ``order`` as an int64 tensor after checking it is a permutation of ``range(size)``."""
    if isinstance(order, Tensor):
        if order.ndim != 1:
            raise ValueError(f"{name} must be 1D, got {order.ndim}D.")
        values = order.to(dtype=torch.int64)
    else:
        values = torch.tensor([int(index) for index in order], dtype=torch.int64)
    if values.numel() != size:
        raise ValueError(f"{name} must be a permutation of range({size}).")
    if size:
        seen = torch.zeros(size, dtype=torch.int64, device=values.device)
        in_range = (values >= 0) & (values < size)
        if not bool(in_range.all()):
            raise ValueError(f"{name} must be a permutation of range({size}).")
        seen.scatter_add_(0, values, torch.ones_like(values))
        if not bool((seen == 1).all()):
            raise ValueError(f"{name} must be a permutation of range({size}).")
    if device is not None:
        values = values.to(device)
    return values


@torch.no_grad()
def permute_2d_block_cyclic_(
    matrix: Tensor,
    global_shape: Tuple[int, int],
    row_order: Sequence[int] | Tensor,
    column_order: Sequence[int] | Tensor,
    block_size: int,
    process_grid_shape: Tuple[int, int],
    *,
    group=None,
) -> Tensor:
    """Apply ``matrix[row_order][:, column_order]`` to a packed matrix in place."""
    check_collective("permute_2d_block_cyclic_", tuple(global_shape), block_size, tuple(process_grid_shape), group=group)
    if matrix.ndim != 2:
        raise ValueError(f"matrix must be 2D, got {matrix.ndim}D.")
    if block_size <= 0:
        raise ValueError(f"block_size must be positive, got {block_size}.")
    rows, columns = global_shape
    if rows < 0 or columns < 0:
        raise ValueError(f"global_shape must be non-negative, got {global_shape}.")
    row_order = validated_permutation(row_order, rows, "row_order", matrix.device)
    column_order = validated_permutation(column_order, columns, "column_order", matrix.device)

    host.require_dist()
    world_size = dist.get_world_size(group)
    rank = dist.get_rank(group)
    process_rows, process_columns = process_grid_shape
    if process_rows <= 0 or process_columns <= 0:
        raise ValueError(
            f"process_grid_shape must contain positive dimensions, got {process_grid_shape}."
        )
    if process_rows * process_columns != world_size:
        raise ValueError("process grid must contain every process-group rank.")

    if world_size > 1:
        joined = torch.cat([row_order, column_order])
        if matrix.is_cuda and dist.get_backend(group) == "gloo":
            joined = joined.cpu()
        low, high = joined.clone(), joined.clone()
        dist.all_reduce(low, op=dist.ReduceOp.MIN, group=group)
        dist.all_reduce(high, op=dist.ReduceOp.MAX, group=group)
        if not torch.equal(low, high):
            raise ValueError("row_order and column_order must match on every rank.")

    local_rows, local_columns = local_2d_block_cyclic_shape(global_shape, block_size, process_grid_shape, rank)
    if matrix.size(0) < local_rows or matrix.size(1) < local_columns:
        raise ValueError(
            f"matrix shape {tuple(matrix.shape)} is smaller than its logical block-cyclic shape "
            f"{(local_rows, local_columns)}."
        )
    if matrix.is_cuda:
        from ..engine import api as engine

        return engine.permute(matrix, global_shape, row_order, column_order, block_size, process_grid_shape, group)
    full = host.gather_block_cyclic(matrix, global_shape, block_size, process_grid_shape, group=group)
    full = full[row_order][:, column_order]
    return host.store_block_cyclic_(matrix, full, global_shape, block_size, process_grid_shape, group=group)


__all__ = ["permute_2d_block_cyclic_", "validated_permutation"]
