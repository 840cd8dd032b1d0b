"""Closed-form 2-D block-cyclic layout math.

The optimizer state of tensor-parallel SOAP lives in ScaLAPACK-style packed buffers: a
row-major ``Pr x Pc`` process grid, square blocks of ``block_size``, column-major local
storage with leading dimension ``max(1, local_rows)``.  The reference enumerates the
owned indices with an O(n) Python loop (``src/soap_tp/ops/_utils.py:47-71``) and sizes
the local buffer from the length of that enumeration (``_utils.py:91-117``).  Here the
same quantities come from closed forms (``numroc``) and from vectorised index tensors
that are cached per ``(n, nb, p, P, device)``, so that planning never loops in Python
over matrix elements.

Conventions (all identical to the reference so that checkpoints interchange):

* rank -> grid coordinates: ``pr = rank // Pc``, ``pc = rank % Pc``;
* owner of global index ``g`` along a dimension: ``(g // nb) % P``;
* local index of ``g``: ``(g // nb // P) * nb + g % nb``;
* tile ``(bi, bj)`` belongs to rank ``(bi % Pr) * Pc + (bj % Pc)``.
"""
from __future__ import annotations

from functools import lru_cache
from typing import Dict, Iterator, Literal, Tuple

import torch
import torch.distributed as dist

Grid = Tuple[int, int]
Shape2 = Tuple[int, int]


def ceil_div(a: int, b: int) -> int:
    if b <= 0:
        raise ValueError(f"b must be positive, got {b}.")
    return -(-a // b)


def num_blocks(dim: int, block_size: int) -> int:
    if dim < 0:
        raise ValueError(f"dim must be non-negative, got {dim}.")
    return ceil_div(dim, block_size)


def block_bounds(block_id: int, block_size: int, dim: int) -> Tuple[int, int]:
    if block_size <= 0:
        raise ValueError(f"block_size must be positive, got {block_size}.")
    start = block_id * block_size
    return start, min(start + block_size, dim)


def validate_process_grid(process_grid_shape: Grid, world_size: int) -> None:
    """Same contract as ``_utils.py:74-88`` of the reference."""
    process_rows, process_columns = process_grid_shape
    if process_rows <= 0 or process_columns <= 0:
        raise ValueError(
            "process_grid_shape must contain positive dimensions, got "
            f"{process_grid_shape}."
        )
    if process_rows * process_columns != world_size:
        raise ValueError(
            f"process_grid_shape={process_grid_shape} does not match "
            f"world_size={world_size}."
        )


def grid_coords(rank: int, process_grid_shape: Grid) -> Tuple[int, int]:
    process_rows, process_columns = process_grid_shape
    if not 0 <= rank < process_rows * process_columns:
        raise ValueError(
            f"rank must be in [0, {process_rows * process_columns}), got {rank}."
        )
    return rank // process_columns, rank % process_columns


def block_cyclic_owner_rank(block_row: int, block_col: int, process_grid_shape: Grid) -> int:
    """Rank that owns tile ``(block_row, block_col)`` (``_utils.py:29-44``)."""
    process_rows, process_columns = process_grid_shape
    if process_rows <= 0 or process_columns <= 0:
        raise ValueError(f"process_grid_shape must be positive, got {process_grid_shape}.")
    return (block_row % process_rows) * process_columns + (block_col % process_columns)


def numroc(size: int, block_size: int, process: int, process_count: int) -> int:
    """Number of indices of ``range(size)`` owned by ``process`` (ScaLAPACK NUMROC)."""
    if size < 0:
        raise ValueError(f"size must be non-negative, got {size}.")
    if block_size <= 0:
        raise ValueError(f"block_size must be positive, got {block_size}.")
    if process_count <= 0:
        raise ValueError(f"process_count must be positive, got {process_count}.")
    if not 0 <= process < process_count:
        raise ValueError(f"process must be in [0, {process_count}), got {process}.")
    full_blocks, remainder = divmod(size, block_size)
    count = (full_blocks // process_count) * block_size
    extra = full_blocks % process_count
    if process < extra:
        count += block_size
    elif process == extra:
        count += remainder
    return count


@lru_cache(maxsize=None)
def _owned_indices_cpu(size: int, block_size: int, process: int, process_count: int) -> torch.Tensor:
    count = numroc(size, block_size, process, process_count)
    local = torch.arange(count, dtype=torch.int64)
    block = torch.div(local, block_size, rounding_mode="floor")
    return (block * process_count + process) * block_size + local % block_size


_DEVICE_INDEX_CACHE: Dict[tuple, torch.Tensor] = {}


def owned_indices(
    size: int,
    block_size: int,
    process: int,
    process_count: int,
    device: torch.device | str | None = None,
) -> torch.Tensor:
    """Global indices owned by ``process`` in local order (int64 tensor, cached).

    Vectorised replacement of ``block_cyclic_indices`` (``_utils.py:47-71``).
    """
    cpu = _owned_indices_cpu(size, block_size, process, process_count)
    if device is None or torch.device(device).type == "cpu":
        return cpu
    key = (size, block_size, process, process_count, str(torch.device(device)))
    cached = _DEVICE_INDEX_CACHE.get(key)
    if cached is None:
        cached = cpu.to(device)
        _DEVICE_INDEX_CACHE[key] = cached
    return cached


def block_cyclic_indices(size: int, block_size: int, process: int, process_count: int) -> Tuple[int, ...]:
    """Tuple form of :func:`owned_indices`, kept for callers of the reference's helper."""
    return tuple(owned_indices(size, block_size, process, process_count).tolist())


def global_to_local(index: torch.Tensor, block_size: int, process_count: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Map global indices to ``(owner process, local index)``."""
    block = torch.div(index, block_size, rounding_mode="floor")
    owner = block % process_count
    local = torch.div(block, process_count, rounding_mode="floor") * block_size + index % block_size
    return owner, local


def local_2d_block_cyclic_shape(
    global_shape: Shape2,
    block_size: int,
    process_grid_shape: Grid,
    rank: int,
) -> Tuple[int, int]:
    rows, columns = global_shape
    process_rows, process_columns = process_grid_shape
    validate_process_grid(process_grid_shape, process_rows * process_columns)
    process_row, process_column = grid_coords(rank, process_grid_shape)
    return (
        numroc(rows, block_size, process_row, process_rows),
        numroc(columns, block_size, process_column, process_columns),
    )


def validate_2d_block_cyclic_buffer(
    name: str,
    matrix: torch.Tensor,
    global_shape: Shape2,
    block_size: int,
    process_grid_shape: Grid,
    rank: int,
) -> Tuple[int, int]:
    """Check the packed-buffer contract (``_utils.py:120-156``) and return the logical shape."""
    if matrix.ndim != 2:
        raise ValueError(f"{name} must be 2D, got {matrix.ndim}D.")
    if matrix.stride(0) != 1:
        raise ValueError(
            f"{name} must use column-major local storage, got stride {tuple(matrix.stride())}."
        )
    local_rows, local_columns = local_2d_block_cyclic_shape(
        global_shape, block_size, process_grid_shape, rank
    )
    if matrix.size(0) < max(1, local_rows):
        raise ValueError(
            f"{name} has {matrix.size(0)} storage rows, expected at least {max(1, local_rows)}."
        )
    if matrix.size(1) < max(1, local_columns):
        raise ValueError(
            f"{name} has {matrix.size(1)} storage columns, expected at least "
            f"{max(1, local_columns)}."
        )
    if matrix.stride(1) < max(1, matrix.size(0)):
        raise ValueError(f"{name} has invalid leading dimension {matrix.stride(1)}.")
    return local_rows, local_columns


def empty_2d_block_cyclic_like_shape(
    local_rows: int,
    local_columns: int,
    *,
    dtype: torch.dtype = torch.float32,
    device: torch.device | str | None = None,
    zero: bool = True,
) -> torch.Tensor:
    leading_dimension = max(1, local_rows)
    storage_columns = max(1, local_columns)
    factory = torch.zeros if zero else torch.empty
    return factory((storage_columns, leading_dimension), dtype=dtype, device=device).T


def allocate_2d_block_cyclic(
    global_shape: Shape2,
    block_size: int,
    process_grid_shape: Grid,
    *,
    dtype: torch.dtype = torch.float32,
    device: torch.device | str | None = None,
) -> torch.Tensor:
    """Zeroed column-major local buffer of the calling rank (``_utils.py:159-189``).

    Shape ``(max(1, local_rows), max(1, local_cols))``, strides ``(1, max(1, local_rows))``;
    a rank that owns nothing gets a 1x1 dummy.  Uses the default process group.
    """
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed must be initialized first.")
    rank = dist.get_rank()
    validate_process_grid(process_grid_shape, dist.get_world_size())
    local_rows, local_columns = local_2d_block_cyclic_shape(
        global_shape, block_size, process_grid_shape, rank
    )
    return empty_2d_block_cyclic_like_shape(local_rows, local_columns, dtype=dtype, device=device)


def iter_2d_block_cyclic_blocks_owned_by_rank(
    num_block_rows: int,
    num_block_cols: int,
    process_grid_shape: Grid,
    rank: int,
) -> Iterator[Tuple[int, int]]:
    process_row, process_column = grid_coords(rank, process_grid_shape)
    process_rows, process_columns = process_grid_shape
    for block_row in range(process_row, num_block_rows, process_rows):
        for block_col in range(process_column, num_block_cols, process_columns):
            yield block_row, block_col


def iter_lower_2d_block_cyclic_blocks_owned_by_rank(
    block_count: int,
    process_grid_shape: Grid,
    rank: int,
) -> Iterator[Tuple[int, int]]:
    for block_row, block_col in iter_2d_block_cyclic_blocks_owned_by_rank(
        block_count, block_count, process_grid_shape, rank
    ):
        if block_row >= block_col:
            yield block_row, block_col


def block_cyclic_tile_views(
    matrix: torch.Tensor,
    global_shape: Shape2,
    block_size: int,
    process_grid_shape: Grid,
    rank: int,
    *,
    mode: Literal["lower", "full"] = "full",
) -> Dict[Tuple[int, int], torch.Tensor]:
    """Views of the global tiles owned by ``rank`` keyed by ``(block_row, block_col)``.

    Mirrors ``_utils.py:192-263``: local tile origin is ``((bi // Pr) * nb, (bj // Pc) * nb)``.
    """
    if mode not in {"lower", "full"}:
        raise ValueError(f"mode must be 'lower' or 'full', got {mode!r}.")
    validate_2d_block_cyclic_buffer("matrix", matrix, global_shape, block_size, process_grid_shape, rank)
    rows, columns = global_shape
    process_rows, process_columns = process_grid_shape
    views: Dict[Tuple[int, int], torch.Tensor] = {}
    for block_row, block_col in iter_2d_block_cyclic_blocks_owned_by_rank(
        num_blocks(rows, block_size), num_blocks(columns, block_size), process_grid_shape, rank
    ):
        if mode == "lower" and block_row < block_col:
            continue
        row_start, row_end = block_bounds(block_row, block_size, rows)
        col_start, col_end = block_bounds(block_col, block_size, columns)
        local_row = (block_row // process_rows) * block_size
        local_col = (block_col // process_columns) * block_size
        views[(block_row, block_col)] = matrix[
            local_row : local_row + row_end - row_start,
            local_col : local_col + col_end - col_start,
        ]
    return views


def most_square_grid(world_size: int) -> Grid:
    """Most-square ``Pr <= Pc`` factorisation, as the reference's timing driver picks it
    (``scripts/run_soap_tp_timing_gpu.py:18-22``)."""
    import math

    process_rows = math.isqrt(world_size)
    while world_size % process_rows:
        process_rows -= 1
    return process_rows, world_size // process_rows


def tp_shard_shape(global_shape: Shape2, shard_dim: int, world_size: int) -> Shape2:
    """Shape of an equal contiguous tensor-parallel shard."""
    if shard_dim not in (0, 1):
        raise ValueError(f"shard_dim must be 0 or 1, got {shard_dim}.")
    rows, columns = global_shape
    sharded = (rows, columns)[shard_dim]
    if sharded % world_size != 0:
        raise ValueError(f"global dimension {shard_dim} must be divisible by the world size.")
    if shard_dim == 0:
        return rows // world_size, columns
    return rows, columns // world_size


__all__ = [
    "allocate_2d_block_cyclic",
    "block_bounds",
    "block_cyclic_indices",
    "block_cyclic_owner_rank",
    "block_cyclic_tile_views",
    "ceil_div",
    "global_to_local",
    "grid_coords",
    "iter_2d_block_cyclic_blocks_owned_by_rank",
    "iter_lower_2d_block_cyclic_blocks_owned_by_rank",
    "local_2d_block_cyclic_shape",
    "most_square_grid",
    "num_blocks",
    "numroc",
    "owned_indices",
    "tp_shard_shape",
    "validate_2d_block_cyclic_buffer",
    "validate_process_grid",
]
