"""Two-sided basis rotation of a packed block-cyclic matrix.

``forward`` computes ``Q_left.T @ X @ Q_right`` and ``backward`` ``Q_left @ X @ Q_right.T``, in
place on ``X`` -- the contract of the reference's ``rotate_2d_block_cyclic_``
(``src/soap_tp/ops/factorizations.py:104-184``), which marshals raw pointers into two SLATE
GEMMs with a freshly allocated intermediate (``src/soap_tp/csrc/slate_bindings.cpp:191-277``)
and brackets the call with two host synchronisations.

On CUDA both GEMMs are stationary-C products on tcgen05 tensor cores with 3xTF32 error
compensation: each rank pulls the operand panels it needs from its peers' packed buffers
(peer loads, fused with the hi/lo split), multiplies locally, and the second GEMM's epilogue
writes the packed result.  Nothing synchronises with the host.
"""
from __future__ import annotations

from typing import Any, Literal, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from ..layout import validate_2d_block_cyclic_buffer, validate_process_grid
from . import _hostpath as host
from ..parallel.guard import check_collective


def validate_world(process_grid_shape: Tuple[int, int]) -> Tuple[int, int]:
    host.require_dist()
    rank, world_size = dist.get_rank(), dist.get_world_size()
    validate_process_grid(process_grid_shape, world_size)
    return rank, world_size


def validate_float_buffer(name: str, matrix: Tensor, global_shape, block_size: int, grid, rank: int):
    if matrix.dtype != torch.float32:
        raise ValueError(f"{name} must use float32, got {matrix.dtype}.")
    return validate_2d_block_cyclic_buffer(name, matrix, global_shape, block_size, grid, rank)


@torch.no_grad()
def _synchronize(device: torch.device) -> None:
    """An injected binding works on raw pointers outside torch's stream ordering."""
    if device.type == "cuda":
        torch.cuda.synchronize(device)


def rotate_2d_block_cyclic_(
    matrix: Tensor,
    Q_left: Tensor,
    Q_right: Tensor,
    global_shape: Tuple[int, int],
    block_size: int,
    process_grid_shape: Tuple[int, int],
    *,
    direction: Literal["forward", "backward"],
    slate_binding: Optional[Any] = None,
) -> Tensor:
    """Rotate a packed matrix in place and return it.

    ``slate_binding``: an object with the reference's ``slate_forward_rotation_float`` /
    ``slate_backward_rotation_float`` entry points; when given it is called (pointer-level convention of
    ``src/soap_tp/ops/factorizations.py:162-182``) instead of the built-in path.
    """
    check_collective("rotate_2d_block_cyclic_", tuple(global_shape), block_size, tuple(process_grid_shape), direction)
    if direction not in {"forward", "backward"}:
        raise ValueError(f"direction must be 'forward' or 'backward', got {direction!r}.")
    rank, _ = validate_world(process_grid_shape)
    rows, columns = global_shape
    validate_float_buffer("matrix", matrix, global_shape, block_size, process_grid_shape, rank)
    validate_float_buffer("Q_left", Q_left, (rows, rows), block_size, process_grid_shape, rank)
    validate_float_buffer("Q_right", Q_right, (columns, columns), block_size, process_grid_shape, rank)
    if len({matrix.device, Q_left.device, Q_right.device}) != 1:
        raise ValueError("matrix and bases must share a device.")
    if len({matrix.data_ptr(), Q_left.data_ptr(), Q_right.data_ptr()}) != 3:
        raise ValueError("matrix and basis buffers must not overlap.")
    if slate_binding is not None:
        function = (slate_binding.slate_forward_rotation_float if direction == "forward"
                    else slate_binding.slate_backward_rotation_float)
        _synchronize(matrix.device)
        function(Q_left.data_ptr(), matrix.data_ptr(), Q_right.data_ptr(), rows, columns, Q_left.stride(1),
                 matrix.stride(1), Q_right.stride(1), block_size, process_grid_shape[0], process_grid_shape[1])
        _synchronize(matrix.device)
        return matrix
    if matrix.is_cuda:
        from ..engine import api as engine

        return engine.rotate(matrix, Q_left, Q_right, global_shape, block_size, process_grid_shape, direction)
    grid = process_grid_shape
    X = host.gather_block_cyclic(matrix, global_shape, block_size, grid)
    QL = host.gather_block_cyclic(Q_left, (rows, rows), block_size, grid)
    QR = host.gather_block_cyclic(Q_right, (columns, columns), block_size, grid)
    Y = QL.T @ X @ QR if direction == "forward" else QL @ X @ QR.T
    return host.store_block_cyclic_(matrix, Y, global_shape, block_size, grid)


__all__ = ["rotate_2d_block_cyclic_", "validate_float_buffer", "validate_world", "_synchronize"]
