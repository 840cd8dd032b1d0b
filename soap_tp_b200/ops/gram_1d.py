"""Gram updates with 1-D row-sharded results (the reference's pre-block-cyclic entry points).

The reference keeps two functions from before its 2-D block-cyclic layout
(``src/soap_tp/ops/preconditioners.py:22-115`` and ``:118-245``); they are not exported from its
``ops`` namespace and have no tests there, but they are part of the module and documented:

* ``update_left_preconditioner_from_col_shards(G_local, L_prev, beta, TP_group=None)``:
  ``G`` is split by columns; rank ``r`` of ``p`` receives rows ``[r m/p, (r+1) m/p)`` of
  ``beta L + (1 - beta) G G^T`` as a row-major ``[m/p, m]`` tensor (the reference: local
  ``G_r G_r^T`` + ``reduce_scatter_tensor``).
* ``update_right_preconditioner_from_col_shards(G_local, R_prev, beta, TP_group=None)``:
  rank ``r`` receives the block row of ``G^T G`` of its own columns, ``[n_local, p n_local]``
  (the reference: ring pass of the shards with double-buffered sends overlapped with GEMMs).

Here both are one gather + one GEMM.  On CUDA every rank publishes its shard in a symmetric
segment, pulls the operand panel it needs with ``dist_gather_kernel`` (peer loads over NVLink,
hi/lo split fused) and runs one 3xTF32 tcgen05 GEMM whose epilogue applies the EMA; the row-major
result is addressed as the column-major transpose, so no transposition pass is needed.  On CPU
tensors the shards are all-gathered and the block row is computed with torch.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
from torch import Tensor

from . import _hostpath as host


def _group_info(TP_group):
    if TP_group is None and not (dist.is_available() and dist.is_initialized()):
        raise ValueError("TP_group is None and the default process group has not been initialized.")
    group = TP_group if TP_group is not None else dist.group.WORLD
    return group, dist.get_rank(group), dist.get_world_size(group)


def _check_inputs(G_local: Tensor, previous: Optional[Tensor], expected_shape, beta: float, name: str) -> Tensor:
    if G_local.ndim != 2:
        raise ValueError(f"G_local must be 2D, got {G_local.ndim}D.")
    if not 0.0 <= beta <= 1.0:
        raise ValueError(f"beta must be in [0, 1], got {beta}.")
    if previous is None:
        return torch.zeros(expected_shape, dtype=G_local.dtype, device=G_local.device)
    if tuple(previous.shape) != tuple(expected_shape):
        raise ValueError(f"{name} must have shape {tuple(expected_shape)}, got {tuple(previous.shape)}.")
    if previous.device != G_local.device:
        raise ValueError(f"{name} is on {previous.device}, expected {G_local.device}.")
    return previous


def _on_engine(G_local: Tensor, previous: Tensor, group) -> bool:
    """The native path needs fp32 row-major state and the whole world as the group."""
    return (G_local.is_cuda and previous.dtype == torch.float32 and previous.is_contiguous()
            and dist.get_world_size(group) == dist.get_world_size())


@torch.no_grad()
def update_left_preconditioner_from_col_shards(G_local: Tensor, L_prev: Optional[Tensor], beta: float, *,
                                               TP_group=None) -> Tensor:
    """Row shard ``r`` of ``beta * L_prev + (1 - beta) * G @ G.T`` for column-sharded ``G``."""
    group, rank, world = _group_info(TP_group)
    m = G_local.shape[0]
    if m % world != 0:
        raise RuntimeError(f"the row count {m} must be divisible by the group size {world}.")
    rows_here = m // world
    L = _check_inputs(G_local, L_prev, (rows_here, m), beta, "L_prev")
    if world > 1 and _on_engine(G_local, L, group):
        from ..engine import distributed as engine

        engine.gram_rows_from_col_shards(G_local, L, beta, side="left")
        return L
    full = host.gather_tp_shards(G_local.contiguous(), 1, group=group) if world > 1 else G_local
    full = full.to(torch.float32)
    block = full[rank * rows_here:(rank + 1) * rows_here] @ full.T
    L.lerp_(block.to(L.dtype), 1.0 - beta)
    return L


@torch.no_grad()
def update_right_preconditioner_from_col_shards(G_local: Tensor, R_prev: Optional[Tensor], beta: float, *,
                                                TP_group=None) -> Tensor:
    """Block row of ``beta * R_prev + (1 - beta) * G.T @ G`` that belongs to this rank's columns."""
    group, rank, world = _group_info(TP_group)
    n_local = G_local.shape[1]
    R = _check_inputs(G_local, R_prev, (n_local, world * n_local), beta, "R_prev")
    if world > 1 and _on_engine(G_local, R, group):
        from ..engine import distributed as engine

        engine.gram_rows_from_col_shards(G_local, R, beta, side="right")
        return R
    if world > 1:
        full = host.gather_tp_shards(G_local.contiguous(), 1, group=group)
        if full.shape[1] != world * n_local:
            raise RuntimeError("every rank must hold the same number of columns.")
    else:
        full = G_local
    full = full.to(torch.float32)
    block = full[:, rank * n_local:(rank + 1) * n_local].T @ full
    R.lerp_(block.to(R.dtype), 1.0 - beta)
    return R


__all__ = ["update_left_preconditioner_from_col_shards", "update_right_preconditioner_from_col_shards"]
