"""``soap_step``: one SOAP update for one tensor-parallel-sharded 2-D parameter.

Behavioural contract of the reference's ``soap_step`` (``src/soap_tp/soap.py:123-506``):

* ``state`` is a plain mutable mapping filled lazily with eight packed fp32 buffers
  (``left_preconditioner, right_preconditioner, left_basis, right_basis, left_work, right_work,
  momentum, variance``; ``soap.py:165-182``) and the integer ``step``;
* the first call seeds ``L`` and ``R`` from the gradient, computes both eigenbases, sets
  ``state["step"] = 0`` and returns exact zeros (``soap.py:193-276``);
* later calls rotate the gradient into the eigenbasis, run Adam there with
  ``eps / sqrt(1 - beta2**step)`` (``soap.py:360-368``), rotate back, return the fp32 update
  shaped like the shard, THEN update ``L`` and ``R`` with the current gradient and, every
  ``basis_refresh_interval`` steps, refresh the bases (``soap.py:425-471``);
* learning rate, weight decay and the parameter update belong to the caller.

CPU tensors run the composable ops one after another.  CUDA tensors run the fused device
pipeline of :mod:`soap_tp_b200.engine`: the redistribution is folded into the rotation's panel
gather, Adam is the epilogue of the forward rotation's second GEMM, and the backward rotation's
epilogue writes the tensor-parallel shard directly.
"""
from __future__ import annotations

import math
from typing import Any, Literal, MutableMapping

import torch
from torch import Tensor

from .ops import (
    adam_update,
    allocate_2d_block_cyclic,
    initialize_basis_2d_block_cyclic_,
    redistribute_2d_block_cyclic_to_tp_shard,
    redistribute_tp_shard_to_2d_block_cyclic,
    refresh_bases_and_transport_optimizer_state_,
    rotate_2d_block_cyclic_,
    update_left_preconditioner_2d_block_cyclic_,
    update_right_preconditioner_2d_block_cyclic_,
)
from .ops.basis import BASIS_IMPLEMENTATIONS
from .parallel.guard import check_collective
from .profiling import GLOBAL_STAGE_TIMER, profile_block_cyclic, profile_enabled, profile_tp_shard

STATE_BUFFER_NAMES = (
    "left_preconditioner",
    "right_preconditioner",
    "left_basis",
    "right_basis",
    "left_work",
    "right_work",
    "momentum",
    "variance",
)


def state_shapes(global_shape) -> dict:
    rows, columns = global_shape
    return {
        "left_preconditioner": (rows, rows),
        "right_preconditioner": (columns, columns),
        "left_basis": (rows, rows),
        "right_basis": (columns, columns),
        "left_work": (rows, rows),
        "right_work": (columns, columns),
        "momentum": (rows, columns),
        "variance": (rows, columns),
    }


def _tap_state(names, step, state, global_shape, block_size, grid, suffix="") -> None:
    shapes = state_shapes(global_shape)
    for name in names:
        profile_block_cyclic(name + suffix, step, state[name], shapes[name], block_size, grid)


@torch.no_grad()
def soap_step(
    gradient_shard: Tensor,
    state: MutableMapping[str, Any],
    *,
    global_shape: tuple[int, int],
    shard_dim: Literal[0, 1],
    block_size: int,
    process_grid_shape: tuple[int, int],
    preconditioner_beta: float = 0.95,
    beta1: float = 0.95,
    beta2: float = 0.95,
    eps: float = 1e-8,
    basis_refresh_interval: int = 10,
    basis_implementation: str = "elpa",
    elpa_binding: Any | None = None,
    slate_binding: Any | None = None,
) -> Tensor:
    """Run one SOAP update for a row- (``shard_dim=0``) or column- (``shard_dim=1``) sharded gradient.

    Returns a new fp32 tensor shaped like ``gradient_shard``.  ``slate_binding`` / ``elpa_binding``: objects with
    the reference's native entry points (``soap_tp_b200.bindings`` has this package's own); when given, the step
    is composed from the public ops and every rotation, ``P Q`` product, QR and (for ``"elpa"``) eigensolve goes
    through the injected object, as in the reference (``src/soap_tp/soap.py:139-141``).
    """
    if basis_refresh_interval <= 0:
        raise ValueError("basis_refresh_interval must be positive.")
    if basis_implementation not in BASIS_IMPLEMENTATIONS:
        raise ValueError(
            f"basis_implementation must be one of {BASIS_IMPLEMENTATIONS}, got "
            f"{basis_implementation!r}."
        )
    rows, columns = global_shape
    grid = process_grid_shape
    initializing = "left_basis" not in state
    check_collective("soap_step", tuple(global_shape), shard_dim, block_size, tuple(grid), basis_refresh_interval,
                     basis_implementation, initializing, -1 if initializing else int(state["step"]))
    device = gradient_shard.device
    timer = GLOBAL_STAGE_TIMER

    if initializing:
        for name, shape in state_shapes(global_shape).items():
            state[name] = allocate_2d_block_cyclic(shape, block_size, grid, device=device)

    profile_step = 0 if initializing else int(state["step"]) + 1
    tracing = profile_enabled(profile_step)

    injected = slate_binding is not None or elpa_binding is not None
    if device.type == "cuda" and not tracing and not injected:
        from .engine import api as engine

        return engine.soap_step(
            gradient_shard,
            state,
            global_shape=global_shape,
            shard_dim=shard_dim,
            block_size=block_size,
            grid=grid,
            preconditioner_beta=preconditioner_beta,
            beta1=beta1,
            beta2=beta2,
            eps=eps,
            basis_refresh_interval=basis_refresh_interval,
            basis_implementation=basis_implementation,
            initializing=initializing,
        )

    gradient_float = gradient_shard.detach().to(torch.float32).contiguous()
    profile_tp_shard("gradient", profile_step, gradient_float, shard_dim)

    if initializing:
        with timer.stage("gram_left", device):
            update_left_preconditioner_2d_block_cyclic_(
                gradient_float, state["left_preconditioner"], preconditioner_beta, block_size, grid,
                shard_dim=shard_dim,
            )
        _tap_state(["left_preconditioner"], profile_step, state, global_shape, block_size, grid)
        with timer.stage("gram_right", device):
            update_right_preconditioner_2d_block_cyclic_(
                gradient_float, state["right_preconditioner"], preconditioner_beta, block_size, grid,
                shard_dim=shard_dim,
            )
        _tap_state(["right_preconditioner"], profile_step, state, global_shape, block_size, grid)
        with timer.stage("basis_init", device):
            initialize_basis_2d_block_cyclic_(
                state["left_preconditioner"], state["left_basis"], state["left_work"],
                torch.empty(rows, dtype=torch.float32, device=device),
                rows, block_size, grid, implementation=basis_implementation, elpa_binding=elpa_binding,
            )
        _tap_state(["left_basis"], profile_step, state, global_shape, block_size, grid)
        with timer.stage("basis_init", device):
            initialize_basis_2d_block_cyclic_(
                state["right_preconditioner"], state["right_basis"], state["right_work"],
                torch.empty(columns, dtype=torch.float32, device=device),
                columns, block_size, grid, implementation=basis_implementation, elpa_binding=elpa_binding,
            )
        _tap_state(["right_basis"], profile_step, state, global_shape, block_size, grid)
        state["step"] = 0
        zero_update = torch.zeros_like(gradient_float)
        profile_tp_shard("returned_update", profile_step, zero_update, shard_dim)
        return zero_update

    step = int(state["step"]) + 1
    _tap_state(
        ["left_preconditioner", "right_preconditioner", "left_basis", "right_basis"],
        profile_step, state, global_shape, block_size, grid,
    )
    _tap_state(["momentum", "variance"], profile_step, state, global_shape, block_size, grid, "_before_adam")

    with timer.stage("redistribute_in", device):
        packed = redistribute_tp_shard_to_2d_block_cyclic(
            gradient_float, global_shape, block_size, grid, shard_dim=shard_dim
        )
    profile_block_cyclic("gradient_2d", profile_step, packed, global_shape, block_size, grid)
    with timer.stage("rotate_forward", device):
        rotate_2d_block_cyclic_(
            packed, state["left_basis"], state["right_basis"], global_shape, block_size, grid,
            direction="forward", slate_binding=slate_binding,
        )
    profile_block_cyclic("projected_gradient", profile_step, packed, global_shape, block_size, grid)
    with timer.stage("adam", device):
        packed_update = adam_update(
            packed, state["momentum"], state["variance"], step, beta1, beta2,
            eps / math.sqrt(1.0 - beta2**step),
        )
    _tap_state(["momentum", "variance"], profile_step, state, global_shape, block_size, grid, "_after_adam")
    profile_block_cyclic("coordinate_update", profile_step, packed_update, global_shape, block_size, grid)
    with timer.stage("rotate_backward", device):
        rotate_2d_block_cyclic_(
            packed_update, state["left_basis"], state["right_basis"], global_shape, block_size, grid,
            direction="backward", slate_binding=slate_binding,
        )
    profile_block_cyclic("backrotated_update", profile_step, packed_update, global_shape, block_size, grid)
    with timer.stage("redistribute_out", device):
        update_shard = redistribute_2d_block_cyclic_to_tp_shard(
            packed_update, global_shape, block_size, grid, shard_dim=shard_dim
        )
    profile_tp_shard("returned_update", profile_step, update_shard, shard_dim)

    with timer.stage("gram_left", device):
        update_left_preconditioner_2d_block_cyclic_(
            gradient_float, state["left_preconditioner"], preconditioner_beta, block_size, grid,
            shard_dim=shard_dim,
        )
    _tap_state(["left_preconditioner"], profile_step, state, global_shape, block_size, grid, "_after_step")
    with timer.stage("gram_right", device):
        update_right_preconditioner_2d_block_cyclic_(
            gradient_float, state["right_preconditioner"], preconditioner_beta, block_size, grid,
            shard_dim=shard_dim,
        )
    _tap_state(["right_preconditioner"], profile_step, state, global_shape, block_size, grid, "_after_step")
    if step % basis_refresh_interval == 0:
        with timer.stage("refresh", device):
            refresh_bases_and_transport_optimizer_state_(
                state["momentum"], state["variance"],
                state["left_preconditioner"], state["right_preconditioner"],
                state["left_basis"], state["right_basis"],
                state["left_work"], state["right_work"],
                global_shape, block_size, grid, slate_binding=slate_binding,
            )
    _tap_state(["left_basis", "right_basis", "momentum", "variance"], profile_step, state, global_shape, block_size, grid, "_after_step")
    state["step"] = step
    return update_shard


__all__ = ["STATE_BUFFER_NAMES", "soap_step", "state_shapes"]
