"""Correctness figures of a benchmark run, computed after (never inside) the timed region.

The headline benchmark drives one 8192 x 8192 parameter; nothing in the timing loop looks at the values it
produces.  These helpers do, on the state the loop leaves behind, at any rank count:

* ``basis_orthogonality``: ``max |Q^T Q - I|`` of a packed basis (all-gathered, one fp32 library GEMM --
  a check, not a product path);
* ``gram_error``: relative Frobenius error of a packed preconditioner against a float64 EMA of the same
  gradient sequence, every rank comparing the block it owns;
* ``side_problem_against_one_gpu``: a short ``soap_step`` trajectory of a smaller square parameter on the
  run's own grid against this package's single-GPU pipeline fed with the gathered gradient.

The reference has no counterpart: its timing driver (``scripts/run_soap_tp_timing_gpu.py``) checks nothing and
its accuracy driver (``scripts/run_soap_accuracy_gpu.py:138-282``) is a separate run at other sizes.
"""
from __future__ import annotations

from typing import Callable, Dict, List, MutableMapping, Sequence, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from ..layout import grid_coords, numroc, owned_indices


def _owned(size: int, block: int, grid, rank: int, device) -> Tuple[Tensor, Tensor]:
    """Global row and column indices of the block of a ``size x size`` matrix that ``rank`` owns."""
    pr, pc = grid_coords(rank, grid)
    return owned_indices(size, block, pr, grid[0], device), owned_indices(size, block, pc, grid[1], device)


def gather_dense(packed: Tensor, shape, block: int, grid) -> Tensor:
    """The dense ``shape`` matrix behind a packed block-cyclic buffer, on every rank's device."""
    world, rank = dist.get_world_size(), dist.get_rank()
    rows, cols = shape
    device = packed.device
    if world == 1:
        return packed[:rows, :cols].clone()
    most = (max(1, numroc(rows, block, 0, grid[0])), max(1, numroc(cols, block, 0, grid[1])))
    mine = torch.zeros(most, dtype=torch.float32, device=device)
    pr, pc = grid_coords(rank, grid)
    lr, lc = numroc(rows, block, pr, grid[0]), numroc(cols, block, pc, grid[1])
    if lr and lc:
        mine[:lr, :lc] = packed[:lr, :lc]
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    dense = torch.empty((rows, cols), dtype=torch.float32, device=device)
    for r, part in enumerate(parts):
        r_row, r_col = grid_coords(r, grid)
        ri = owned_indices(rows, block, r_row, grid[0], device)
        ci = owned_indices(cols, block, r_col, grid[1], device)
        if len(ri) and len(ci):
            dense[ri[:, None], ci] = part[: len(ri), : len(ci)]
    return dense


def basis_orthogonality(packed: Tensor, size: int, block: int, grid) -> float:
    dense = gather_dense(packed, (size, size), block, grid)
    previous = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        gram = dense.T @ dense
    finally:
        torch.backends.cuda.matmul.allow_tf32 = previous
    gram.diagonal().sub_(1.0)
    return float(gram.abs().max())


def gram_error(state: MutableMapping, gradients: Callable[[int], Tensor], history: Sequence[int], shape, block: int, grid,
               beta: float) -> Dict[str, float]:
    """``history`` lists, call by call, the index handed to ``gradients(index) -> full fp32 gradient`` (this
    rank's device).  Returns the relative Frobenius errors of ``L`` and ``R`` over all ranks' blocks."""
    rank = dist.get_rank()
    rows, cols = shape
    device = state["left_preconditioner"].device
    left = torch.zeros((rows, rows), dtype=torch.float64, device=device)
    right = torch.zeros((cols, cols), dtype=torch.float64, device=device)
    cache: Dict[int, Tuple[Tensor, Tensor]] = {}
    for index in history:
        if index not in cache:
            if len(cache) >= 2:
                cache.pop(next(iter(cache)))
            g = gradients(index).double()
            cache[index] = (g @ g.T, g.T @ g)
        ggt, gtg = cache[index]
        left.mul_(beta).add_(ggt, alpha=1.0 - beta)
        right.mul_(beta).add_(gtg, alpha=1.0 - beta)
    result = {}
    for name, expected, size in (("left", left, rows), ("right", right, cols)):
        ri, ci = _owned(size, block, grid, rank, device)
        sums = torch.zeros(2, dtype=torch.float64, device=device)
        if len(ri) and len(ci):
            want = expected[ri[:, None], ci]
            got = state[f"{name}_preconditioner"][: len(ri), : len(ci)].double()
            sums[0], sums[1] = (got - want).square().sum(), want.square().sum()
        if dist.get_world_size() > 1:
            dist.all_reduce(sums)
        result[name] = float((sums[0] / sums[1]).sqrt())
    return result


def side_problem_against_one_gpu(step_fn_factory: Callable[[], Callable[[Tensor], Tensor]], size: int, block: int, grid,
                                 shard_dim: int, steps: int, interval: int, scale: float = 1e-2,
                                 implementation: str = "householder", state: MutableMapping = None) -> Dict[str, float]:
    """Run ``steps`` calls on a ``size x size`` parameter through the distributed path (``step_fn_factory()``
    returns a fresh ``step(shard) -> update shard``) and, on every rank, through the single-GPU pipeline with
    the full gradient; report the worst relative L2 distance of the updates and the step it occurred at."""
    from ..engine import local
    from ..layout import empty_2d_block_cyclic_like_shape
    from ..step import state_shapes

    world, rank = dist.get_world_size(), dist.get_rank()
    device = torch.device("cuda", torch.cuda.current_device())
    step_fn = step_fn_factory()
    shape = (size, size)
    single: dict = {}
    worst, worst_step = 0.0, -1
    per_step: List[float] = []
    generator = torch.Generator(device=device)
    for index in range(steps):
        generator.manual_seed(77_000 + index)
        full = torch.randn(shape, generator=generator, device=device) * scale
        shard = full.chunk(world, dim=shard_dim)[rank].contiguous()
        update = step_fn(shard)
        parts = [torch.empty_like(update) for _ in range(world)]
        dist.all_gather(parts, update.contiguous())
        gathered = torch.cat(parts, dim=shard_dim)
        initializing = "left_basis" not in single
        if initializing:
            for name, buffer_shape in state_shapes(shape).items():
                single[name] = empty_2d_block_cyclic_like_shape(*buffer_shape, device=device, zero=True)
        expected = local.soap_step(full, single, global_shape=shape, beta=0.95, beta1=0.95, beta2=0.95, eps=1e-8,
                                   interval=interval, implementation=implementation, initializing=initializing)
        if index == 0:
            continue
        distance = float((gathered - expected).norm() / expected.norm())
        per_step.append(distance)
        if distance > worst:
            worst, worst_step = distance, index
    result = {"worst_relative_l2": worst, "at_step": worst_step, "steps": steps, "size": size,
              "per_step": [float(f"{d:.3e}") for d in per_step]}
    if state is not None:
        # the preconditioners are rounding-level functions of the gradients; the bases after a refresh carry the
        # conditioning of the QR factor (a perturbation of relative size eps moves Q by about eps * cond(P Q))
        for name in ("left_preconditioner", "right_preconditioner", "left_basis"):
            dense = gather_dense(state[name], shape, block, grid)
            reference = single[name][:size, :size]
            if name == "left_basis":
                signs = torch.sign((dense * reference).sum(dim=0))
                dense = dense * torch.where(signs == 0, torch.ones_like(signs), signs)
            result[name + "_relative_difference"] = float((dense - reference).norm() / reference.norm())
    return result
