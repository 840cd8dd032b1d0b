#!/usr/bin/env python3
"""Rewrite ``SoapTP`` checkpoints for another process grid or block size (offline, CPU).

    python -m soap_tp_b200.utils.regrid --inputs 'ckpt/optim_rank{rank}.pt' --old-world 8 \
        --new-grid 4 2 --new-block-size 256 --outputs 'ckpt_4x2/optim_rank{rank}.pt'

Packed 2-D block-cyclic state (``left_preconditioner`` ... ``variance``, the layout of
``src/soap_tp/ops/_utils.py:268-304`` in the reference) is only valid for the grid and block size it was written
with, and ``SoapTP.load_state_dict`` refuses anything else.  The reference has no conversion tool: a job that changes
its grid has to start its optimizer state again.  This one reads every rank's ``state_dict`` file (``torch.save`` of
``SoapTP.state_dict()``), reassembles each packed matrix densely on the host, and writes one file per NEW rank.

* Packed two-sided SOAP entries are converted for any new grid (the new world size is ``Pr * Pc``).
* Every other entry (AdamW moments, one-sided SOAP state) is a function of this rank's parameter shard; it is carried
  over unchanged when the world size stays the same and otherwise needs the model's own resharding, so the tool
  stops with the list of such entries unless ``--drop-other-state`` is given (those parameters then restart their
  optimizer state).
"""
from __future__ import annotations

import argparse
import copy
from typing import Any, Dict, List, Sequence, Tuple

import torch
from torch import Tensor

from ..layout import empty_2d_block_cyclic_like_shape, grid_coords, numroc, owned_indices
from ..step import state_shapes

Grid = Tuple[int, int]


def unpack_dense(parts: Sequence[Tensor], shape: Tuple[int, int], block_size: int, grid: Grid) -> Tensor:
    """Dense ``shape`` matrix from the packed local buffers of all ``Pr * Pc`` ranks (row-major rank order)."""
    dense = torch.empty(shape, dtype=parts[0].dtype)
    for rank, local in enumerate(parts):
        pr, pc = grid_coords(rank, grid)
        rows, cols = owned_indices(shape[0], block_size, pr, grid[0]), owned_indices(shape[1], block_size, pc, grid[1])
        expected = (max(1, numroc(shape[0], block_size, pr, grid[0])), max(1, numroc(shape[1], block_size, pc, grid[1])))
        if tuple(local.shape) != expected:        # a rank that owns nothing holds a 1 x 1 dummy
            raise ValueError(f"rank {rank}: packed buffer {tuple(local.shape)} does not belong to a {shape} matrix on grid "
                             f"{grid} with block size {block_size}.")
        if len(rows) and len(cols):
            dense[rows[:, None], cols] = local.cpu()[: len(rows), : len(cols)]
    return dense


def pack_dense(dense: Tensor, block_size: int, grid: Grid) -> List[Tensor]:
    """Packed column-major local buffers of every rank of ``grid``."""
    parts = []
    for rank in range(grid[0] * grid[1]):
        pr, pc = grid_coords(rank, grid)
        rows, cols = owned_indices(dense.shape[0], block_size, pr, grid[0]), owned_indices(dense.shape[1], block_size, pc, grid[1])
        local = empty_2d_block_cyclic_like_shape(len(rows), len(cols), dtype=dense.dtype)
        if len(rows) and len(cols):
            local[: len(rows), : len(cols)] = dense[rows[:, None], cols]
        parts.append(local)
    return parts


def regrid_state_dicts(state_dicts: Sequence[Dict[str, Any]], new_grid: Grid, new_block_size: int | None = None,
                       drop_other_state: bool = False) -> List[Dict[str, Any]]:
    """``SoapTP.state_dict()`` of every old rank -> ``state_dict`` of every rank of ``new_grid``."""
    old_world, new_world = len(state_dicts), new_grid[0] * new_grid[1]
    layouts = state_dicts[0].get("soap_tp_layout", {})
    for rank, sd in enumerate(state_dicts):
        if sd.get("soap_tp_layout", {}) != layouts:
            raise ValueError(f"rank {rank} was written with another layout header than rank 0.")
    template = 0 if new_world != old_world else None
    results = []
    for rank in range(new_world):
        source = state_dicts[rank if template is None else template]
        results.append({"state": {}, "param_groups": copy.deepcopy(source["param_groups"]), "soap_tp_layout": {}})
    others = []
    for index, entry in state_dicts[0]["state"].items():
        layout = layouts.get(index, layouts.get(str(index)))
        if layout is None or "left_basis" not in entry:
            if new_world == old_world:
                for rank in range(new_world):
                    results[rank]["state"][index] = state_dicts[rank]["state"][index]
            else:
                others.append(index)
            continue
        shape, old_nb, old_grid = tuple(layout["global_shape"]), int(layout["block_size"]), tuple(layout["grid"])
        if old_grid[0] * old_grid[1] != old_world:
            raise ValueError(f"parameter {index}: layout grid {old_grid} does not match the {old_world} input files.")
        nb = int(new_block_size or old_nb)
        new_entries: List[Dict[str, Any]] = [dict(step=int(entry["step"])) for _ in range(new_world)]
        for name, matrix_shape in state_shapes(shape).items():
            dense = unpack_dense([sd["state"][index][name] for sd in state_dicts], matrix_shape, old_nb, old_grid)
            for rank, local in enumerate(pack_dense(dense, nb, new_grid)):
                new_entries[rank][name] = local
        for rank in range(new_world):
            results[rank]["state"][index] = new_entries[rank]
            results[rank]["soap_tp_layout"][index] = dict(global_shape=list(shape), shard_dim=layout["shard_dim"],
                                                          block_size=nb, grid=list(new_grid))
    if others and not drop_other_state:
        raise ValueError(f"parameters {others} carry per-shard state (AdamW moments or one-sided SOAP); with a new world "
                         "size they follow the model's own resharding.  Pass drop_other_state=True to restart them.")
    if new_block_size is not None:
        for result in results:
            for group in result["param_groups"]:
                if "block_size" in group:
                    group["block_size"] = int(new_block_size)
    return results


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--inputs", required=True, help="path pattern with {rank}")
    parser.add_argument("--old-world", type=int, required=True)
    parser.add_argument("--new-grid", type=int, nargs=2, required=True, metavar=("PR", "PC"))
    parser.add_argument("--new-block-size", type=int, default=None)
    parser.add_argument("--outputs", required=True, help="path pattern with {rank}")
    parser.add_argument("--drop-other-state", action="store_true")
    args = parser.parse_args(argv)
    state_dicts = [torch.load(args.inputs.format(rank=rank), map_location="cpu", weights_only=False)
                   for rank in range(args.old_world)]
    converted = regrid_state_dicts(state_dicts, tuple(args.new_grid), args.new_block_size, args.drop_other_state)
    for rank, result in enumerate(converted):
        torch.save(result, args.outputs.format(rank=rank))
    print(f"wrote {len(converted)} files for grid {tuple(args.new_grid)}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
