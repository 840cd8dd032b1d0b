#!/usr/bin/env python3
"""Time ``soap_step`` on one GPU per rank and print the ``SOAP_TIMING`` event stream.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m soap_tp_b200.bench.timing --size 8192 --block-size 128 --shard-dim 1 --steps 100

Counterpart of the reference's ``scripts/run_soap_tp_timing_gpu.py`` with the same command-line
options (``--size --world-size --steps --block-size --shard-dim --basis-implementation
--basis-refresh-interval --seed``, ``:39-69`` there) and the same event stream
(``configuration`` / ``initialization`` / ``step`` / ``summary``, ``:167-209``), with two changes:
ranks come from ``torchrun`` (no MPI), and each step is timed ON THE DEVICE with CUDA events and
reduced with MAX over ranks (the reference wraps a host clock around two host synchronisations).
``--sweep`` runs the rectangular shape / shard-dimension / block-size sweep; ``--stage-timing``
adds per-stage device times.
"""
from __future__ import annotations

import argparse
import os
import statistics

import torch
import torch.distributed as dist

from .. import soap_step
from ..layout import most_square_grid
from ..profiling import GLOBAL_STAGE_TIMER, emit_timing


def parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--size", type=int, default=8192)
    parser.add_argument("--rows", type=int, default=None, help="rectangular parameter: rows (default --size)")
    parser.add_argument("--cols", type=int, default=None, help="rectangular parameter: columns (default --size)")
    parser.add_argument("--world-size", type=int, default=None, help="checked against the launcher's world size")
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--block-size", type=int, default=128)
    parser.add_argument("--shard-dim", type=int, choices=(0, 1), default=0)
    parser.add_argument("--basis-implementation", default="householder")
    parser.add_argument("--basis-refresh-interval", type=int, default=10)
    parser.add_argument("--seed", type=int, default=42)
    parser.add_argument("--device", choices=("cuda", "cpu"), default="cuda")
    parser.add_argument("--sweep", action="store_true", help="4096x16384 and 16384x4096, both shard dims, blocks 64/128/256")
    parser.add_argument("--stage-timing", action="store_true")
    args = parser.parse_args(argv)
    for name in ("size", "steps", "block_size", "basis_refresh_interval"):
        if getattr(args, name) <= 0:
            parser.error(f"--{name.replace('_', '-')} must be positive")
    return args


def run_case(args, rows: int, cols: int, shard_dim: int, block_size: int, device: torch.device) -> dict:
    rank, world = dist.get_rank(), dist.get_world_size()
    grid = most_square_grid(world)
    if (rows, cols)[shard_dim] % world:
        raise ValueError(f"dimension {shard_dim} of {rows}x{cols} must be divisible by {world} ranks")
    local_shape = (rows // world, cols) if shard_dim == 0 else (rows, cols // world)
    generator = torch.Generator(device=device).manual_seed(args.seed + rank)
    gradient = torch.normal(0.0, 2.0, size=local_shape, generator=generator, dtype=torch.float32, device=device)
    state: dict = {}
    cuda = device.type == "cuda"

    def timed_step() -> float:
        dist.barrier()
        if cuda:
            torch.cuda.synchronize(device)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        else:
            import time

            begin = time.perf_counter()
        soap_step(gradient, state, global_shape=(rows, cols), shard_dim=shard_dim, block_size=block_size,
                  process_grid_shape=grid, basis_refresh_interval=args.basis_refresh_interval,
                  basis_implementation=args.basis_implementation)
        if cuda:
            stop.record()
            torch.cuda.synchronize(device)
            seconds = start.elapsed_time(stop) / 1e3
        else:
            seconds = time.perf_counter() - begin
        elapsed = torch.tensor([seconds], dtype=torch.float64, device=device)
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        return float(elapsed.item())

    emit_timing("configuration", timer="device_events_max_over_ranks" if cuda else "host_clock_max_over_ranks",
                matrix_size=rows if rows == cols else [rows, cols], ranks=world, process_grid=list(grid),
                local_shape=list(local_shape), block_size=block_size, shard_dim=shard_dim,
                basis_implementation=args.basis_implementation, basis_refresh_interval=args.basis_refresh_interval,
                measured_steps=args.steps, tensor_profile=False, slurm_job_id=os.environ.get("SLURM_JOB_ID"))
    GLOBAL_STAGE_TIMER.enabled = bool(args.stage_timing)
    GLOBAL_STAGE_TIMER.reset()
    initialization = timed_step()
    emit_timing("initialization", step=0, seconds=initialization)
    seconds = []
    for step in range(1, args.steps + 1):
        seconds.append(timed_step())
        emit_timing("step", step=step, seconds=seconds[-1])
    summary = dict(matrix_size=rows if rows == cols else [rows, cols], ranks=world, initialization_seconds=initialization,
                   measured_steps=args.steps, seconds_per_step=statistics.mean(seconds),
                   median_seconds_per_step=statistics.median(seconds), min_seconds_per_step=min(seconds),
                   max_seconds_per_step=max(seconds))
    if args.stage_timing:
        summary["stage_milliseconds"] = GLOBAL_STAGE_TIMER.summary()
    emit_timing("summary", **summary)
    return summary


def main(argv=None) -> int:
    args = parse_args(argv)
    created = False
    if not dist.is_initialized():
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        if args.device == "cuda":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl" if args.device == "cuda" else "gloo", rank=rank, world_size=world)
        created = True
    if args.world_size is not None and args.world_size != dist.get_world_size():
        raise RuntimeError(f"expected {args.world_size} ranks, got {dist.get_world_size()}")
    device = torch.device("cuda", torch.cuda.current_device()) if args.device == "cuda" else torch.device("cpu")
    try:
        if args.sweep:
            for rows, cols in ((4096, 16384), (16384, 4096)):
                for shard_dim in (0, 1):
                    for block in (64, 128, 256):
                        run_case(args, rows, cols, shard_dim, block, device)
        else:
            run_case(args, args.rows or args.size, args.cols or args.size, args.shard_dim, args.block_size, device)
    finally:
        if created:
            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
