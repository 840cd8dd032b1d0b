#!/usr/bin/env python3
"""Accuracy sweep: ``soap_step`` against the dense single-process oracle over a range of sizes.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m soap_tp_b200.bench.accuracy --sizes 8 16 64 256 1024 --steps 10 --rtol 1e-5

Counterpart of the reference's ``scripts/run_soap_accuracy_gpu.py`` (sizes x basis implementations,
block = ``min(size / max(grid), cap)`` as in ``:17-25`` there, failures collected and the sweep
continues, ``:231-261``).  Rank 0 runs the dense oracle, prints one accuracy line per step in the
format ``utils/plot_accuracy.py`` parses, and additionally prints the oracle's own sensitivity to a
1e-6 relative perturbation of the gradients (the conditioning floor any fp32 implementation is
subject to), so a "failure" against a flat ``--rtol`` can be told apart from a real defect.
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

from .. import soap_step
from ..layout import most_square_grid
from ..utils.dense_soap import DenseSOAP, relative_l2


def parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--sizes", type=int, nargs="+", default=[8, 16, 32, 64, 128, 256, 512, 1024])
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--rtol", type=float, default=1e-5)
    parser.add_argument("--block-cap", type=int, default=128)
    parser.add_argument("--basis-implementations", nargs="+", default=["householder"])
    parser.add_argument("--basis-refresh-interval", type=int, default=2)
    parser.add_argument("--shard-dims", type=int, nargs="+", default=[0, 1])
    parser.add_argument("--device", choices=("cuda", "cpu"), default="cuda")
    parser.add_argument("--seed", type=int, default=0)
    return parser.parse_args(argv)


def run_one(args, size: int, shard_dim: int, implementation: str, device) -> list:
    rank, world = dist.get_rank(), dist.get_world_size()
    grid = most_square_grid(world)
    block = max(1, min(size // max(grid), args.block_cap))
    shape = (size, size)
    hyper = dict(beta1=0.8, beta2=0.9, preconditioner_beta=0.75, eps=1e-6, basis_refresh_interval=args.basis_refresh_interval)
    oracle, shadow = (DenseSOAP(shape, **hyper), DenseSOAP(shape, **hyper)) if rank == 0 else (None, None)
    state: dict = {}
    failures = []
    for step in range(args.steps):
        generator = torch.Generator().manual_seed(args.seed * 7919 + step)
        G = torch.randn(shape, generator=generator) * 2.0
        shard = G.chunk(world, dim=shard_dim)[rank].contiguous().to(device)
        update = soap_step(shard, state, global_shape=shape, shard_dim=shard_dim, block_size=block, process_grid_shape=grid,
                           preconditioner_beta=0.75, beta1=0.8, beta2=0.9, eps=1e-6,
                           basis_refresh_interval=args.basis_refresh_interval, basis_implementation=implementation)
        parts = [torch.empty_like(update) for _ in range(world)]
        dist.all_gather(parts, update.contiguous())
        full = torch.cat(parts, dim=shard_dim).cpu()
        if rank == 0:
            expected = oracle.step(G)
            perturbed = shadow.step(G * (1.0 + 1e-6 * torch.randn(shape, generator=generator)))
            if step == 0:
                continue
            error, floor = relative_l2(full, expected), relative_l2(perturbed, expected)
            print(f"{size}x{size} dim{shard_dim} basis={implementation} | step {step} | SOAP relL2={error:.2e} "
                  f"(floor={floor:.2e}) | PARAM relL2={error:.2e}", flush=True)
            if error > max(args.rtol, 3.0 * floor):
                failures.append((size, shard_dim, implementation, step, error, floor))
    return failures


def main(argv=None) -> int:
    args = parse_args(argv)
    created = False
    if not dist.is_initialized():
        rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29543")
        if args.device == "cuda":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl" if args.device == "cuda" else "gloo", rank=rank, world_size=world)
        created = True
    device = torch.device("cuda", torch.cuda.current_device()) if args.device == "cuda" else torch.device("cpu")
    failures = []
    try:
        for size in args.sizes:
            if size % dist.get_world_size():
                continue
            for implementation in args.basis_implementations:
                for shard_dim in args.shard_dims:
                    try:
                        failures += run_one(args, size, shard_dim, implementation, device)
                    except Exception as error:  # keep sweeping, as the reference's sweep does
                        failures.append((size, shard_dim, implementation, "exception", repr(error), None))
        if dist.get_rank() == 0:
            print(f"accuracy sweep finished with {len(failures)} entries above max(rtol, 3 x floor): {failures}", flush=True)
    finally:
        if created:
            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
