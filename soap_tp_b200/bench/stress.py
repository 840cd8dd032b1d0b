#!/usr/bin/env python3
"""Basis initialisation and refresh on one large, well-conditioned Gram matrix.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m soap_tp_b200.bench.stress --size 16384

The matrix is ``P = A A^T / n + 1e-3 I`` with ``A`` an ``n x 2n`` matrix of i.i.d. N(0, 1) entries (seeded), packed
on the most square grid of the launched ranks with block size 128.  Timed on the device (CUDA events, maximum over
ranks) and checked against the defining properties:

* ``initialize_basis_2d_block_cyclic_`` with every requested eigensolver (``householder``, ``jacobi``): largest
  ``|Q^T Q - I|`` and largest ``|P Q - Q diag(values)|`` relative to the largest eigenvalue;
* one ``refresh_bases_and_transport_optimizer_state_`` (power iteration, Householder QR, momentum transport, variance
  permutation) on a square parameter of the same side: orthogonality of the refreshed bases.

The reference runs the same operations through ELPA and SLATE (``src/soap_tp/ops/factorizations.py:363-614``); it has
no stress driver of its own.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .. import ops
from ..layout import allocate_2d_block_cyclic, grid_coords, most_square_grid, owned_indices
from .checks import gather_dense


def timed(fn, device) -> float:
    dist.barrier()
    torch.cuda.synchronize(device)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    fn()
    stop.record()
    torch.cuda.synchronize(device)
    elapsed = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device=device)
    dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    return float(elapsed)


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--size", type=int, default=16384)
    parser.add_argument("--block-size", type=int, default=128)
    parser.add_argument("--implementations", nargs="+", default=["householder", "jacobi"])
    parser.add_argument("--seed", type=int, default=0)
    args = parser.parse_args(argv)
    created = False
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29547")
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl", rank=int(os.environ.get("RANK", "0")), world_size=int(os.environ.get("WORLD_SIZE", "1")))
        created = True
    rank, world = dist.get_rank(), dist.get_world_size()
    device = torch.device("cuda", torch.cuda.current_device())
    n, nb = args.size, args.block_size
    grid = most_square_grid(world)
    pr, pc = grid_coords(rank, grid)
    ri, ci = owned_indices(n, nb, pr, grid[0], device), owned_indices(n, nb, pc, grid[1], device)
    generator = torch.Generator(device=device).manual_seed(args.seed)
    A = torch.randn(n, 2 * n, generator=generator, device=device)
    # this rank's block of P = A A^T / n + 1e-3 I (library GEMM: set-up, not a product path)
    block = A[ri] @ A[ci].T / n
    block += 1e-3 * (ri[:, None] == ci[None, :])
    del A
    P = allocate_2d_block_cyclic((n, n), nb, grid, device=device)
    P[: len(ri), : len(ci)] = block
    report = {"size": n, "ranks": world, "grid": list(grid), "block_size": nb}
    for name in args.implementations:
        Q, work = (allocate_2d_block_cyclic((n, n), nb, grid, device=device) for _ in range(2))
        values = torch.empty(n, dtype=torch.float32, device=device)
        run = lambda: ops.initialize_basis_2d_block_cyclic_(P, Q, work, values, n, nb, grid, implementation=name)
        run()                                                       # first call: workspaces, module loading
        milliseconds = timed(run, device)
        dense_q = gather_dense(Q, (n, n), nb, grid)
        dense_p = gather_dense(P, (n, n), nb, grid)
        torch.backends.cuda.matmul.allow_tf32 = False
        gram = dense_q.T @ dense_q
        gram.diagonal().sub_(1.0)
        residual = dense_p @ dense_q - dense_q * values
        report[name] = {"milliseconds": round(milliseconds, 1), "max_abs_QtQ_minus_I": float(gram.abs().max()),
                        "max_abs_residual_over_largest_eigenvalue": float(residual.abs().max() / values.abs().max())}
        del dense_p, gram, residual
        if name == args.implementations[0]:
            basis = Q
    # one refresh on a square parameter whose two preconditioners are P: bases = the eigenbasis just computed
    momentum = allocate_2d_block_cyclic((n, n), nb, grid, device=device).normal_(generator=generator)
    variance = allocate_2d_block_cyclic((n, n), nb, grid, device=device).uniform_(generator=generator)
    left_q, right_q = basis.clone(), basis.clone()
    works = [allocate_2d_block_cyclic((n, n), nb, grid, device=device) for _ in range(2)]
    refresh = lambda: ops.refresh_bases_and_transport_optimizer_state_(momentum, variance, P, P.clone(), left_q, right_q,
                                                                        works[0], works[1], (n, n), nb, grid)
    refresh()
    milliseconds = timed(refresh, device)
    dense_q = gather_dense(left_q, (n, n), nb, grid)
    gram = dense_q.T @ dense_q
    gram.diagonal().sub_(1.0)
    report["refresh"] = {"milliseconds": round(milliseconds, 1), "max_abs_QtQ_minus_I": float(gram.abs().max())}
    from ..engine import kernels

    kernels.check_status()
    if rank == 0:
        print(json.dumps(report), flush=True)
    if created:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
