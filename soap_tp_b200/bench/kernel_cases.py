#!/usr/bin/env python3
"""Run ONE kernel-level case a few times: the unit that gets profiled.

    python -m soap_tp_b200.bench.kernel_cases gemm --size 4096 [--mode store|split|adam|ema]
    python -m soap_tp_b200.bench.kernel_cases qr --size 4096
    python -m soap_tp_b200.bench.kernel_cases panel --rows 4096
    python -m soap_tp_b200.bench.kernel_cases update --size 4096      # QR trailing update (K = 128, planes RMW)
    python -m soap_tp_b200.bench.kernel_cases adam --size 8192
    python -m soap_tp_b200.bench.kernel_cases split --size 8192
    python -m soap_tp_b200.bench.kernel_cases eig --size 4096 [--solver householder|jacobi]
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m soap_tp_b200.bench.kernel_cases \
        gather --size 8192                                          # peer pull, traffic mix of an 8-GPU (2, 4) grid

Each case allocates a few hundred MB at most, launches the kernel ``--repeats`` times and prints
the CUDA-event time per launch, so the same command line serves for timing and, under ``ncu -k
regex:<kernel> -c 1``, for a bounded profile capture.
"""
from __future__ import annotations

import argparse

import torch


def timed(fn, repeats: int) -> float:
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(repeats):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / repeats * 1e3


def gather_case(args) -> int:
    """Time ``dist_gather_kernel`` on the three pulls of a steady step as rank 0 of an 8-rank (2, 4) grid sees
    them: one eighth of the source is local, seven eighths sit in a peer GPU's memory.  Needs two ranks (two
    GPUs); each holds the seven remote shards its partner reads.  Prints microseconds and GB/s of source bytes
    for the 16-byte kernels and for the element-wise kernel."""
    import os

    import torch.distributed as dist

    from ..engine import kernels as k
    from ..parallel.comm import get_communicator

    n, nb, virtual, Pr, Pc = args.size, 128, 8, 2, 4
    shard = n * n // virtual
    single = "WORLD_SIZE" not in os.environ or int(os.environ["WORLD_SIZE"]) == 1
    if single:
        # one process, one GPU: all eight "ranks" are slices of one local buffer (what an ncu capture can run;
        # the figures then are those of the kernel against local HBM, not against NVLink)
        device = torch.device("cuda", torch.cuda.current_device())
        rank, comm = 0, None
        buffer = torch.randn(virtual * shard, device=device)
        table = torch.tensor([buffer.data_ptr() + 4 * v * shard for v in range(virtual)], dtype=torch.int64, device=device)
    else:
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
        dist.init_process_group("nccl", device_id=device)
        if dist.get_world_size() != 2:
            raise SystemExit("the gather case needs one rank (local memory) or exactly two ranks")
        rank = dist.get_rank()
        comm = get_communicator(device)
        segment = comm.segment("gather_case", virtual * shard)
        segment.local.normal_()
        comm.barrier()
        # virtual rank 0's data is mine, virtual ranks 1..7 live in the partner's segment
        partner = segment.peer_ptrs[1 - rank]
        table = torch.tensor([segment.peer_ptrs[rank]] + [partner + 4 * v * shard for v in range(1, virtual)],
                             dtype=torch.int64, device=device)
    planes = k.Planes.empty(n, n // Pr, device)
    stream = lambda: torch.cuda.current_stream().cuda_stream

    def pull(kind, cols_out, jP, transpose):
        k._C.dist_gather(table.data_ptr(), kind, n, n, nb, nb, Pr, Pc, virtual, 0, 1, 1, 0, 0, 0, jP, nb, 0, 0,
                         int(transpose), 0, 0, 0, planes.hi.data_ptr(), planes.lo.data_ptr(), 1, planes.ld, n, cols_out,
                         stream())

    cases = [("gradient panel from column shards (turn)", 2, n // Pr, Pr, False),
             ("intermediate from packed blocks (copy)", 0, n // Pr, Pr, False),
             ("Gram operand from column shards, transposed (copy)", 2, n // Pc, Pc, True)]
    for name, kind, cols_out, jP, transpose in cases:
        for scalar in (False, True):
            k._C.force_scalar_gather(scalar)
            us = timed(lambda: pull(kind, cols_out, jP, transpose), args.repeats)
            best = torch.tensor([us], device=device)
            if not single:
                dist.all_reduce(best, op=dist.ReduceOp.MAX)
            if rank == 0:
                bytes_read = 4.0 * n * cols_out
                print(f"{name}: {'element-wise' if scalar else '16-byte'} {float(best):.1f} us, "
                      f"{bytes_read / float(best) / 1e3:.0f} GB/s of source bytes ({bytes_read * 7 / 8 / float(best) / 1e3:.0f} "
                      f"GB/s over NVLink), {3 * bytes_read / float(best) / 1e6:.2f} TB/s of local traffic incl. both planes")
        k._C.force_scalar_gather(False)
    k.check_status()
    if not single:
        comm.barrier()
        dist.destroy_process_group()
    return 0


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("case", choices=("gemm", "qr", "qrpair", "panel", "update", "adam", "split", "gather", "eig"))
    parser.add_argument("--solver", choices=("householder", "jacobi"), default="householder", help="eig: which eigensolver")
    parser.add_argument("--size", type=int, default=4096)
    parser.add_argument("--rows", type=int, default=4096)
    parser.add_argument("--mode", default="store")
    parser.add_argument("--repeats", type=int, default=3)
    parser.add_argument("--pairs", action="store_true", help="panel: the two-columns-per-exchange kernel")
    parser.add_argument("--rows-per-cta", type=int, default=256, choices=(128, 256), help="panel --pairs: CTA height")
    parser.add_argument("--mixed", action="store_true", help="gemm: operands as mixed planes (bf16 correction products)")
    parser.add_argument("--trace", action="store_true",
                        help="panel: print clock64 stamps of one column step (needs a library built with SOAP_QR_TRACE=1)")
    args = parser.parse_args(argv)

    from ..engine import kernels as k
    from ..engine import qr

    if args.case == "gather":
        return gather_case(args)
    n = args.size
    device = torch.device("cuda", torch.cuda.current_device())
    generator = torch.Generator(device=device).manual_seed(0)
    rand = lambda *shape: torch.randn(*shape, generator=generator, device=device)
    if args.case == "gemm":
        a, b = k.split_planes(rand(n, n), mixed=args.mixed), k.split_planes(rand(n, n), mixed=args.mixed)
        out = torch.zeros(n, n, device=device).T
        if args.mode == "store":
            fn = lambda: k.gemm(a, b, out=out)
        elif args.mode == "ema":
            fn = lambda: k.gemm(a, a, out=out, alpha=0.05, beta=0.95, symmetric=True)
        elif args.mode == "split":
            planes = k.Planes.empty(n, n, device, mixed=args.mixed)
            fn = lambda: k.gemm(a, b, mode=k.EPI_SPLIT, out_planes=planes)
        else:
            planes = k.Planes.empty(n, n, device, mixed=args.mixed)
            momentum, variance = torch.zeros(n, n, device=device).T, torch.zeros(n, n, device=device).T
            adam = dict(beta1=0.95, beta2=0.95, eps=1e-8, bias_correction1=0.5, bias_correction2=0.5)
            fn = lambda: k.gemm(a, b, mode=k.EPI_ADAM, out_planes=planes, momentum=momentum, variance=variance, adam=adam)
        us = timed(fn, args.repeats)
        form = "tf32 + 2 bf16 corrections" if args.mixed else "3 tf32 MMAs"
        print(f"gemm_tf32x3 {args.mode} {n}^3 ({form}): {us:.1f} us/launch, {2 * n**3 / us / 1e6:.1f} TFLOP/s fp32-equivalent "
              f"({(4 if args.mixed else 6) * n**3 / us / 1e6:.1f} TFLOP/s in tf32-MMA units)")
    elif args.case == "qr":
        matrix, Q = rand(n, n).T, torch.empty(n, n, device=device).T
        us = timed(lambda: qr.householder_qr(matrix.clone(), Q), args.repeats)
        print(f"householder_qr {n}: {us / 1e3:.2f} ms")
    elif args.case == "qrpair":
        jobs = [(rand(n, n).T, torch.empty(n, n, device=device).T, None) for _ in range(2)]
        us = timed(lambda: qr.householder_qr_pair(jobs), args.repeats)
        print(f"householder_qr_pair 2 x {n}: {us / 1e3:.2f} ms")
    elif args.case in ("panel", "update"):
        ws = qr._workspace(max(n, args.rows), device)
        k.split_planes(rand(max(n, args.rows), max(n, args.rows)), out=ws["C"])
        if args.case == "panel":
            r = args.rows
            panel, v, vt, T, Tt = ws["C"].sub(0, 0, r, 128), ws["V"].sub(0, 0, r, 128), ws["Vt"][0], ws["T"][0], ws["Tt"][0]
            kernel = k._C.qr_panel_pairs if args.pairs else k._C.qr_panel
            extra = (args.rows_per_cta,) if args.pairs else ()
            fn = lambda: kernel(panel.hi.data_ptr(), panel.lo.data_ptr(), panel.ld, r, 128, v.hi.data_ptr(),
                                v.lo.data_ptr(), v.ld, vt.hi.data_ptr(), vt.lo.data_ptr(), vt.ld,
                                ws["tau"].data_ptr(), T.hi.data_ptr(), T.lo.data_ptr(), Tt.hi.data_ptr(),
                                Tt.lo.data_ptr(), T.ld, ws["exchange"].data_ptr(),
                                k.status_word(device).data_ptr(), k._stream(), *extra)
            label = f"qr_panel_pairs ({args.rows_per_cta}-row CTAs)" if args.pairs else "qr_panel"
            print(f"{label} rows={r}: {timed(fn, args.repeats):.1f} us/launch")
            if args.pairs:
                steps = torch.zeros(1, dtype=torch.int64, device=device)
                kernel(panel.hi.data_ptr(), panel.lo.data_ptr(), panel.ld, r, 128, v.hi.data_ptr(), v.lo.data_ptr(), v.ld,
                       vt.hi.data_ptr(), vt.lo.data_ptr(), vt.ld, ws["tau"].data_ptr(), T.hi.data_ptr(), T.lo.data_ptr(),
                       Tt.hi.data_ptr(), Tt.lo.data_ptr(), T.ld, ws["exchange"].data_ptr(),
                       k.status_word(device).data_ptr(), k._stream(), args.rows_per_cta, steps.data_ptr())
                print(f"exchange steps for 128 columns: {int(steps.item())}")
            if args.trace:
                # stamps taken by thread 0 of CTA 0 around column 64 (see the kernel); differences in SM cycles
                stamps = torch.zeros(16, dtype=torch.int64, device=device)
                k._C.qr_panel(panel.hi.data_ptr(), panel.lo.data_ptr(), panel.ld, r, 128, v.hi.data_ptr(),
                              v.lo.data_ptr(), v.ld, vt.hi.data_ptr(), vt.lo.data_ptr(), vt.ld, ws["tau"].data_ptr(),
                              T.hi.data_ptr(), T.lo.data_ptr(), Tt.hi.data_ptr(), Tt.lo.data_ptr(), T.ld,
                              ws["exchange"].data_ptr(), k.status_word(device).data_ptr(), k._stream(),
                              stamps.data_ptr(), 0)
                torch.cuda.synchronize()
                s = stamps.tolist()
                order = [5, 7, 8, 1, 2, 3, 6, 0, 4]
                names = ["loop top", "sweep 1 FMAs", "shuffles", "pivot row + publish", "T column (CTA 0)",
                         "exchange", "barrier 1", "scalars + sweep 2 + barrier 2"]
                print(f"column 64 of CTA 0: {s[4] - s[5]} cycles")
                for a, b, name in zip(order[:-1], order[1:], names):
                    print(f"  {name:32s} {s[b] - s[a]}")
        else:
            k.split_planes(rand(n, n), out=ws["V"])
            z, w = ws["V"].sub(0, 0, 128, n), ws["V"].sub(128, 0, 128, n - 128)
            trailing = ws["C"].sub(0, 128, n, n - 128)
            fn = lambda: k.gemm(z, w, mode=k.EPI_SPLIT, out_planes=trailing, alpha=-1.0, beta=1.0)
            us = timed(fn, args.repeats)
            print(f"trailing update {n} x {n - 128}, K=128: {us:.1f} us/launch, "
                  f"{n * (n - 128) * 16 / us / 1e6:.2f} TB/s of plane traffic")
    elif args.case == "eig":
        from ..engine import jacobi, tridiag

        G = rand(n, n) * 1e-2
        P = (0.05 * (G.double() @ G.double().T)).float().T.contiguous().T      # a Gram matrix, as at initialisation
        Q, values, work = torch.empty(n, n, device=device).T, torch.empty(n, device=device), torch.empty(n, n, device=device).T
        solver = tridiag if args.solver == "householder" else jacobi
        us = timed(lambda: solver.symmetric_eigenbasis(P, Q, work, values), max(1, args.repeats - 2))
        residual = float((P @ Q - Q * values).abs().max() / values.abs().max())
        print(f"symmetric eigensolver ({args.solver}) {n}: {us / 1e3:.1f} ms, largest |P Q - Q diag| / largest eigenvalue {residual:.2e}")
    elif args.case == "adam":
        g, m, v = (torch.rand(n, n, device=device).T for _ in range(3))
        us = timed(lambda: k.adam_update(g, m, v, 0.9, 0.99, 1e-8, 0.5, 0.5), args.repeats)
        print(f"adam {n}^2: {us:.1f} us/launch, {n * n * 24 / us / 1e6:.2f} TB/s")
    else:
        source, planes = rand(n, n), k.Planes.empty(n, n, device)
        us = timed(lambda: k.split_planes(source, out=planes, transpose=True), args.repeats)
        print(f"split_planes (transposing) {n}^2: {us:.1f} us/launch, {n * n * 12 / us / 1e6:.2f} TB/s")
    k.check_status()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
