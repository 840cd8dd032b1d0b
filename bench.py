#!/usr/bin/env python3
"""Headline benchmark: ``soap_step`` milliseconds per step on one 8192 x 8192 fp32 parameter.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Configuration (the reference's strong-scaling harness, ``scripts/slurm/frontier/
submit_soap_tp_scaling.sh:56-60`` and ``scripts/run_soap_tp_timing_gpu.py:126-209``, at the
benchmark shape): one 8192 x 8192 fp32 parameter, column shards (``shard_dim=1``), block size 128,
most-square process grid ((1,1), (1,2), (2,2), (2,4)), gradients i.i.d. N(0, 1) * 1e-2 seeded per
step, betas (0.95, 0.95), basis refresh every 10 steps.  STRONG scaling: the parameter is fixed
while N grows.  The first call (basis initialisation) is part of the warm-up.

Two measurements are reported in one JSON line on rank 0:

* ``value``  -- device time of K ``soap_step`` calls whose gradients are resident on the GPU
  (CUDA events, barrier + synchronise on both sides, maximum over ranks) / K;
* ``e2e``    -- the same K calls through the public API where every step first copies its gradient
  shard from pinned host memory to the device and ends with a device-to-host read of the update
  norm (host wall clock around barrier + synchronise, maximum over ranks) / K.

For N > 1 the script expects one process per GPU (``python -m torch.distributed.run
--nproc-per-node N ...``); started without that environment it re-launches itself that way.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
SIZE, BLOCK, SHARD_DIM, REFRESH = 8192, 128, 1, 10
GRAD_SCALE = 1e-2
METRIC = "soap_step ms/step, 8192^2 fp32 (device time, max over ranks; refresh every 10 steps included)"


def parse_args() -> argparse.Namespace:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--size", type=int, default=SIZE, help="matrix size (the metric of record is 8192)")
    parser.add_argument("--block-size", type=int, default=BLOCK)
    parser.add_argument("--shard-dim", type=int, choices=(0, 1), default=SHARD_DIM)
    parser.add_argument("--refresh-interval", type=int, default=REFRESH)
    parser.add_argument("--basis-implementation", default=None)
    parser.add_argument("--stage-timing", action="store_true", help="also print per-stage device times (stderr)")
    args = parser.parse_args()
    if args.warmup < 1:
        parser.error("--warmup must be at least 1 (the first call initialises the bases)")
    return args


class ClockSampler:
    """Samples SM clocks and throttle reasons with ``nvidia-smi`` while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int) -> None:
        self.device_index = device_index
        self.lines: list[str] = []
        self.proc: subprocess.Popen | None = None
        self.thread: threading.Thread | None = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxima, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 8:
                continue
            try:
                clocks.append(float(fields[1]))
                maxima.append(float(fields[2]))
                power.append(float(fields[3]))
            except ValueError:
                continue
            for name, flag in zip(names, fields[4:8]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max(maxima) if maxima else None,
            "power_w_max": max(power) if power else None,
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


def relaunch_under_torchrun(args: argparse.Namespace) -> int:
    import socket

    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), str(Path(__file__).resolve()), *sys.argv[1:]]
    return subprocess.call(command)


def gradient_for(step: int, rank: int, shape, device, generator_cache: dict):
    """Seeded per step (and rank): i.i.d. N(0, 1) * 1e-2."""
    import torch

    generator = generator_cache.setdefault("g", torch.Generator(device=device))
    generator.manual_seed(1_000_003 * step + rank)
    return torch.randn(shape, generator=generator, dtype=torch.float32, device=device) * GRAD_SCALE


def run(args: argparse.Namespace) -> int:
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)

    sys.path.insert(0, str(ROOT))
    from soap_tp_b200.layout import most_square_grid

    size = args.size
    grid = most_square_grid(world)
    if size % world:
        raise SystemExit(f"size {size} must be divisible by {world} ranks")
    shard_shape = (size // world, size) if args.shard_dim == 0 else (size, size // world)

    if args.impl == "reference":
        sys.path.insert(0, str(ROOT / "baseline"))
        import reference_arm

        step_fn, launches, basis = reference_arm.make_step(
            size=size, block_size=args.block_size, shard_dim=args.shard_dim, grid=grid,
            refresh_interval=args.refresh_interval, device=device)
    else:
        from soap_tp_b200 import soap_step
        from soap_tp_b200.engine import kernels

        basis = args.basis_implementation or "jacobi"
        state: dict = {}

        def step_fn(gradient):
            return soap_step(gradient, state, global_shape=(size, size), shard_dim=args.shard_dim,
                             block_size=args.block_size, process_grid_shape=grid,
                             basis_refresh_interval=args.refresh_interval, basis_implementation=basis)

        launches = kernels.total_launches
        if args.stage_timing:
            from soap_tp_b200.profiling import GLOBAL_STAGE_TIMER

            GLOBAL_STAGE_TIMER.enabled = True

    def fence() -> None:
        dist.barrier()
        torch.cuda.synchronize(device)

    cache: dict = {}
    pool = 4  # distinct resident gradients cycled through the timed region
    counter = 0

    # ---- warm-up (first call = basis initialisation) ----
    init_start = time.perf_counter()
    for _ in range(args.warmup):
        step_fn(gradient_for(counter, rank, shard_shape, device, cache))
        counter += 1
        if counter == 1:
            fence()
            init_seconds = time.perf_counter() - init_start
    fence()

    # ---- device-timed region ----
    # The reference arm needs seconds per steady step and minutes per refresh step at the size of record,
    # so it runs ONE loop (the end-to-end one below) and takes both numbers from it: CUDA events around that
    # loop give the device time (the prefetched copy and the 4-byte read-back are under 1 % of its step).
    single_loop = args.impl == "reference"
    budget_seconds = float(os.environ.get("SOAP_TP_REFERENCE_BUDGET_SECONDS", "1200"))
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches_before = launches()
    device_ms = None
    if not single_loop:
        if args.impl == "ours" and args.stage_timing:
            GLOBAL_STAGE_TIMER.reset()
        resident = [gradient_for(counter + i, rank, shard_shape, device, cache) for i in range(pool)]
        fence()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(args.steps):
            step_fn(resident[i % pool])
        stop.record()
        fence()
        device_ms = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device=device)
        dist.all_reduce(device_ms, op=dist.ReduceOp.MAX)
        launches_timed = launches() - launches_before
        if args.impl == "ours" and args.stage_timing:
            stages = GLOBAL_STAGE_TIMER.summary()
            GLOBAL_STAGE_TIMER.enabled = False
            if rank == 0:
                print(json.dumps({"stage_ms_per_step_max_over_ranks":
                                  {n: round(v / args.steps, 3) for n, v in stages.items()}}), file=sys.stderr)
        clocks = sampler.stop() if rank == 0 else {}
        counter += args.steps

    # ---- end-to-end region: pinned host -> device every step, metric back to the host ----
    host_pool = [torch.empty(shard_shape, dtype=torch.float32).pin_memory() for _ in range(pool)]
    for i, buffer in enumerate(host_pool):
        buffer.copy_(gradient_for(counter + i, rank, shard_shape, device, cache))
    # Every step's input crosses PCIe inside the timed region; the copy of step i + 1 is issued on a copy
    # stream while step i computes (two device buffers), as an input pipeline would do it.
    device_buffers = [torch.empty(shard_shape, dtype=torch.float32, device=device) for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=device)
    arrived = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    used = [False, False]
    # the step's metric comes back into pinned memory every step; the host reads it one step later, as a
    # training loop that logs its loss without stalling the device does
    metric_host = torch.empty(2, dtype=torch.float32).pin_memory()
    metric_ready = [torch.cuda.Event() for _ in range(2)]
    metrics_read = []

    def prefetch(index: int) -> None:
        slot = index % 2
        with torch.cuda.stream(copy_stream):
            if used[slot]:
                copy_stream.wait_event(consumed[slot])
            device_buffers[slot].copy_(host_pool[index % pool], non_blocking=True)
            arrived[slot].record(copy_stream)

    fence()
    loop_start, loop_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_start = time.perf_counter()
    loop_start.record()
    prefetch(0)
    steps_done = 0
    for i in range(args.steps):
        slot = i % 2
        if i + 1 < args.steps:
            prefetch(i + 1)
        torch.cuda.current_stream().wait_event(arrived[slot])
        update = step_fn(device_buffers[slot])
        consumed[slot].record()
        used[slot] = True
        metric_host[slot:slot + 1].copy_(torch.linalg.vector_norm(update).reshape(1), non_blocking=True)
        metric_ready[slot].record()
        if i > 0:
            metric_ready[1 - slot].synchronize()
            metrics_read.append(float(metric_host[1 - slot]))
        steps_done += 1
        if single_loop:
            # every rank must take the same decision: agree on the slowest rank's clock
            elapsed = torch.tensor([time.perf_counter() - e2e_start], dtype=torch.float64, device=device)
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
            if float(elapsed.item()) > budget_seconds and steps_done < args.steps:
                break
    loop_stop.record()
    if steps_done:
        metric_ready[(steps_done - 1) % 2].synchronize()
        metrics_read.append(float(metric_host[(steps_done - 1) % 2]))
    fence()
    e2e_ms = torch.tensor([(time.perf_counter() - e2e_start) * 1e3], dtype=torch.float64, device=device)
    dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    if single_loop:
        device_ms = torch.tensor([loop_start.elapsed_time(loop_stop)], dtype=torch.float64, device=device)
        dist.all_reduce(device_ms, op=dist.ReduceOp.MAX)
        launches_timed = launches() - launches_before
        clocks = sampler.stop() if rank == 0 else {}
        if steps_done < args.steps:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable":
                                  f"the unmodified reference did not finish {args.steps} steps within "
                                  f"{budget_seconds:.0f} s at {world} GPU(s): {steps_done} steps took "
                                  f"{float(e2e_ms.item()) / 1e3:.0f} s (refresh steps run Python index planning "
                                  "over every matrix element)"}), flush=True)
            dist.destroy_process_group()
            return 0

    if args.impl == "ours":
        from soap_tp_b200.engine import kernels

        kernels.check_status()
        if args.stage_timing and rank == 0:
            print(json.dumps({"launch_counts": kernels.LAUNCH_COUNTS}), file=sys.stderr)

    ms_per_step = float(device_ms.item()) / args.steps
    e2e_per_step = float(e2e_ms.item()) / args.steps
    shard_bytes = shard_shape[0] * shard_shape[1] * 4
    if rank == 0:
        line = {
            "metric": METRIC,
            "value": round(ms_per_step, 4),
            "unit": "ms/step",
            "impl": args.impl,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": False,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "fp32 state; 3xTF32 tcgen05 products (fp32-class accuracy)" if args.impl == "ours" else "fp32",
            "data": "synthetic: gradients i.i.d. N(0,1)*1e-2 seeded per step; random-init state from the first gradient",
            "config": {
                "model": f"one {size}x{size} fp32 parameter (SOAP-TP state: L, R, Q_L, Q_R, momentum, variance)",
                "global_batch": None,
                "seq_len": None,
                "parallelism": f"tp{world} column shards, 2-D block-cyclic grid {grid[0]}x{grid[1]}, block {args.block_size}",
                "shard_dim": args.shard_dim,
                "basis_refresh_interval": args.refresh_interval,
                "basis_implementation": basis,
                "l2": "no flush: each step streams > 1 GiB of operand planes and state per GPU (L2 is 126 MB); "
                      f"{pool} distinct resident gradients are cycled",
                "initialization_seconds": round(init_seconds, 3),
                "timed_loop": ("one loop: device events around the end-to-end loop" if single_loop
                               else "device loop on resident gradients, then a separate end-to-end loop"),
            },
            "clocks": clocks,
            "e2e": {
                "value": round(e2e_per_step, 4),
                "unit": "ms/step",
                "h2d_bytes_per_step": shard_bytes,
                "d2h_bytes_per_step": 4,
            },
            "gpu_launches": int(launches_timed),
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()
    return 0


def main() -> int:
    args = parse_args()
    if args.impl == "reference" and not (ROOT / "baseline" / "_ref" / "soap_tp").exists():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed "
                          "(python -m pip install --no-index --no-build-isolation --target baseline/_ref "
                          "<checkout of the reference>)"}), flush=True)
        return 0
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        return relaunch_under_torchrun(args)
    return run(args)


if __name__ == "__main__":
    raise SystemExit(main())
